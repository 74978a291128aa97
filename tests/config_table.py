"""One line per BASELINE config with three numbers measured in the same run on the same box: this library's kernel
(CUDA events), the reference project's own CUDA kernel where one of its kernels can express the config (compiled for
sm_100a into oracle/_ref), and the CPU golden restatement on the host cores (bounded sample). Not collected by pytest.

    python tests/config_table.py [--launches 30] [--cpu-seconds 4]

Sizes are the configs' own except where stated in the line (`images`): config 5 runs 64 of its 1024 4K images per
launch (the reference kernel's 32-bit offsets stop at 2 GiB per call = 86 images), config 3 runs 64 of 128.
"""
import argparse
import json
import os
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402
from oracle import oracle as O  # noqa: E402
from oracle import ref_cuda  # noqa: E402

MEAN = (123.675, 116.28, 103.53)
INV_STD = tuple(float(np.float32(1.0) / np.float32(s)) for s in (58.395, 57.12, 57.375))


def gpu_us(fn, launches):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches * 1000.0


def cpu_images_per_s(images, spec, dtype, threads, seconds, **kw):
    """CPU golden restatement on `threads` host threads over the given sample, repeated for about `seconds`."""
    O.resize_crop(images[:1], spec, dtype, True, nthreads=threads, **{k: (v[:1] if v is not None else None) for k, v in kw.items()})
    done, t0 = 0, time.perf_counter()
    while True:
        O.resize_crop(images, spec, dtype, True, nthreads=threads, **kw)
        done += len(images)
        dt = time.perf_counter() - t0
        if dt >= seconds:
            return done / dt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--launches", type=int, default=30)
    ap.add_argument("--cpu-seconds", type=float, default=4.0)
    a = ap.parse_args()
    pkg = ge.load_package()
    have_ref = ref_cuda.lib() is not None
    threads = os.cpu_count() or 1
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    rows = []

    def emit(name, images, new_us, ref_us, ref_note, cpu_rate, cpu_sample):
        rows.append({"config": name, "images": images, "new_us_per_launch": round(new_us, 1),
                     "new_images_per_s": round(images / new_us * 1e6),
                     "reference_cuda_us_per_launch": None if ref_us is None else round(ref_us, 1),
                     "reference_cuda_images_per_s": None if ref_us is None else round(images / ref_us * 1e6),
                     "reference_cuda_note": ref_note, "cpu_golden_images_per_s": round(cpu_rate, 1),
                     "cpu_threads": threads, "cpu_sample": cpu_sample})
        print(json.dumps(rows[-1]), flush=True)

    # ---- config 1: 4 x 480x640 -> 256 -> 224, BGR, x/255, f32 NCHW (L2 resident; a latency, not a bandwidth, figure)
    n = 4
    src = torch.randint(0, 256, (n, 480, 640, 3), dtype=torch.uint8, device="cuda", generator=g)
    out = torch.empty((n, 3, 224, 224), dtype=torch.float32, device="cuda")
    ref = torch.empty_like(out)
    t_new = gpu_us(lambda: pkg.resize_crop_convert_reformat_into(out, src, (256, 256), 1, (16, 16), layout="NCHW", manip=1,
                                                                 scale=1 / 255.0, srcCast=False), a.launches)
    t_ref = gpu_us(lambda: ref_cuda.rccr_tensor(src, ref, True, (256, 256), 1, (16, 16), 1, 1 / 255.0, 0.0, False),
                   a.launches) if have_ref else None
    spec = O.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=O.LINEAR, src_cast=False, manip=1,
                        scale=1 / 255.0, offset=0.0)
    host = list(src.cpu().numpy())
    emit("1: 4 x 480x640 -> 256^2 -> 224^2 linear, BGR, x/255, f32 NCHW", n, t_new, t_ref, "identical work",
         cpu_images_per_s(host, spec, np.float32, threads, a.cpu_seconds), "all 4 images per pass")

    # ---- config 2
    n = 256
    src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g)
    out = torch.empty((n, 3, 224, 224), dtype=torch.float32, device="cuda")
    ref = torch.empty_like(out)
    t_new = gpu_us(lambda: pkg.fused_preprocess_into(out, src, resize_dim=(256, 256), interp=1, crop_pos=(16, 16),
                                                     layout="NCHW", base=MEAN, mul=INV_STD, srcCast=False), a.launches)
    t_ref = gpu_us(lambda: ref_cuda.rccr_tensor(src, ref, True, (256, 256), 1, (16, 16), 0, INV_STD[0],
                                                -MEAN[0] * INV_STD[0], False), a.launches) if have_ref else None
    spec = O.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=O.LINEAR, src_cast=False, base=MEAN,
                        mul=INV_STD)
    k = min(n, max(32, 2 * threads))
    host = list(src[:k].cpu().numpy())
    emit("2: 256 x 1080p -> 256^2 -> 224^2 linear, mean/std, f32 NCHW", n, t_new, t_ref,
         "scalar constants; the Normalize pass the reference still needs is not included",
         cpu_images_per_s(host, spec, np.float32, threads, a.cpu_seconds), f"{k} of 256 images per pass")

    # ---- config 4: letterbox
    n = 64
    out = torch.empty((n, 3, 640, 640), dtype=torch.float32, device="cuda")
    s4 = src[:n]
    t_new = gpu_us(lambda: pkg.fused_preprocess_into(out, s4, resize_dim=(640, 360), interp=1, layout="NCHW", manip=1,
                                                     scale=1 / 255.0, srcCast=True, dst_pos=(0, 140), region_size=(640, 360),
                                                     pad_value=114.0), a.launches)
    ref4 = torch.empty((n, 3, 360, 640), dtype=torch.float32, device="cuda")
    t_ref = gpu_us(lambda: ref_cuda.rccr_tensor(s4, ref4, True, (640, 360), 1, (0, 0), 1, 1 / 255.0, 0.0, True),
                   a.launches) if have_ref else None
    spec = O.ResizeSpec(resize=(640, 360), crop=(0, 0), out_size=(640, 360), interp=O.LINEAR, src_cast=True, manip=1,
                        scale=1 / 255.0, offset=0.0, canvas=(640, 640), dst_pos=(0, 140), pad_value=114.0)
    k = min(n, max(16, threads))
    host = list(s4[:k].cpu().numpy())
    emit("4: 64 x 1080p -> 640x360 linear in a 640^2 canvas, pad 114, BGR, x/255, f32 NCHW", n, t_new, t_ref,
         "resized 640x360 region only: the reference needs CopyMakeBorder for the canvas",
         cpu_images_per_s(host, spec, np.float32, threads, a.cpu_seconds), f"{k} of 64 images per pass")
    # ---- configs 2 and 4 as chains of this library's own stand-alone operators (the shape of the reference's unfused
    # pipelines: Resize -> [CopyMakeBorder] -> Normalize / ConvertTo -> Reformat), against the fused call above. The
    # chains round to uint8 after the resize, so their values differ from the fused result; this is a timing line.
    def chain_line(name, images, stages, fused_us):
        times = {k: round(gpu_us(fn, a.launches), 1) for k, fn in stages}
        line = {"config": name, "images": images, "stage_us": times, "chain_us_per_launch": round(sum(times.values()), 1),
                "fused_us_per_launch": round(fused_us, 1), "launches_in_chain": len(stages)}
        line["fused_speedup"] = round(line["chain_us_per_launch"] / fused_us, 2)
        print(json.dumps(line), flush=True)

    n2 = 256
    small = torch.empty((n2, 256, 256, 3), dtype=torch.uint8, device="cuda")
    normed = torch.empty((n2, 224, 224, 3), dtype=torch.float32, device="cuda")
    planar = torch.empty((n2, 3, 224, 224), dtype=torch.float32, device="cuda")
    mean_t = torch.tensor(MEAN, dtype=torch.float32, device="cuda").reshape(1, 1, 1, 3)
    mul_t = torch.tensor(INV_STD, dtype=torch.float32, device="cuda").reshape(1, 1, 1, 3)
    fused2 = gpu_us(lambda: pkg.fused_preprocess_into(planar, src, resize_dim=(256, 256), interp=1, crop_pos=(16, 16),
                                                      layout="NCHW", base=MEAN, mul=INV_STD, srcCast=False), a.launches)
    chain_line("2 as a chain: Resize 256^2 u8 -> (crop view) Normalize -> f32 -> Reformat NCHW", n2,
               [("resize", lambda: pkg.resize_into(small, src, 1)),
                ("normalize", lambda: pkg.normalize_into(normed, small[:, 16:240, 16:240], mean_t, mul_t)),
                ("reformat", lambda: pkg.reformat_into(planar, normed, src_layout="NHWC", dst_layout="NCHW"))], fused2)
    del small, normed, planar

    n4 = 64
    s4 = src[:n4]
    r4 = torch.empty((n4, 360, 640, 3), dtype=torch.uint8, device="cuda")
    b4 = torch.empty((n4, 640, 640, 3), dtype=torch.uint8, device="cuda")
    f4 = torch.empty((n4, 640, 640, 3), dtype=torch.float32, device="cuda")
    p4 = torch.empty((n4, 3, 640, 640), dtype=torch.float32, device="cuda")
    fused4 = gpu_us(lambda: pkg.fused_preprocess_into(p4, s4, resize_dim=(640, 360), interp=1, layout="NCHW", manip=1,
                                                      scale=1 / 255.0, srcCast=True, dst_pos=(0, 140), region_size=(640, 360),
                                                      pad_value=114.0), a.launches)
    chain_line("4 as a chain: Resize 640x360 u8 -> CopyMakeBorder 640^2 (114) -> ConvertTo f32 x1/255 -> Reformat NCHW "
               "(no channel swap in the chain)", n4,
               [("resize", lambda: pkg.resize_into(r4, s4, 1)),
                ("copymakeborder", lambda: pkg.copymakeborder_into(b4, r4, 0, (114.0, 114.0, 114.0), top=140, left=0)),
                ("convertto", lambda: pkg.convertto_into(f4, b4, 1 / 255.0, 0.0)),
                ("reformat", lambda: pkg.reformat_into(p4, f4, src_layout="NHWC", dst_layout="NCHW"))], fused4)
    del r4, b4, f4, p4
    del src, out, ref, ref4, s4

    # ---- config 5: 4K, linear and nearest
    n = 64
    src = torch.randint(0, 256, (n, 2160, 3840, 3), dtype=torch.uint8, device="cuda", generator=g)
    out = torch.empty((n, 3, 448, 448), dtype=torch.float16, device="cuda")
    ref = torch.empty((n, 3, 448, 448), dtype=torch.float32, device="cuda")
    k = min(n, max(8, threads // 2))
    host = list(src[:k].cpu().numpy())
    for interp, name in ((1, "linear"), (0, "nearest")):
        t_new = gpu_us(lambda: pkg.fused_preprocess_into(out, src, resize_dim=(512, 512), interp=interp, crop_pos=(32, 32),
                                                         layout="NCHW", base=MEAN, mul=INV_STD, srcCast=False), a.launches)
        t_ref = gpu_us(lambda: ref_cuda.rccr_tensor(src, ref, True, (512, 512), interp, (32, 32), 0, INV_STD[0],
                                                    -MEAN[0] * INV_STD[0], False), a.launches) if have_ref else None
        spec = O.ResizeSpec(resize=(512, 512), crop=(32, 32), out_size=(448, 448), interp=interp, src_cast=False, base=MEAN,
                            mul=INV_STD)
        emit(f"5 {name}: 4K -> 512^2 -> 448^2, mean/std, f16 NCHW (64 of 1024 images per launch)", n, t_new, t_ref,
             "float32 output and scalar constants (the reference has neither float16 nor per-channel constants)",
             cpu_images_per_s(host, spec, np.float16, threads, a.cpu_seconds), f"{k} images per pass")
    del src, out, ref

    # ---- config 3: variable-shape batch, random crop -> 224^2, flip p = 0.5, mean/std, f16 NCHW
    n = 64
    rng = np.random.default_rng(1234)
    sizes = [(int(rng.integers(480, 3841)), int(rng.integers(360, 2161))) for _ in range(n)]
    imgs = [torch.randint(0, 256, (h, (w * 3 + 31) // 32 * 32), dtype=torch.uint8, device="cuda", generator=g)
            [:, : w * 3].unflatten(1, (w, 3)) for w, h in sizes]
    batch = pkg.ImageBatchVarShape(imgs)
    rects = []
    for w, h in sizes:
        area = rng.uniform(0.08, 1.0) * w * h
        ar = np.exp(rng.uniform(np.log(3 / 4), np.log(4 / 3)))
        cw, ch = min(w, int(round(np.sqrt(area * ar)))), min(h, int(round(np.sqrt(area / ar))))
        rects.append((int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch))
    roi_np = np.array(rects, np.int32)
    flip_np = np.where(rng.random(n) < 0.5, 1, 2).astype(np.int32)
    roi, flip = torch.from_numpy(roi_np).cuda(), torch.from_numpy(flip_np).cuda()
    out = torch.empty((n, 3, 224, 224), dtype=torch.float16, device="cuda")
    t_new = gpu_us(lambda: pkg.fused_preprocess_into(out, batch, resize_dim=(224, 224), interp=1, layout="NCHW", base=MEAN,
                                                     mul=INV_STD, srcCast=True, roi=roi, flip_code=flip), a.launches)
    ref = torch.empty((n, 3, 224, 224), dtype=torch.float32, device="cuda")
    t_ref = gpu_us(lambda: ref_cuda.rccr_varshape(batch.descriptor_table(), n, ref, True, (224, 224), 1, (0, 0), 0,
                                                  INV_STD[0], -MEAN[0] * INV_STD[0], True), a.launches) if have_ref else None
    spec = O.ResizeSpec(resize=(224, 224), crop=(0, 0), out_size=(224, 224), interp=O.LINEAR, src_cast=True, base=MEAN,
                        mul=INV_STD)
    k = min(n, max(16, threads))
    host = [im.cpu().numpy() for im in imgs[:k]]
    emit("3: 64 random-size images, random crop -> 224^2 linear, flip p=0.5, mean/std, f16 NCHW", n, t_new, t_ref,
         "whole images instead of crop rectangles, no flip, float32, scalar constants (its var-shape kernel takes none of those)",
         cpu_images_per_s(host, spec, np.float16, threads, a.cpu_seconds, roi=roi_np[:k], flip=flip_np[:k]),
         f"{k} of 64 images per pass")
    return 0


if __name__ == "__main__":
    sys.exit(main())
