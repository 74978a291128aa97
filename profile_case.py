"""A small, self-ending run of one kernel, sized for an `ncu` capture.

    python profile_case.py [--case classify|4k|letterbox|varshape|cfnr|resize-rgb|...] [--images 32] [--path 0|1|2|3]
                           [--launches 5] [--graph]

`--case` names the operator and shape (`--help` lists them: the fused passes of bench.py's configurations, image lists with and
without rectangles, the element types of CropFlipNormalizeReformat, and the stand-alone operators). `--graph` replays the launches
from one CUDA graph, i.e. reports device time with no host work between the kernels; without it the figure includes whatever
the Python call costs when that is longer than the kernel (also printed, as `host ... us per call`). `classify` is the 1080p -> 256x256 -> 224x224 float32 NCHW case of bench.py at a reduced batch: 32 images are
199 MB of source, larger than the 126 MB L2, so DRAM counters still mean something, while the whole run holds well
under 1 GB on the device. Prints the device time per launch measured with CUDA events (never quote that figure from
a run under a profiler).
"""
import argparse
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402

MEAN = (123.675, 116.28, 103.53)
INV_STD = tuple(float(np.float32(1.0) / np.float32(s)) for s in (58.395, 57.12, 57.375))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="classify", choices=("classify", "classify-nhwc-u8", "classify-nhwc-f32", "classify-nhwc-u8-nearest", "4k", "4k-nearest", "letterbox", "cfnr", "cfnr-u8c1", "cfnr-f32c1", "cfnr-rgba8-f32", "cfnr-rgb8p-f32", "cfnr-rgbf32", "varshape", "varshape-narrow", "varshape-small", "varshape-1080p", "varshape-mixed", "resize-rgba", "resize-rgba-nearest", "resize-rgb", "normalize-rgba", "normalize-rgb-f32", "reformat-u8", "reformat-f32", "convertto-u8-f32", "convertto-f32-u8", "border-rgb", "border-rgb-reflect", "border-rgba-f32", "rrc-rgb", "rrc-rgb-nearest"))
    ap.add_argument("--images", type=int, default=32)
    ap.add_argument("--path", type=int, default=0)
    ap.add_argument("--launches", type=int, default=5)
    ap.add_argument("--graph", action="store_true", help="replay the launches from a CUDA graph: device time with no host "
                    "work between launches (small batches otherwise measure the Python call, not the kernel)")
    a = ap.parse_args()
    pkg = ge.load_package()
    pkg.set_kernel_path(a.path)
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    n = a.images
    if a.case == "classify":
        src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g)
        out = torch.empty((n, 3, 224, 224), dtype=torch.float32, device="cuda")
        kw = dict(resize_dim=(256, 256), interp=1, crop_pos=(16, 16), layout="NCHW", base=MEAN, mul=INV_STD, srcCast=False)
    elif a.case in ("classify-nhwc-u8", "classify-nhwc-f32", "classify-nhwc-u8-nearest"):
        # the reference's Python operator benchmark: resize 256x256 linear, centre crop 224x224, channel reverse,
        # interleaved output (bench/python/all_ops/op_resize_crop_convert_reformat.py:25-45)
        src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g)
        out = torch.empty((n, 224, 224, 3), dtype=torch.float32 if a.case.endswith("f32") else torch.uint8, device="cuda")
        kw = dict(resize_dim=(256, 256), interp=int(not a.case.endswith("nearest")), crop_pos=(16, 16), layout="NHWC", manip=1, srcCast=True)
    elif a.case in ("4k", "4k-nearest"):
        src = torch.randint(0, 256, (n, 2160, 3840, 3), dtype=torch.uint8, device="cuda", generator=g)
        out = torch.empty((n, 3, 448, 448), dtype=torch.float16, device="cuda")
        kw = dict(resize_dim=(512, 512), interp=int(a.case == "4k"), crop_pos=(32, 32), layout="NCHW", base=MEAN,
                  mul=INV_STD, srcCast=False)
    elif a.case in ("varshape", "varshape-narrow", "varshape-small"):
        # config 3: variable-shape RGB batch, one random rectangle per image -> 224x224 linear, horizontal flip p=0.5,
        # mean/std, float16 NCHW
        rng = np.random.default_rng(1234)
        # narrow: every row segment fits a small ring slot; small: the whole batch (40 MB) stays in L2
        wmax, hmax = {"varshape": (3840, 2160), "varshape-narrow": (1300, 975), "varshape-small": (640, 480)}[a.case]
        sizes = [(int(rng.integers(480, wmax + 1)), int(rng.integers(360, hmax + 1))) for _ in range(n)]
        imgs = [torch.randint(0, 256, (h, (w * 3 + 31) // 32 * 32), dtype=torch.uint8, device="cuda", generator=g)
                [:, : w * 3].unflatten(1, (w, 3)) for w, h in sizes]
        src = pkg.ImageBatchVarShape(imgs)
        rects = []
        for w, h in sizes:
            area = rng.uniform(0.08, 1.0) * w * h
            ar = np.exp(rng.uniform(np.log(3 / 4), np.log(4 / 3)))
            cw, ch = min(w, int(round(np.sqrt(area * ar)))), min(h, int(round(np.sqrt(area / ar))))
            rects.append((int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch))
        roi = torch.tensor(rects, dtype=torch.int32, device="cuda")
        flip = torch.tensor(np.where(rng.random(n) < 0.5, 1, 2), dtype=torch.int32, device="cuda")
        out = torch.empty((n, 3, 224, 224), dtype=torch.float16, device="cuda")
        kw = dict(resize_dim=(224, 224), interp=1, layout="NCHW", base=MEAN, mul=INV_STD, srcCast=True, roi=roi,
                  flip_code=flip)
        src_bytes = sum(r[2] * r[3] * 3 for r in rects)
        print(f"varshape: crop rectangles hold {src_bytes / 1e6:.1f} MB, output {out.numel() * 2 / 1e6:.1f} MB")
    elif a.case in ("varshape-1080p", "varshape-mixed"):
        # ResizeCropConvertReformat on an image list, the reference operator's own variable-shape form (no rectangles, no
        # flip, scalar constants): every image 1080x1920, or sizes from 0.5x to 1x of that
        rng = np.random.default_rng(7)
        if a.case == "varshape-1080p":
            sizes = [(1920, 1080)] * n
        else:
            sizes = [(int(1920 * f), int(1080 * f)) for f in rng.uniform(0.5, 1.0, n)]
        imgs = [torch.randint(0, 256, (h, (w * 3 + 31) // 32 * 32), dtype=torch.uint8, device="cuda", generator=g)
                [:, : w * 3].unflatten(1, (w, 3)) for w, h in sizes]
        src = pkg.ImageBatchVarShape(imgs)
        out = torch.empty((n, 3, 224, 224), dtype=torch.float32, device="cuda")
        kw = dict(resize_dim=(256, 256), interp=1, crop_pos=(16, 16), layout="NCHW", scale=1 / 255.0, srcCast=False)
    elif a.case == "letterbox":
        src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g)
        out = torch.empty((n, 3, 640, 640), dtype=torch.float32, device="cuda")
        kw = dict(resize_dim=(640, 360), interp=1, layout="NCHW", manip=1, scale=1.0 / 255.0, srcCast=True,
                  dst_pos=(0, 140), region_size=(640, 360), pad_value=114.0)
    if a.case.startswith("resize-"):
        # stand-alone Resize on a shape of the reference's test table (1080 wide x 1920 high -> 720 x 1280,
        # tests/cvcuda/system/TestOpResize.cpp:70), RGBA8 or RGB8, n images per launch
        ch = 3 if a.case == "resize-rgb" else 4
        src = torch.randint(0, 256, (n, 1920, 1080, ch), dtype=torch.uint8, device="cuda", generator=g)
        out = torch.empty((n, 1280, 720, ch), dtype=torch.uint8, device="cuda")
        interp = 0 if a.case.endswith("nearest") else 1
        print(f"resize: {src.numel() / 1e6:.1f} MB in, {out.numel() / 1e6:.1f} MB out")

        def run():
            pkg.resize_into(out, src, interp)
    elif a.case.startswith("normalize-"):
        # stand-alone Normalize on 1080x1920 images with per-channel mean / standard deviation: RGBA8 -> RGBA8 (the
        # reference test's format) or RGB8 -> float32 (the step a classification pipeline runs after its resize)
        ch = 4 if a.case == "normalize-rgba" else 3
        src = torch.randint(0, 256, (n, 1080, 1920, ch), dtype=torch.uint8, device="cuda", generator=g)
        out = torch.empty((n, 1080, 1920, ch), dtype=torch.uint8 if ch == 4 else torch.float32, device="cuda")
        base = torch.tensor((MEAN + (127.5,))[:ch], dtype=torch.float32, device="cuda").reshape(1, 1, 1, ch)
        scale = torch.tensor(((58.395, 57.12, 57.375) + (64.0,))[:ch], dtype=torch.float32, device="cuda").reshape(1, 1, 1, ch)
        print(f"normalize: {src.numel() / 1e6:.1f} MB in, {out.numel() * out.element_size() / 1e6:.1f} MB out")

        def run():
            pkg.normalize_into(out, src, base, scale, pkg.NORMALIZE_SCALE_IS_STDDEV, 64.0 if ch == 4 else 1.0,
                               128.0 if ch == 4 else 0.0, 0.0)
    elif a.case.startswith("reformat-"):
        # stand-alone Reformat, 1080x1920 RGB, NHWC -> NCHW
        dt = torch.uint8 if a.case.endswith("u8") else torch.float32
        src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g).to(dt)
        out = torch.empty((n, 3, 1080, 1920), dtype=dt, device="cuda")
        print(f"reformat: {2 * src.numel() * src.element_size() / 1e6:.1f} MB in + out")

        def run():
            pkg.reformat_into(out, src, src_layout="NHWC", dst_layout="NCHW")
    elif a.case.startswith("convertto-"):
        # stand-alone ConvertTo on 1080x1920 RGB: uint8 -> float32 (x 1/255) or float32 -> uint8 (x 255)
        to_f32 = a.case.endswith("u8-f32")
        src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g)
        src = src if to_f32 else src.float() / 255.0
        out = torch.empty((n, 1080, 1920, 3), dtype=torch.float32 if to_f32 else torch.uint8, device="cuda")
        print(f"convertto: {(src.numel() * src.element_size() + out.numel() * out.element_size()) / 1e6:.1f} MB in + out")

        def run():
            pkg.convertto_into(out, src, 1.0 / 255.0 if to_f32 else 255.0, 0.0)
    elif a.case.startswith("border-"):
        # stand-alone CopyMakeBorder: 1080x1920 images into 1144x1984 (32 pixels on every side; the letterbox / padding
        # step of a detection pipeline), constant or reflect-101 border
        f32 = a.case.endswith("f32")
        ch = 4 if "rgba" in a.case else 3
        src = torch.randint(0, 256, (n, 1080, 1920, ch), dtype=torch.uint8, device="cuda", generator=g)
        src = src.float() if f32 else src
        out = torch.empty((n, 1144, 1984, ch), dtype=src.dtype, device="cuda")
        mode = pkg.Border.REFLECT101 if a.case.endswith("reflect") else pkg.Border.CONSTANT
        print(f"copymakeborder: {(src.numel() * src.element_size() + out.numel() * out.element_size()) / 1e6:.1f} MB in + out")

        def run():
            pkg.copymakeborder_into(out, src, mode, (114.0, 114.0, 114.0, 0.0), top=32, left=32)
    elif a.case.startswith("rrc-"):
        # RandomResizedCrop with the reference's default limits (scale 0.08..1, ratio 3/4..4/3), seed 1: 1080x1920 RGB
        # -> 224x224; the rectangles are drawn once, the timed call is the resized-crop launch the operator makes
        src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g)
        out = torch.empty((n, 224, 224, 3), dtype=torch.uint8, device="cuda")
        rects = pkg.random_crop_rects([(1920, 1080)] * n, seed=1)
        table = torch.tensor(rects, dtype=torch.int32, device="cuda")
        interp = 0 if a.case.endswith("nearest") else 1
        tapped = sum((min(h, 224) * (2 - (interp == 0))) * w * 3 for (_, _, w, h) in rects)
        print(f"random_resized_crop: crop area {sum(w * h for (_, _, w, h) in rects) * 3 / 1e6:.1f} MB, "
              f"rows tapped about {tapped / 1e6:.1f} MB, output {out.numel() / 1e6:.1f} MB")

        def run():
            pkg.resized_crop_into(out, src, table, interp)
    elif a.case == "cfnr":
        # CropFlipNormalizeReformat on the reference benchmark's image size (bench/BenchCropFlipNormalizeReformat.cpp:
        # 1080x1920, crop = full image, flip both axes), here 3-channel uint8 -> float32 NCHW with per-channel constants
        imgs = [torch.randint(0, 256, (1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g) for _ in range(n)]
        batch = pkg.ImageBatchVarShape(imgs)
        out = torch.empty((n, 3, 1080, 1920), dtype=torch.float32, device="cuda")
        rect = torch.tensor([[0, 0, 1920, 1080]] * n, dtype=torch.int32, device="cuda").reshape(n, 1, 1, 4)
        flip = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        base = torch.tensor(MEAN, dtype=torch.float32, device="cuda").reshape(1, 1, 1, 3)
        scale = torch.tensor(INV_STD, dtype=torch.float32, device="cuda").reshape(1, 1, 1, 3)

        def run():
            pkg.crop_flip_normalize_reformat_into(out, batch, rect, flip, base, scale, layout="NCHW",
                                                  border=pkg.Border.REFLECT101)
    elif a.case.startswith("cfnr-"):
        # the other element types of CropFlipNormalizeReformat, same image size, crop and flip. u8c1 / f32c1 are the
        # reference benchmark's own cases: one channel, output of the input's type, interleaved
        kind = a.case[5:]
        sdt, ch, planar, ddt, lay = {"u8c1": (torch.uint8, 1, False, torch.uint8, "NHWC"), "f32c1": (torch.float32, 1, False, torch.float32, "NHWC"),
                                     "rgba8-f32": (torch.uint8, 4, False, torch.float32, "NCHW"),
                                     "rgb8p-f32": (torch.uint8, 3, True, torch.float32, "NCHW"),
                                     "rgbf32": (torch.float32, 3, False, torch.float32, "NHWC")}[kind]
        shape = (ch, 1080, 1920) if planar else (1080, 1920, ch)
        if sdt == torch.uint8:
            imgs = [torch.randint(0, 256, shape, dtype=torch.uint8, device="cuda", generator=g) for _ in range(n)]
        else:
            imgs = [torch.rand(shape, dtype=torch.float32, device="cuda", generator=g) * 255 for _ in range(n)]
        batch = pkg.ImageBatchVarShape(imgs, planar=planar)
        out = torch.empty((n, ch, 1080, 1920) if lay == "NCHW" else (n, 1080, 1920, ch), dtype=ddt, device="cuda")
        rect = torch.tensor([[0, 0, 1920, 1080]] * n, dtype=torch.int32, device="cuda").reshape(n, 1, 1, 4)
        flip = torch.full((n,), -1, dtype=torch.int32, device="cuda")
        base = torch.tensor((MEAN + (10.0,))[:ch], dtype=torch.float32, device="cuda").reshape(1, 1, 1, ch)
        scale = torch.tensor((INV_STD + (0.02,))[:ch], dtype=torch.float32, device="cuda").reshape(1, 1, 1, ch)
        moved = n * 1080 * 1920 * ch * (imgs[0].element_size() + out.element_size())
        print(f"bytes per launch {moved}")

        def run():
            pkg.crop_flip_normalize_reformat_into(out, batch, rect, flip, base, scale, 1.234, 2.345, 12.34, 0, layout=lay,
                                                  border=pkg.Border.REFLECT101)
    else:
        def run():
            pkg.fused_preprocess_into(out, src, **kw)
    for _ in range(3):
        run()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    import time
    if a.graph:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(a.launches):
                run()
        graph.replay()
        torch.cuda.synchronize()
        e0.record()
        graph.replay()
        e1.record()
        host_us = 0.0
    else:
        e0.record()
        t0 = time.perf_counter()
        for _ in range(a.launches):
            run()
        host_us = (time.perf_counter() - t0) / a.launches * 1e6
        e1.record()
    torch.cuda.synchronize()
    print(f"case {a.case} images {n} path {a.path}{' graph' if a.graph else ''}: {e0.elapsed_time(e1) / a.launches * 1000:.1f} us per launch, "
          f"host {host_us:.1f} us per call, device error {pkg.read_device_error()}")


if __name__ == "__main__":
    main()
