"""Times the reference project's own CUDA kernels (compiled for sm_100a into oracle/_ref) next to this library's kernels,
on the same GPU, same inputs, CUDA events on the launching stream. Not collected by pytest.

    python tests/reference_cuda_timing.py [--images 256] [--launches 50]

What the reference can and cannot do in one kernel matters for a like-for-like reading:
* classification batch (bench.py's workload): the reference operator has one scalar scale/offset, so its kernel is timed
  with scalar constants (float32 NCHW) -- the per-channel Normalize pass its pipeline would still need is NOT included;
  this library's kernel does the per-channel form in the same pass.
* the reference's own Python benchmark shape (resize 256, crop 224, channel reverse, uint8 NHWC): identical work.
* CropFlipNormalizeReformat on 1080p RGB: identical work.
The reference refuses dense inputs above 2 GiB, so at most 345 1080p images per call.
"""
import argparse
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as ge  # noqa: E402
from oracle import ref_cuda  # noqa: E402

MEAN = (123.675, 116.28, 103.53)
INV_STD = tuple(float(np.float32(1.0) / np.float32(s)) for s in (58.395, 57.12, 57.375))


def timed(fn, launches):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(launches):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / launches * 1000.0  # microseconds


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--images", type=int, default=256)
    ap.add_argument("--launches", type=int, default=50)
    a = ap.parse_args()
    if ref_cuda.lib() is None:
        print(json.dumps({"unavailable": "reference CUDA kernels were not built"}))
        return 0
    pkg = ge.load_package()
    n = a.images
    g = torch.Generator(device="cuda")
    g.manual_seed(1234)
    src = torch.randint(0, 256, (n, 1080, 1920, 3), dtype=torch.uint8, device="cuda", generator=g)
    rows = []

    # 1. classification batch, float32 NCHW
    out_new = torch.empty((n, 3, 224, 224), dtype=torch.float32, device="cuda")
    out_ref = torch.empty_like(out_new)
    t_new = timed(lambda: pkg.fused_preprocess_into(out_new, src, resize_dim=(256, 256), interp=1, crop_pos=(16, 16),
                                                    layout="NCHW", base=MEAN, mul=INV_STD, srcCast=False), a.launches)
    t_ref = timed(lambda: ref_cuda.rccr_tensor(src, out_ref, True, (256, 256), 1, (16, 16), 0, INV_STD[0],
                                               -MEAN[0] * INV_STD[0], False), a.launches)
    rows.append({"case": "1080p->256->224 linear, f32 NCHW (reference: scalar constants, no Normalize pass)",
                 "images": n, "new_us": t_new, "reference_us": t_ref, "speedup": t_ref / t_new})

    # 2. the reference's Python benchmark shape, uint8 NHWC, channel reverse, identical work
    out_new8 = torch.empty((n, 224, 224, 3), dtype=torch.uint8, device="cuda")
    out_ref8 = torch.empty_like(out_new8)
    t_new = timed(lambda: pkg.resize_crop_convert_reformat_into(out_new8, src, (256, 256), 1, (16, 16), layout="NHWC",
                                                                manip=1, srcCast=True), a.launches)
    t_ref = timed(lambda: ref_cuda.rccr_tensor(src, out_ref8, False, (256, 256), 1, (16, 16), 1, 1.0, 0.0, True),
                  a.launches)
    diff = (out_new8.int() - out_ref8.int()).abs().max().item()
    rows.append({"case": "1080p->256->224 linear, u8 NHWC, channel reverse (identical work)", "images": n,
                 "new_us": t_new, "reference_us": t_ref, "speedup": t_ref / t_new, "max_abs_diff": diff})

    # 3. same, nearest
    t_new = timed(lambda: pkg.resize_crop_convert_reformat_into(out_new8, src, (256, 256), 0, (16, 16), layout="NHWC",
                                                                manip=1), a.launches)
    t_ref = timed(lambda: ref_cuda.rccr_tensor(src, out_ref8, False, (256, 256), 0, (16, 16), 1, 1.0, 0.0, True),
                  a.launches)
    rows.append({"case": "1080p->256->224 nearest, u8 NHWC, channel reverse (identical work)", "images": n,
                 "new_us": t_new, "reference_us": t_ref, "speedup": t_ref / t_new,
                 "bit_equal": bool(torch.equal(out_new8, out_ref8))})

    # 4. var-shape batch through the reference's var-shape kernel
    m = min(n, 64)
    imgs = [src[i] for i in range(m)]
    batch = pkg.ImageBatchVarShape(imgs)
    out_new = torch.empty((m, 3, 224, 224), dtype=torch.float32, device="cuda")
    out_ref = torch.empty_like(out_new)
    t_new = timed(lambda: pkg.resize_crop_convert_reformat_into(out_new, batch, (256, 256), 1, (16, 16), layout="NCHW",
                                                                scale=1 / 255.0, srcCast=False), a.launches)
    t_ref = timed(lambda: ref_cuda.rccr_varshape(batch.descriptor_table(), m, out_ref, True, (256, 256), 1, (16, 16), 0,
                                                 1 / 255.0, 0.0, False), a.launches)
    rows.append({"case": "var-shape batch of 1080p images ->256->224 linear, f32 NCHW (identical work)", "images": m,
                 "new_us": t_new, "reference_us": t_ref, "speedup": t_ref / t_new})

    # 5. CropFlipNormalizeReformat, 1080p RGB u8 -> f32 NCHW, crop = full image, flip both axes
    k = min(n, 32)
    batch = pkg.ImageBatchVarShape([src[i] for i in range(k)])
    out_new = torch.empty((k, 3, 1080, 1920), dtype=torch.float32, device="cuda")
    out_ref = torch.empty_like(out_new)
    rect = torch.tensor([[0, 0, 1920, 1080]] * k, dtype=torch.int32, device="cuda").reshape(k, 1, 1, 4)
    flip = torch.full((k,), -1, dtype=torch.int32, device="cuda")
    base = torch.tensor(MEAN, dtype=torch.float32, device="cuda").reshape(1, 1, 1, 3)
    scale = torch.tensor(INV_STD, dtype=torch.float32, device="cuda").reshape(1, 1, 1, 3)
    t_new = timed(lambda: pkg.crop_flip_normalize_reformat_into(out_new, batch, rect, flip, base, scale, layout="NCHW",
                                                                border=pkg.Border.REFLECT101), a.launches)
    t_ref = timed(lambda: ref_cuda.cfnr_u8(batch.descriptor_table(), k, 3, out_ref, True, rect, flip, base, scale, 4, 0.0,
                                           1.0, 0.0, 0.0, 0), a.launches)
    diff = (out_new - out_ref).abs().max().item()
    rows.append({"case": "CropFlipNormalizeReformat 1080p RGB u8 -> f32 NCHW, flip -1 (identical work)", "images": k,
                 "new_us": t_new, "reference_us": t_ref, "speedup": t_ref / t_new, "max_abs_diff": diff})

    for r in rows:
        print(json.dumps(r))
    return 0


if __name__ == "__main__":
    sys.exit(main())
