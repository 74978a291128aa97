"""GPU: seeded random sweep over the whole argument space of the resize path (shapes, scales, crops, placements,
regions of interest, flips, layouts, element types, affine forms), both kernels against the CPU oracle -- the stand-in for
the reference's time-boxed stress loops (tests/cvcuda/stressTest)."""
import numpy as np
import pytest
import torch

from gpu_util import assert_parity, kernel_path, padded_images, to_dev

pytestmark = pytest.mark.gpu

TORCH = {np.uint8: torch.uint8, np.float32: torch.float32, np.float16: torch.float16}


def _case(rng):
    n = int(rng.integers(1, 5))
    varshape = bool(rng.integers(2))
    sizes = [(int(rng.integers(1, 400)), int(rng.integers(1, 300))) for _ in range(n)]
    if not varshape:
        sizes = [sizes[0]] * n
    use_roi = varshape and bool(rng.integers(2))
    rois = None
    if use_roi:
        rois = []
        for w, h in sizes:
            rw, rh = int(rng.integers(1, w + 1)), int(rng.integers(1, h + 1))
            rois.append((int(rng.integers(0, w - rw + 1)), int(rng.integers(0, h - rh + 1)), rw, rh))
        rois = np.array(rois, np.int32)
    resize = (int(rng.integers(2, 300)), int(rng.integers(2, 200)))
    out = (int(rng.integers(1, resize[0] + 1)), int(rng.integers(1, resize[1] + 1)))
    crop = (int(rng.integers(0, resize[0] - out[0] + 1)), int(rng.integers(0, resize[1] - out[1] + 1)))
    canvas = None
    pos = (0, 0)
    if rng.integers(3) == 0:
        canvas = (out[0] + int(rng.integers(0, 40)), out[1] + int(rng.integers(0, 30)))
        pos = (int(rng.integers(0, canvas[0] - out[0] + 1)), int(rng.integers(0, canvas[1] - out[1] + 1)))
    flips = rng.integers(-1, 3, n).astype(np.int32) if rng.integers(2) else None
    per_channel = bool(rng.integers(2))
    return dict(sizes=sizes, varshape=varshape, rois=rois, resize=resize, out=out, crop=crop, canvas=canvas, pos=pos,
                flips=flips, interp=int(rng.integers(2)), src_cast=bool(rng.integers(2)), manip=int(rng.integers(2)),
                dtype=[np.uint8, np.float32, np.float16][int(rng.integers(3))], planar=bool(rng.integers(2)),
                per_channel=per_channel, scale=float(np.float32(rng.uniform(-2, 2))),
                offset=float(np.float32(rng.uniform(-50, 300))),
                base=tuple(float(np.float32(v)) for v in rng.uniform(0, 200, 3)),
                mul=tuple(float(np.float32(v)) for v in rng.uniform(0.001, 1.5, 3)),
                pad=float(rng.integers(0, 256)), pad_to=[1, 4, 16, 32][int(rng.integers(4))],
                offset_bytes=int(rng.integers(0, 4)))


@pytest.mark.parametrize("seed", range(60))
def test_random_resize_cases(pkg, oracle, seed):
    rng = np.random.default_rng(90000 + seed)
    c = _case(rng)
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for w, h in c["sizes"]]
    spec = oracle.ResizeSpec(resize=c["resize"], crop=c["crop"], out_size=c["out"], interp=c["interp"],
                             src_cast=c["src_cast"], manip=c["manip"], scale=c["scale"], offset=c["offset"],
                             base=c["base"] if c["per_channel"] else None, mul=c["mul"] if c["per_channel"] else None,
                             gscale=1.25 if c["per_channel"] else 1.0, shift=-3.0 if c["per_channel"] else 0.0,
                             canvas=c["canvas"], dst_pos=c["pos"], pad_value=c["pad"])
    want = oracle.resize_crop(images, spec, c["dtype"], c["planar"], roi=c["rois"], flip=c["flips"])
    if c["varshape"]:
        src = pkg.ImageBatchVarShape(padded_images(images, pad_to=c["pad_to"], offset=c["offset_bytes"]))
    else:
        src = to_dev(np.stack(images))
    cw, ch = spec.canvas_size
    n = len(images)
    shape = (n, 3, ch, cw) if c["planar"] else (n, ch, cw, 3)
    kw = dict(resize_dim=c["resize"], interp=c["interp"], crop_pos=c["crop"], layout="NCHW" if c["planar"] else "NHWC",
              manip=c["manip"], srcCast=c["src_cast"], pad_value=c["pad"])
    if c["per_channel"]:
        kw.update(base=c["base"], mul=c["mul"], gscale=1.25, shift=-3.0)
    else:
        kw.update(scale=c["scale"], offset=c["offset"])
    if c["canvas"] is not None:
        kw.update(dst_pos=c["pos"], region_size=c["out"])
    if c["rois"] is not None:
        kw["roi"] = to_dev(c["rois"])
    if c["flips"] is not None:
        kw["flip_code"] = to_dev(c["flips"])
    for path in (1, 2, 3):
        out = torch.zeros(shape, dtype=TORCH[c["dtype"]], device="cuda")
        with kernel_path(pkg, path):
            pkg.fused_preprocess_into(out, src, **kw)
            torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, exact=(c["interp"] == 0), what=f"seed {seed} path {path} {c}")
    assert pkg.read_device_error() == 0
