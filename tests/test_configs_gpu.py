"""The benchmark configurations through the fused entry point, checked three ways:

* against committed outputs of CHAINS of the reference's own golden functions (tests/golden/fused_golden.npz);
* against those chains computed on the spot by the reference's compiled goldens (oracle/_ref, when it travelled with
  the tree), at the configurations' real image sizes -- the CUDA result is compared with the reference code itself, not
  with the restatement;
* at each configuration's full batch (256 / 128 / 64 images; 90 4K images so that sample offsets pass 2 GiB), on a
  sample of the images.

Tolerances are those of gpu_util (nearest bit-exact, float32 1e-5, float16 1 unit in the last place); the observed
differences are zero.
"""
import numpy as np
import pytest
import torch

from gpu_util import assert_parity, kernel_path, to_dev
from ref_tables import INV_STD, MEAN, fused_fixture_cases

pytestmark = pytest.mark.gpu

PATHS = (1, 2, 3)  # per-pixel gather, staged pipeline, row walk


def _fused(pkg, kind, inputs, par, dtype, path):
    tdt = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16}[np.dtype(dtype)]
    with kernel_path(pkg, path):
        if kind == 0:
            rw, rh, cx, cy, ow, oh, interp = (int(v) for v in par)
            out = torch.empty((len(inputs), 3, oh, ow), dtype=tdt, device="cuda")
            pkg.fused_preprocess_into(out, to_dev(inputs), resize_dim=(rw, rh), interp=interp, crop_pos=(cx, cy), layout="NCHW",
                                      base=MEAN, mul=INV_STD, srcCast=False)
        elif kind == 1:
            images, rects, flips = inputs
            ow, oh = (int(v) for v in par)
            out = torch.empty((len(images), 3, oh, ow), dtype=tdt, device="cuda")
            batch = pkg.ImageBatchVarShape([to_dev(im) for im in images])
            pkg.fused_preprocess_into(out, batch, resize_dim=(ow, oh), interp=1, layout="NCHW", base=MEAN, mul=INV_STD,
                                      srcCast=True, roi=to_dev(rects), flip_code=to_dev(flips))
        else:
            rw, rh, cw, ch, dx, dy, pad = (int(v) for v in par)
            out = torch.full((len(inputs), 3, ch, cw), -1.0, dtype=tdt, device="cuda")
            pkg.fused_preprocess_into(out, to_dev(inputs), resize_dim=(rw, rh), interp=1, layout="NCHW", manip=1,
                                      scale=1.0 / 255.0, srcCast=True, dst_pos=(dx, dy), region_size=(rw, rh),
                                      pad_value=float(pad))
        torch.cuda.synchronize()
    return out.cpu().numpy()


def test_fused_passes_equal_the_committed_reference_chains(pkg):
    for k, kind, inputs, par, ref in fused_fixture_cases():
        for path in PATHS:
            got = _fused(pkg, kind, inputs, par, ref.dtype, path)
            exact = kind == 0 and int(par[6]) == 0
            assert_parity(got, ref, exact=exact, what=f"fixture {k} path {path}")
            assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), f"fixture {k} path {path}: expected bit-equality"
    assert pkg.read_device_error() == 0


def _need_ref(oracle):
    if oracle.ref() is None:
        pytest.skip("the reference's compiled goldens are not on this machine")


def test_config2_against_the_reference_chain(pkg, oracle):
    _need_ref(oracle)
    src = np.random.default_rng(1234).integers(0, 256, (2, 1080, 1920, 3), dtype=np.uint8)
    want = oracle.ref_resize_then_normalize(src, (256, 256), (16, 16), (224, 224), 1, MEAN, INV_STD)
    for path in PATHS:
        got = _fused(pkg, 0, src, (256, 256, 16, 16, 224, 224, 1), np.float32, path)
        assert_parity(got, want, what=f"config 2 path {path}")


def test_config3_against_the_reference_chain(pkg, oracle):
    _need_ref(oracle)
    rng = np.random.default_rng(4)
    sizes = [(3840, 2160), (480, 360), (1733, 977), (2048, 1151)]
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (w, h) in sizes]
    rects = np.array([(1000, 500, 2000, 1600), (0, 0, 480, 360), (37, 11, 900, 800), (1024, 3, 1000, 1148)], np.int32)
    flips = np.array([1, 2, 1, 1], np.int32)
    want = oracle.ref_crop_resize_flip_normalize(images, rects, flips, (224, 224), MEAN, INV_STD, np.float16)
    for path in PATHS:
        got = _fused(pkg, 1, (images, rects, flips), (224, 224), np.float16, path)
        assert_parity(got, want, what=f"config 3 path {path}")


def test_config4_against_the_reference_chain(pkg, oracle):
    _need_ref(oracle)
    src = np.random.default_rng(8).integers(0, 256, (2, 1080, 1920, 3), dtype=np.uint8)
    want = oracle.ref_letterbox(src, (640, 360), (640, 640), (0, 140), 114, 1.0 / 255.0)
    for path in PATHS:
        got = _fused(pkg, 2, src, (640, 360, 640, 640, 0, 140, 114), np.float32, path)
        assert_parity(got, want, what=f"config 4 path {path}")


@pytest.mark.parametrize("interp", [0, 1])
def test_config5_against_the_reference_chain(pkg, oracle, interp):
    _need_ref(oracle)
    src = np.random.default_rng(16).integers(0, 256, (1, 2160, 3840, 3), dtype=np.uint8)
    want = oracle.ref_resize_then_normalize(src, (512, 512), (32, 32), (448, 448), interp, MEAN, INV_STD, np.float16)
    for path in PATHS:
        got = _fused(pkg, 0, src, (512, 512, 32, 32, 448, 448, interp), np.float16, path)
        assert_parity(got, want, exact=(interp == 0), what=f"config 5 interp {interp} path {path}")


# ------------------------------------------------------------------------------------------------ full batches

def _device_batch(n, h, w, seed):
    g = torch.Generator(device="cuda")
    g.manual_seed(seed)
    return torch.randint(0, 256, (n, h, w, 3), dtype=torch.uint8, device="cuda", generator=g)


def _expect_dense(oracle, images, spec, dtype, chain):
    """The restatement on the sampled images, and -- where the reference's goldens are here -- the chain, which must agree."""
    want = oracle.resize_crop(list(images), spec, dtype, True, nthreads=8)
    if oracle.ref() is not None:
        ref = chain(images)
        assert np.array_equal(want.view(np.uint8), ref.view(np.uint8)), "restatement and reference chain disagree"
    return want


def test_config2_full_batch_of_256(pkg, oracle):
    n, sample = 256, [0, 1, 127, 200, 255]
    src = _device_batch(n, 1080, 1920, 2)
    out = torch.empty((n, 3, 224, 224), dtype=torch.float32, device="cuda")
    pkg.fused_preprocess_into(out, src, resize_dim=(256, 256), interp=1, crop_pos=(16, 16), layout="NCHW", base=MEAN,
                              mul=INV_STD, srcCast=False)
    torch.cuda.synchronize()
    images = src[sample].cpu().numpy()
    spec = oracle.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=1, src_cast=False, base=MEAN,
                             mul=INV_STD)
    want = _expect_dense(oracle, images, spec, np.float32,
                         lambda b: oracle.ref_resize_then_normalize(b, (256, 256), (16, 16), (224, 224), 1, MEAN, INV_STD))
    assert_parity(out[sample].cpu().numpy(), want, what="config 2, 256 images")
    assert bool(torch.isfinite(out).all()) and pkg.read_device_error() == 0


def test_config3_full_batch_of_128(pkg, oracle):
    """128 images with H in [360, 2160], W in [480, 3840], one random rectangle each (8-100 % of the area, aspect 3/4..4/3),
    horizontal flip with p = 0.5, float16 NCHW; every eighth image is checked."""
    rng = np.random.default_rng(1234)
    n = 128
    sizes = [(int(rng.integers(480, 3841)), int(rng.integers(360, 2161))) for _ in range(n)]
    rects = np.array(pkg.random_crop_rects(sizes, seed=1234), np.int32)
    flips = np.where(rng.random(n) < 0.5, 1, 2).astype(np.int32)
    g = torch.Generator(device="cuda")
    g.manual_seed(3)
    images = [torch.randint(0, 256, (h, w, 3), dtype=torch.uint8, device="cuda", generator=g) for (w, h) in sizes]
    out = torch.empty((n, 3, 224, 224), dtype=torch.float16, device="cuda")
    pkg.fused_preprocess_into(out, pkg.ImageBatchVarShape(images), resize_dim=(224, 224), interp=1, layout="NCHW", base=MEAN,
                              mul=INV_STD, srcCast=True, roi=to_dev(rects), flip_code=to_dev(flips))
    torch.cuda.synchronize()
    sample = list(range(0, n, 8)) + [n - 1]
    host = [images[i].cpu().numpy() for i in sample]
    spec = oracle.ResizeSpec(resize=(224, 224), out_size=(224, 224), interp=1, src_cast=True, base=MEAN, mul=INV_STD)
    want = oracle.resize_crop(host, spec, np.float16, True, roi=rects[sample], flip=flips[sample], nthreads=8)
    if oracle.ref() is not None:
        ref = oracle.ref_crop_resize_flip_normalize(host, rects[sample], flips[sample], (224, 224), MEAN, INV_STD, np.float16)
        assert np.array_equal(want.view(np.uint16), ref.view(np.uint16)), "restatement and reference chain disagree"
    assert_parity(out[sample].cpu().numpy(), want, what="config 3, 128 images")
    assert bool(torch.isfinite(out.float()).all()) and pkg.read_device_error() == 0


def test_config4_full_batch_of_64(pkg, oracle):
    n, sample = 64, [0, 31, 63]
    src = _device_batch(n, 1080, 1920, 4)
    out = torch.full((n, 3, 640, 640), -1.0, dtype=torch.float32, device="cuda")
    pkg.fused_preprocess_into(out, src, resize_dim=(640, 360), interp=1, layout="NCHW", manip=1, scale=1.0 / 255.0,
                              srcCast=True, dst_pos=(0, 140), region_size=(640, 360), pad_value=114.0)
    torch.cuda.synchronize()
    images = src[sample].cpu().numpy()
    spec = oracle.ResizeSpec(resize=(640, 360), out_size=(640, 360), interp=1, src_cast=True, manip=1, scale=1.0 / 255.0,
                             canvas=(640, 640), dst_pos=(0, 140), pad_value=114.0)
    want = _expect_dense(oracle, images, spec, np.float32,
                         lambda b: oracle.ref_letterbox(b, (640, 360), (640, 640), (0, 140), 114, 1.0 / 255.0))
    assert_parity(out[sample].cpu().numpy(), want, what="config 4, 64 images")
    pad = np.float32(114.0) * np.float32(1.0 / 255.0)
    assert bool((out[:, :, :140] == float(pad)).all()) and bool((out[:, :, 500:] == float(pad)).all())


@pytest.mark.parametrize("interp", [0, 1])
def test_config5_batch_past_two_gib(pkg, oracle, interp):
    """90 4K images = 2.24 GB: the reference refuses more than 86 per call (32-bit sample offsets,
    src/cvcuda/priv/OpResizeCropConvertReformat.cu:515-519); here the images beyond 2 GiB must come out right."""
    n, sample = 90, [0, 85, 86, 87, 89]
    src = _device_batch(n, 2160, 3840, 5)
    out = torch.empty((n, 3, 448, 448), dtype=torch.float16, device="cuda")
    pkg.fused_preprocess_into(out, src, resize_dim=(512, 512), interp=interp, crop_pos=(32, 32), layout="NCHW", base=MEAN,
                              mul=INV_STD, srcCast=False)
    torch.cuda.synchronize()
    images = src[sample].cpu().numpy()
    spec = oracle.ResizeSpec(resize=(512, 512), crop=(32, 32), out_size=(448, 448), interp=interp, src_cast=False, base=MEAN,
                             mul=INV_STD)
    want = _expect_dense(oracle, images, spec, np.float16,
                         lambda b: oracle.ref_resize_then_normalize(b, (512, 512), (32, 32), (448, 448), interp, MEAN,
                                                                    INV_STD, np.float16))
    assert_parity(out[sample].cpu().numpy(), want, exact=(interp == 0), what=f"config 5 interp {interp}, 90 images")
    assert pkg.read_device_error() == 0
    del src
