"""GPU parity: CropFlipNormalizeReformat against the CPU oracle, through the library's C entry point."""
import os

import numpy as np
import pytest
import torch

import ref_tables as T
from gpu_util import _TORCH_DTYPE, assert_parity, kernel_path, padded_images, to_dev

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _run(pkg, images, src_planar, rects, flips, osz, dst_dtype, dst_planar, border, bvalue, base, scale, gscale, shift,
         eps, flags, pad_to=32, offset=0):
    n = len(images)
    ch = images[0].shape[0] if src_planar else images[0].shape[2]
    batch = pkg.ImageBatchVarShape(padded_images(images, pad_to=pad_to, offset=offset, planar=src_planar),
                                   planar=src_planar)
    shape = (n, ch, osz[1], osz[0]) if dst_planar else (n, osz[1], osz[0], ch)
    out = pkg.crop_flip_normalize_reformat(
        batch, shape, _TORCH_DTYPE[np.dtype(dst_dtype)], "NCHW" if dst_planar else "NHWC",
        to_dev(np.asarray(rects, np.int32).reshape(n, 1, 1, 4)), to_dev(np.asarray(flips, np.int32)),
        to_dev(np.asarray(base, np.float32).reshape(1, 1, 1, -1)), to_dev(np.asarray(scale, np.float32).reshape(1, 1, 1, -1)),
        gscale, shift, eps, flags, border, bvalue)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("idx", range(len(T.CFNR_ROWS)))
def test_reference_table(pkg, oracle, idx):
    """The reference's 18 test rows with inputs drawn like its driver draws them (border value 1.0)."""
    row = T.CFNR_ROWS[idx]
    for seed in (idx, 1000 + idx):
        images, rects, flips, base, scale, osz = T.cfnr_case(row, seed)
        want = oracle.crop_flip_normalize(images, row.src_planar, rects, flips, osz, row.dst_dtype, row.dst_planar,
                                          row.border, 1.0, base, scale, row.gscale, row.gshift, row.eps, row.flags)
        for path in (0, 1):  # 0: automatic (the four-pixel kernel where it applies), 1: per-pixel kernel
            with kernel_path(pkg, path):
                got = _run(pkg, images, row.src_planar, rects, flips, osz, row.dst_dtype, row.dst_planar, row.border,
                           1.0, base, scale, row.gscale, row.gshift, row.eps, row.flags)
            assert_parity(got, want, what=f"row {idx} seed {seed} path {path}")


def test_golden_fixtures(pkg):
    """Fixtures computed by the reference's own golden function (tests/golden/make_golden.py)."""
    z = np.load(os.path.join(GOLDEN, "cfnr_golden.npz"))
    for k in range(int(z["cfnr_count"])):
        x, y, w, h, flip, ow, oh, sp, dp, border, flags = (int(v) for v in z[f"cfnr{k}_par"])
        gs, sh, eps = (float(v) for v in z[f"cfnr{k}_f"])
        ref = z[f"cfnr{k}_ref"]
        got = _run(pkg, [z[f"cfnr{k}_src"]], bool(sp), [[x, y, w, h]], [flip], (ow, oh), ref.dtype, bool(dp), border, 1.0,
                   z[f"cfnr{k}_base"], z[f"cfnr{k}_scale"], gs, sh, eps, flags)[0]
        assert_parity(got, ref, what=f"fixture {k}")


@pytest.mark.parametrize("border", range(5))
@pytest.mark.parametrize("src_dtype,dst_dtype", [(np.uint8, np.float32), (np.uint8, np.float16), (np.int16, np.int8),
                                                 (np.float32, np.uint16), (np.uint16, np.int16), (np.int8, np.int32),
                                                 (np.int32, np.uint8), (np.uint32, np.float32), (np.float32, np.uint32)])
def test_dtype_and_border_matrix(pkg, oracle, border, src_dtype, dst_dtype):
    if np.dtype(src_dtype) not in _TORCH_DTYPE or np.dtype(dst_dtype) not in _TORCH_DTYPE:
        pytest.skip("this torch build has no such tensor type")
    rng = np.random.default_rng(border * 17 + np.dtype(src_dtype).num)
    for src_planar, dst_planar, ch in ((False, True, 3), (True, False, 4), (False, False, 1), (True, True, 2)):
        images = []
        for _ in range(3):
            w, h = int(rng.integers(1, 40)), int(rng.integers(1, 40))
            shape = (ch, h, w) if src_planar else (h, w, ch)
            if src_dtype == np.float32:
                images.append(rng.uniform(-50, 300, shape).astype(np.float32))
            else:
                info = np.iinfo(src_dtype)
                images.append(rng.integers(max(info.min, -300), min(info.max, 300) + 1, shape).astype(src_dtype))
        rects = [(int(rng.integers(-45, 45)), int(rng.integers(-45, 45)), int(rng.integers(1, 60)), int(rng.integers(1, 60)))
                 for _ in images]
        flips = rng.integers(-2, 4, len(images)).astype(np.int32)
        base = rng.uniform(-20, 100, 4).astype(np.float32)
        scale = rng.uniform(0.1, 2.0, 4).astype(np.float32)
        for flags, eps in ((0, 0.0), (1, 0.37)):
            want = oracle.crop_flip_normalize(images, src_planar, rects, flips, (50, 47), dst_dtype, dst_planar, border,
                                              7.9, base, scale, 1.3, -2.5, eps, flags)
            got = _run(pkg, images, src_planar, rects, flips, (50, 47), dst_dtype, dst_planar, border, 7.9, base, scale,
                       1.3, -2.5, eps, flags, pad_to=4, offset=4)
            assert_parity(got, want, what=f"border {border} planar {src_planar}->{dst_planar} flags {flags}")


@pytest.mark.parametrize("border", range(5))
@pytest.mark.parametrize("dst_dtype,dst_planar", [(np.float32, True), (np.float16, True), (np.uint8, True),
                                                  (np.float32, False), (np.uint8, False)])
def test_uint8_rgb_fast_kernel(pkg, oracle, border, dst_dtype, dst_planar):
    """The four-pixels-per-thread kernel: every flip code, crops hanging over each image edge, widths that are not a
    multiple of four, padded and unaligned source rows, against the oracle and against the per-pixel kernel."""
    rng = np.random.default_rng(500 + border)
    sizes = [(37, 23), (64, 16), (130, 9), (5, 41), (257, 3), (96, 96)]
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for w, h in sizes]
    rects = [(-3, -2, 30, 20), (0, 0, 64, 16), (7, 1, 140, 7), (1, 30, 9, 20), (250, -1, 20, 6), (8, 8, 80, 80)]
    flips = np.array([1, 0, -1, 2, 1, -1], np.int32)
    base = np.array([10.5, 20.25, 30.125], np.float32)
    scale = np.array([0.5, 0.25, 1.5], np.float32)
    for out_w, out_h in ((131, 40), (64, 16), (3, 5)):
        want = oracle.crop_flip_normalize(images, False, rects, flips, (out_w, out_h), dst_dtype, dst_planar, border, 5.0,
                                          base, scale, 1.25, -0.5, 0.0, 0)
        for pad_to, offset in ((32, 0), (1, 1)):
            got = {}
            for path in (0, 1):
                with kernel_path(pkg, path):
                    got[path] = _run(pkg, images, False, rects, flips, (out_w, out_h), dst_dtype, dst_planar, border, 5.0,
                                     base, scale, 1.25, -0.5, 0.0, 0, pad_to=pad_to, offset=offset)
                assert_parity(got[path], want, what=f"{out_w}x{out_h} pad {pad_to} path {path}")
            assert np.array_equal(got[0].view(np.uint8), got[1].view(np.uint8))


def test_benchmark_shape_of_the_reference(pkg, oracle):
    """The reference's own benchmark case: 1080x1920 single channel, REFLECT101, flip -1, crop = full image,
    global scale 1.234, shift 2.345 (bench/BenchCropFlipNormalizeReformat.cpp:32-49)."""
    rng = np.random.default_rng(8)
    for dt in (np.uint8, np.float32):
        img = (rng.uniform(0, 255, (1080, 1920, 1))).astype(dt)
        want = oracle.crop_flip_normalize([img], False, [(0, 0, 1920, 1080)], [-1], (1920, 1080), dt, False, 4, 0.0,
                                          [0.0], [1.0], 1.234, 2.345, 0.0, 0, nthreads=8)
        got = _run(pkg, [img], False, [(0, 0, 1920, 1080)], [-1], (1920, 1080), dt, False, 4, 0.0, [0.0], [1.0], 1.234,
                   2.345, 0.0, 0)
        assert_parity(got, want, what=str(dt))


def test_bad_arguments(pkg):
    img = torch.zeros((8, 8, 3), dtype=torch.uint8, device="cuda")
    batch = pkg.ImageBatchVarShape([img])
    rect = to_dev(np.array([[0, 0, 8, 8]], np.int32).reshape(1, 1, 1, 4))
    flip = to_dev(np.array([0], np.int32))
    one = to_dev(np.ones((1, 1, 1, 1), np.float32))
    two = to_dev(np.ones((1, 1, 1, 2), np.float32))
    out = torch.zeros((1, 8, 8, 3), dtype=torch.float32, device="cuda")
    for kwargs, base, scale in (({}, two, one), ({}, one, two), ({"border": 7}, one, one)):
        with pytest.raises(pkg.ops.Error) as e:
            pkg.crop_flip_normalize_reformat_into(out, batch, rect, flip, base, scale, **kwargs)
        assert e.value.status == pkg.ops.Status.ERROR_INVALID_ARGUMENT
    with pytest.raises(pkg.ops.Error):
        pkg.crop_flip_normalize_reformat_into(out, batch, rect, flip, one, one, layout="CHW")
