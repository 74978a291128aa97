"""CPU: the stand-alone Resize restatement (oracle/resize_oracle.c) against the reference's own golden function
(compiled into oracle/_ref where the reference tree is present) and against the committed fixtures it produced."""
import os

import numpy as np
import pytest

import ref_tables as T

HERE = os.path.dirname(os.path.abspath(__file__))


def _image(rng, w, h, ch, dt):
    if dt == np.float32:
        return rng.uniform(0.0, 300.0, (h, w, ch)).astype(np.float32)
    info = np.iinfo(dt)
    return rng.integers(info.min, info.max + 1, (h, w, ch)).astype(dt)


def test_restatement_matches_the_committed_reference_outputs(oracle):
    g = np.load(os.path.join(HERE, "golden", "resize_golden.npz"))
    n = int(g["resize_count"])
    assert n == 96
    for k in range(n):
        src, ref = g[f"resize{k}_src"], g[f"resize{k}_ref"]
        dw, dh, interp = (int(v) for v in g[f"resize{k}_par"])
        got = oracle.resize_plain([src], [(dw, dh)], interp, golden_float=True)[0]
        assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), f"fixture {k}"


@pytest.mark.parametrize("row", T.RESIZE_ROWS, ids=lambda r: f"{r.src_w}x{r.src_h}-{r.dst_w}x{r.dst_h}-i{r.interp}-{r.channels}x{np.dtype(r.dtype).name}")
def test_restatement_matches_the_reference_golden_on_its_test_table(oracle, row):
    if oracle.ref() is None or not hasattr(oracle.ref(), "ref_resize"):
        pytest.skip("reference golden not compiled here")
    rng = np.random.default_rng(7)
    # the big rows of the table are covered at a quarter of their size: the golden is a plain double loop
    scale = 4 if row.src_w * row.src_h > 500000 else 1
    sw, sh, dw, dh = row.src_w // scale, row.src_h // scale, row.dst_w // scale, row.dst_h // scale
    im = _image(rng, sw, sh, row.channels, row.dtype)
    got = oracle.resize_plain([im], [(dw, dh)], row.interp, golden_float=True)[0]
    ref = oracle.ref_resize(im, (dw, dh), row.interp)
    assert np.array_equal(got.view(np.uint8), ref.view(np.uint8))


def test_float_linear_without_the_golden_rounding(oracle):
    """The product keeps float32 blends as computed (like the reference's CUDA operator); the golden rounds them."""
    rng = np.random.default_rng(3)
    im = rng.uniform(0.0, 10.0, (9, 11, 3)).astype(np.float32)
    a = oracle.resize_plain([im], [(20, 17)], 1, golden_float=True)[0]
    b = oracle.resize_plain([im], [(20, 17)], 1, golden_float=False)[0]
    tiny = np.finfo(np.float32).tiny  # the golden clamps to [numeric_limits<float>::min(), max()]: zero becomes FLT_MIN
    assert np.all((a == np.rint(a)) | (a == tiny)) and np.abs(a - b).max() <= 0.5
    assert not np.array_equal(a, b)


def test_int16_linear_keeps_the_sign_unlike_the_golden(oracle):
    """The golden rounds |blend| (ResizeUtils.cpp:226); the product follows the reference's CUDA operators, which keep the
    sign of an int16 blend. On non-negative data the two forms agree."""
    neg = np.full((6, 7, 3), -100, np.int16)
    assert np.all(oracle.resize_plain([neg], [(13, 9)], 1, golden_float=False)[0] == -100)
    assert np.all(oracle.resize_plain([neg], [(13, 9)], 1, golden_float=True)[0] == 100)
    rng = np.random.default_rng(4)
    pos = rng.integers(0, 32768, (9, 11, 3)).astype(np.int16)
    assert np.array_equal(oracle.resize_plain([pos], [(20, 17)], 1, golden_float=False)[0],
                          oracle.resize_plain([pos], [(20, 17)], 1, golden_float=True)[0])
