"""CPU: the stand-alone CopyMakeBorder restatement (oracle/preproc_oracle.c: oracle_copy_make_border) against the
reference's own golden function (compiled into oracle/_ref where the reference tree is present), against the committed
outputs of that function, and on hand-checked values."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("dt", [np.uint8, np.uint16, np.int16, np.int32, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("border", range(5))
def test_restatement_matches_the_reference_golden(oracle, dt, border):
    if oracle.ref() is None or not hasattr(oracle.ref(), "ref_copy_make_border"):
        pytest.skip("reference golden not compiled here")
    rng = np.random.default_rng(border)
    for ch in (1, 3, 4):
        for (sw, sh, dw, dh, top, left) in [(9, 7, 20, 15, 3, 5), (5, 5, 5, 5, 0, 0), (4, 3, 30, 29, 13, 11), (1, 1, 7, 7, 3, 3)]:
            if dt == np.float32:
                b = rng.uniform(-100, 100, (2, sh, sw, ch)).astype(dt)
            else:
                info = np.iinfo(dt)
                b = rng.integers(info.min, int(info.max) + 1, (2, sh, sw, ch)).astype(dt)
            value = (12.7, 200.2, 3.0, 77.9)
            got = np.stack(oracle.copy_make_border(list(b), [(dw, dh)] * 2, top, left, border, value))
            ref = oracle.ref_copy_make_border(b, (dw, dh), top, left, border, value)
            assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), (ch, sw, sh, dw, dh)


def test_restatement_matches_the_committed_reference_outputs(oracle):
    g = np.load(os.path.join(HERE, "golden", "border_golden.npz"))
    n = int(g["border_count"])
    assert n >= 20
    for k in range(n):
        src = g[f"border{k}_src"]
        top, bottom, left, right, border = (int(v) for v in g[f"border{k}_par"])
        size = (src.shape[2] + left + right, src.shape[1] + top + bottom)
        got = np.stack(oracle.copy_make_border(list(src), [size] * len(src), top, left, border, g[f"border{k}_val"]))
        assert np.array_equal(got.view(np.uint8), g[f"border{k}_ref"].view(np.uint8)), f"fixture {k}"


def test_known_values(oracle):
    """A 1 x 3 row [1 2 3] extended by 4 on the left and 3 on the right, by each rule (the textbook patterns)."""
    row = np.array([[[1], [2], [3]]], np.uint8)
    want = {0: [9, 9, 9, 9, 1, 2, 3, 9, 9, 9],   # constant
            1: [1, 1, 1, 1, 1, 2, 3, 3, 3, 3],   # replicate      aaaa|abc|ccc
            2: [3, 3, 2, 1, 1, 2, 3, 3, 2, 1],   # reflect        ccba|abc|cba
            3: [3, 1, 2, 3, 1, 2, 3, 1, 2, 3],   # wrap           cabc|abc|abc
            4: [1, 2, 3, 2, 1, 2, 3, 2, 1, 2]}   # reflect-101    abcb|abc|bab
    for border, pattern in want.items():
        got = oracle.copy_make_border([row], [(10, 1)], 0, 4, border, (9.9,))[0]
        assert got[0, :, 0].tolist() == pattern, border
    # per-image offsets and sizes; the fraction of the border value is dropped, out-of-range values clamp
    a, b = np.full((2, 2, 1), 5, np.int16), np.full((1, 1, 1), 7, np.int16)
    out = oracle.copy_make_border([a, b], [(3, 3), (2, 4)], np.array([1, 3]), np.array([0, 1]), 0, (-40000.5,))
    assert out[0][:, :, 0].tolist() == [[-32768] * 3, [5, 5, -32768], [5, 5, -32768]]
    assert out[1][:, :, 0].tolist() == [[-32768, -32768]] * 3 + [[-32768, 7]]
