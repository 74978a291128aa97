"""CPU: the stand-alone Normalize restatement (oracle/normalize_oracle.c) against the reference's own golden function
(compiled into oracle/_ref where the reference tree is present) over the reference's test table."""
import os

import numpy as np
import pytest

import ref_tables as T

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.mark.parametrize("idx", range(len(T.NORMALIZE_ROWS)))
def test_restatement_matches_the_reference_golden_on_its_test_table(oracle, idx):
    if oracle.ref() is None or not hasattr(oracle.ref(), "ref_normalize"):
        pytest.skip("reference golden not compiled here")
    row = T.NORMALIZE_ROWS[idx]
    images, base, scale = T.normalize_case(row, 300 + idx)
    got = oracle.normalize(images, base, scale, None, row.gscale, row.gshift, row.eps, row.flags)
    for i, im in enumerate(images):
        b = base if row.scalar_base else base[i:i + 1]
        s = scale if row.scalar_scale else scale[i:i + 1]
        ref = oracle.ref_normalize(im, b, s, row.gscale, row.gshift, row.eps, row.flags)
        assert np.array_equal(got[i], ref), f"image {i}"


def test_restatement_matches_the_committed_reference_outputs(oracle):
    g = np.load(os.path.join(HERE, "golden", "normalize_golden.npz"))
    n = int(g["norm_count"])
    assert n == len(T.NORMALIZE_ROWS)
    for k in range(n):
        gs, sh, eps, flags = g[f"norm{k}_par"]
        got = oracle.normalize([g[f"norm{k}_src"]], g[f"norm{k}_base"], g[f"norm{k}_scale"], None, float(gs), float(sh),
                               float(eps), int(flags))[0]
        assert np.array_equal(got, g[f"norm{k}_ref"]), f"fixture {k}"


def test_known_values(oracle):
    """Hand-checked values: round half to even, clamping, the standard-deviation form."""
    im = np.array([[[0, 1, 2, 255]]], dtype=np.uint8)
    one = np.ones((1, 1, 1, 1), np.float32)
    out = oracle.normalize([im], one * 0, one * 0.5)[0]  # v * 0.5: 0, 0.5 -> 0, 1, 127.5 -> 128
    assert out.tolist() == [[[0, 0, 1, 128]]]
    out = oracle.normalize([im], one * 1, one * 2.0, shift=-1.0)[0]  # (v-1)*2-1: -3 -> 0, -1 -> 0, 1, 507 -> 255
    assert out.tolist() == [[[0, 0, 1, 255]]]
    out = oracle.normalize([im], one * 0, one * 3.0, np.float32, epsilon=16.0, flags=1)[0]  # v / sqrt(9 + 16) = v / 5
    assert np.allclose(out, im.astype(np.float32) * np.float32(0.2))
