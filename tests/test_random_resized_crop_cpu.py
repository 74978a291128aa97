"""CPU: the rectangle generator of RandomResizedCrop (host code of the library, no GPU needed) against the reference test's
GetCropParams (compiled into oracle/_ref where the reference tree is present) and against the committed sequences of that
function; the resized-crop restatement against the reference golden called with crop arguments."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
SIZES = [(42, 48), (113, 12), (421, 148), (313, 212), (1920, 1080), (21, 21), (5, 400)] * 3


@pytest.fixture(scope="module")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.mark.parametrize("seed", [1, 2, 7, 12345, 4000000000])
def test_generator_matches_the_reference_function(pkg, oracle, seed):
    if oracle.ref() is None or not hasattr(oracle.ref(), "ref_random_crop_rects"):
        pytest.skip("reference golden not compiled here")
    for par in ((0.08, 1.0, 0.75, 4.0 / 3.0), (0.5, 0.9, 0.5, 2.0), (1.0, 1.0, 3.0, 4.0), (0.2, 1.0, 0.8, 1.3)):
        got = np.array(pkg.random_crop_rects(SIZES, *par, seed=seed), np.int32)
        assert np.array_equal(got, oracle.ref_random_crop_rects(seed, SIZES, *par)), par


def test_generator_matches_the_committed_reference_sequences(pkg):
    g = np.load(os.path.join(HERE, "golden", "random_crop_golden.npz"))
    assert int(g["count"]) == 20
    for k in range(int(g["count"])):
        sizes = [tuple(int(v) for v in s) for s in g[f"seq{k}_sizes"]]
        got = np.array(pkg.random_crop_rects(sizes, *[float(v) for v in g[f"seq{k}_par"]], seed=int(g[f"seq{k}_seed"])), np.int32)
        assert np.array_equal(got, g[f"seq{k}_rects"]), f"sequence {k}"


def test_generator_properties(pkg):
    """Rectangles lie inside their image; scale and ratio limits hold up to the rounding of the side lengths; ratio limits no
    random try can meet give the central crop; bad limits are refused; seed 0 gives a different sequence each time."""
    rects = pkg.random_crop_rects([(640, 480)] * 200, 0.25, 0.5, 0.9, 1.1, seed=5)
    for (l, t, w, h) in rects:
        assert 0 <= l and 0 <= t and l + w <= 640 and t + h <= 480 and w > 0 and h > 0
        assert 0.25 * 640 * 480 * 0.98 <= w * h <= 0.5 * 640 * 480 * 1.02
        assert 0.88 <= w / h <= 1.12
    assert pkg.random_crop_rects([(100, 400)], 1.0, 1.0, 3.0, 4.0, seed=9) == [(0, 183, 100, 33)]   # cols / minRatio high
    assert pkg.random_crop_rects([(400, 100)], 1.0, 1.0, 0.2, 0.25, seed=9) == [(187, 0, 25, 100)]  # rows * maxRatio wide
    with pytest.raises(pkg.ops.Error):
        pkg.random_crop_rects([(10, 10)], 1.0, 0.5)
    with pytest.raises(pkg.ops.Error):
        pkg.random_crop_rects([(10, 10)], 0.5, 1.0, 2.0, 1.0)
    a = pkg.random_crop_rects([(1000, 1000)] * 8, seed=0)
    b = pkg.random_crop_rects([(1000, 1000)] * 8, seed=0)
    assert a != b


@pytest.mark.parametrize("dt", [np.uint8, np.uint16, np.int16, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("interp", [0, 1])
def test_resized_crop_restatement_matches_the_reference_golden(oracle, dt, interp):
    if oracle.ref() is None or not hasattr(oracle.ref(), "ref_resized_crop"):
        pytest.skip("reference golden not compiled here")
    rng = np.random.default_rng(interp)
    for ch in (1, 3, 4):
        for (sw, sh, dw, dh, rect) in [(42, 48, 23, 24, (5, 7, 30, 20)), (113, 12, 12, 36, (0, 0, 113, 12)),
                                       (21, 21, 42, 42, (3, 2, 10, 17)), (50, 40, 20, 20, (49, 39, 1, 1)),
                                       (50, 40, 33, 17, (10, 10, 40, 30))]:
            if dt == np.float32:
                im = rng.uniform(0, 300, (sh, sw, ch)).astype(dt)
            else:
                info = np.iinfo(dt)
                im = rng.integers(info.min, int(info.max) + 1, (sh, sw, ch)).astype(dt)
            got = oracle.resize_plain([im], [(dw, dh)], interp, golden_float=True, rects=[rect])[0]
            ref = oracle.ref_resize(im, (dw, dh), interp, rect)
            assert np.array_equal(got.view(np.uint8), ref.view(np.uint8)), (ch, sw, sh, dw, dh, rect)
