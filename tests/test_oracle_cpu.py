"""CPU: the C restatement against (a) fixtures produced by the reference's own golden code, (b) that golden code
itself over the reference's test tables when it could be compiled here, (c) hand-computable cases."""
import os

import numpy as np
import pytest

import ref_tables as T

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _same(a, b):
    return a.shape == b.shape and np.array_equal(a.view(np.uint8), b.view(np.uint8))


def test_rccr_fixtures(oracle):
    z = np.load(os.path.join(GOLDEN, "rccr_golden.npz"))
    for i in range(int(z["rccr_count"])):
        rw, rh, interp, ow, oh, cx, cy, manip, planar, cast = (int(v) for v in z[f"rccr{i}_par"])
        sc, off = (float(v) for v in z[f"rccr{i}_aff"])
        ref = z[f"rccr{i}_ref"]
        spec = oracle.ResizeSpec(resize=(rw, rh), crop=(cx, cy), out_size=(ow, oh), interp=interp, src_cast=bool(cast),
                                 manip=manip, scale=sc, offset=off)
        got = oracle.resize_crop(list(z[f"rccr{i}_src"]), spec, ref.dtype, bool(planar))
        assert _same(got, ref), f"fixture {i}"


def test_cfnr_fixtures(oracle):
    z = np.load(os.path.join(GOLDEN, "cfnr_golden.npz"))
    for k in range(int(z["cfnr_count"])):
        x, y, w, h, flip, ow, oh, sp, dp, border, flags = (int(v) for v in z[f"cfnr{k}_par"])
        gs, sh, eps = (float(v) for v in z[f"cfnr{k}_f"])
        ref = z[f"cfnr{k}_ref"]
        got = oracle.crop_flip_normalize([z[f"cfnr{k}_src"]], bool(sp), np.array([[x, y, w, h]]), np.array([flip]),
                                         (ow, oh), ref.dtype, bool(dp), border, 1.0, z[f"cfnr{k}_base"],
                                         z[f"cfnr{k}_scale"], gs, sh, eps, flags)[0]
        assert _same(got, ref), f"fixture {k}"


@pytest.mark.parametrize("idx", range(len(T.RCCR_ROWS)))
def test_rccr_reference_table(oracle, idx):
    """Every positive row of the reference's test table, on its ramp input: restatement == reference golden."""
    if oracle.ref() is None:
        pytest.skip("reference golden not compiled on this machine")
    r = T.RCCR_ROWS[idx]
    w, h, n = r.src
    n = min(n, 2)  # every image of a batch holds the same ramp
    src = T.ramp_batch(n, h, w)
    ref = oracle.ref_rccr(src, r.resize, r.crop, r.out, r.interp, r.manip, r.scale, r.offset, r.src_cast, r.dtype,
                          r.planar)
    spec = oracle.ResizeSpec(resize=r.resize, crop=r.crop, out_size=r.out, interp=r.interp, src_cast=r.src_cast,
                             manip=r.manip, scale=r.scale, offset=r.offset)
    got = oracle.resize_crop(list(src), spec, r.dtype, r.planar, nthreads=4)
    assert _same(got, ref)


@pytest.mark.parametrize("idx", range(len(T.CFNR_ROWS)))
def test_cfnr_reference_table(oracle, idx):
    if oracle.ref() is None:
        pytest.skip("reference golden not compiled on this machine")
    row = T.CFNR_ROWS[idx]
    images, rects, flips, base, scale, osz = T.cfnr_case(row, seed=idx)
    got = oracle.crop_flip_normalize(images, row.src_planar, rects, flips, osz, row.dst_dtype, row.dst_planar,
                                     row.border, 1.0, base, scale, row.gscale, row.gshift, row.eps, row.flags, nthreads=2)
    for i, im in enumerate(images):
        ref = oracle.ref_cfnr(im, row.src_planar, rects[i], int(flips[i]), osz, row.dst_dtype, row.dst_planar,
                              row.border, 1.0, base, scale, row.gscale, row.gshift, row.eps, row.flags)
        assert _same(got[i], ref), f"image {i}"


def test_saturate_cast_matches_reference(oracle):
    if oracle.ref() is None:
        pytest.skip("reference golden not compiled on this machine")
    R, L = oracle.ref(), oracle.lib()
    rng = np.random.default_rng(7)
    vals = np.concatenate([np.arange(-300, 600, 0.25, dtype=np.float32),
                           rng.uniform(-70000, 70000, 4000).astype(np.float32)])
    for v in vals:
        v = float(v)
        assert R.ref_sat_u8_f32(v) == L.oracle_sat_u8(v)
        assert R.ref_sat_s16_f32(v) == L.oracle_sat_s16(v)
        assert R.ref_sat_s32_f32(v) == L.oracle_sat_s32(v)


def test_round_half_to_even(oracle):
    L = oracle.lib()
    assert [L.oracle_sat_u8(v) for v in (0.5, 1.5, 2.5, 254.5, 255.5, 300.0, -0.5, -7.0)] == [0, 2, 2, 254, 255, 255, 0, 0]


def test_f16_conversion_is_rne(oracle):
    rng = np.random.default_rng(3)
    vals = rng.uniform(-70000, 70000, 2000).astype(np.float32)
    got = np.array([oracle.lib().oracle_f32_to_f16_bits(float(v)) for v in vals], np.uint16)
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    assert np.array_equal(got, want)


def test_identity_resize_is_a_copy(oracle):
    rng = np.random.default_rng(0)
    src = rng.integers(0, 256, (2, 9, 11, 3), dtype=np.uint8)
    for interp in (0, 1):
        spec = oracle.ResizeSpec(resize=(11, 9), out_size=(11, 9), interp=interp, src_cast=False)
        out = oracle.resize_crop(list(src), spec, np.uint8, planar=False)
        assert np.array_equal(out, src)


def test_nearest_2x_upsample_and_reverse(oracle):
    src = np.arange(2 * 3 * 3, dtype=np.uint8).reshape(1, 2, 3, 3)
    spec = oracle.ResizeSpec(resize=(6, 4), out_size=(6, 4), interp=0, manip=1)
    out = oracle.resize_crop(list(src), spec, np.uint8, planar=False)[0]
    want = np.repeat(np.repeat(src[0], 2, axis=0), 2, axis=1)[..., ::-1]
    assert np.array_equal(out, want)


def test_flip_codes_and_zero_fill(oracle):
    img = np.arange(4 * 5, dtype=np.uint8).reshape(4, 5, 1)
    one = np.array([1.0], np.float32)
    zero = np.array([0.0], np.float32)
    for code, want in ((1, img[:, ::-1]), (0, img[::-1]), (-1, img[::-1, ::-1]), (2, img)):
        out = oracle.crop_flip_normalize([img], False, np.array([[0, 0, 5, 4]]), np.array([code]), (6, 5), np.uint8,
                                         False, 0, 0.0, zero, one)[0]
        assert np.array_equal(out[:4, :5], want)
        assert not out[4:].any() and not out[:, 5:].any()


@pytest.mark.parametrize("border,want", [
    (0, [9, 9, 0, 1, 2, 3, 9, 9]),  # constant 9
    (1, [0, 0, 0, 1, 2, 3, 3, 3]),  # replicate
    (2, [1, 0, 0, 1, 2, 3, 3, 2]),  # reflect (edge duplicated)
    (3, [2, 3, 0, 1, 2, 3, 0, 1]),  # wrap
    (4, [2, 1, 0, 1, 2, 3, 2, 1]),  # reflect101
])
def test_border_rules(oracle, border, want):
    img = np.arange(4, dtype=np.uint8).reshape(1, 4, 1)
    out = oracle.crop_flip_normalize([img], False, np.array([[-2, 0, 8, 1]]), np.array([2]), (8, 1), np.uint8, False,
                                     border, 9.0, np.array([0.0], np.float32), np.array([1.0], np.float32))[0]
    assert out[0, :, 0].tolist() == want


def test_threads_do_not_change_results(oracle):
    rng = np.random.default_rng(5)
    src = rng.integers(0, 256, (3, 40, 50, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(24, 20), crop=(2, 1), out_size=(20, 18), interp=1, src_cast=False,
                             base=(1.0, 2.0, 3.0), mul=(0.5, 0.25, 0.125))
    a = oracle.resize_crop(list(src), spec, np.float32, True, nthreads=1)
    b = oracle.resize_crop(list(src), spec, np.float32, True, nthreads=7)
    assert np.array_equal(a, b)


def test_algorithmic_bytes_of_the_north_star_config(oracle):
    """1080p -> 256x256 linear -> centre 224x224: 448 source rows of 5056 sector-granular bytes each."""
    spec = oracle.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=1)
    assert oracle.resize_source_bytes(1920, 1080, 1920 * 3, spec) == 2265088


# ------------------------------------------------------------------------------------------------ fused passes vs chains

from ref_tables import INV_STD, MEAN, fused_fixture_cases  # noqa: E402


def restated_fused(oracle, kind, inputs, par, dtype):
    """The restatement's one-pass result for a fixture case."""
    if kind == 0:
        rw, rh, cx, cy, ow, oh, interp = (int(v) for v in par)
        spec = oracle.ResizeSpec(resize=(rw, rh), crop=(cx, cy), out_size=(ow, oh), interp=interp, src_cast=False, base=MEAN,
                                 mul=INV_STD)
        return oracle.resize_crop(list(inputs), spec, dtype, True)
    if kind == 1:
        images, rects, flips = inputs
        ow, oh = (int(v) for v in par)
        spec = oracle.ResizeSpec(resize=(ow, oh), out_size=(ow, oh), interp=1, src_cast=True, base=MEAN, mul=INV_STD)
        return oracle.resize_crop(images, spec, dtype, True, roi=rects, flip=flips)
    rw, rh, cw, ch, dx, dy, pad = (int(v) for v in par)
    spec = oracle.ResizeSpec(resize=(rw, rh), out_size=(rw, rh), interp=1, src_cast=True, manip=1, scale=1.0 / 255.0,
                             canvas=(cw, ch), dst_pos=(dx, dy), pad_value=float(pad))
    return oracle.resize_crop(list(inputs), spec, dtype, True)


def test_fused_passes_equal_chains_of_the_reference_goldens_fixtures(oracle):
    """Per-channel affine in the resize path, float16 store, rectangle + flip, letterbox: the restatement's one pass equals,
    bit for bit, the committed outputs of chains of the reference's own golden functions."""
    count = 0
    for k, kind, inputs, par, ref in fused_fixture_cases():
        got = restated_fused(oracle, kind, inputs, par, ref.dtype)
        assert _same(got, ref), f"fixture {k} (kind {kind})"
        count += 1
    assert count == 6


def test_fused_passes_equal_chains_of_the_reference_goldens_at_config_shapes(oracle):
    """The same on the benchmark configurations' real image sizes (one or two images each), with the chains computed here
    by the reference's compiled goldens."""
    if oracle.ref() is None:
        pytest.skip("reference golden not compiled on this machine")
    rng = np.random.default_rng(1234)
    src = rng.integers(0, 256, (1, 1080, 1920, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=1, src_cast=False, base=MEAN,
                             mul=INV_STD)
    assert _same(oracle.resize_crop(list(src), spec, np.float32, True, nthreads=4),
                 oracle.ref_resize_then_normalize(src, (256, 256), (16, 16), (224, 224), 1, MEAN, INV_STD)), "config 2"
    spec = oracle.ResizeSpec(resize=(640, 360), out_size=(640, 360), interp=1, src_cast=True, manip=1, scale=1.0 / 255.0,
                             canvas=(640, 640), dst_pos=(0, 140), pad_value=114.0)
    assert _same(oracle.resize_crop(list(src), spec, np.float32, True, nthreads=4),
                 oracle.ref_letterbox(src, (640, 360), (640, 640), (0, 140), 114, 1.0 / 255.0)), "config 4"
    big = rng.integers(0, 256, (1, 2160, 3840, 3), dtype=np.uint8)
    for interp in (0, 1):
        spec = oracle.ResizeSpec(resize=(512, 512), crop=(32, 32), out_size=(448, 448), interp=interp, src_cast=False,
                                 base=MEAN, mul=INV_STD)
        assert _same(oracle.resize_crop(list(big), spec, np.float16, True, nthreads=4),
                     oracle.ref_resize_then_normalize(big, (512, 512), (32, 32), (448, 448), interp, MEAN, INV_STD,
                                                      np.float16)), f"config 5 interp {interp}"
    images = [big[0, :1500, :2900], src[0]]
    rects = np.array([(100, 200, 1700, 1290), (480, 0, 960, 1080)], np.int32)
    flips = np.array([1, 2], np.int32)
    spec = oracle.ResizeSpec(resize=(224, 224), out_size=(224, 224), interp=1, src_cast=True, base=MEAN, mul=INV_STD)
    assert _same(oracle.resize_crop(images, spec, np.float16, True, roi=rects, flip=flips, nthreads=4),
                 oracle.ref_crop_resize_flip_normalize(images, rects, flips, (224, 224), MEAN, INV_STD, np.float16)), "config 3"
