"""Worker of tests/test_real_nvcv_gpu.py (run as a child process, one per library): drives the reference's header-only C++
wrappers, its real libnvcv_types tensors and image batches, against either the B200 library or the reference's own
operators, and compares every result with the CPU oracle. Prints one JSON object {case: "ok" | message}.

A child process, because the B200 library binds the nvcv* functions it finds first, once per process, and the other GPU
tests use an object-model test double.
"""
import json
import os
import sys
import traceback

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)

import ref_tables as T  # noqa: E402
from oracle import oracle as O  # noqa: E402
from oracle import ref_ops as R  # noqa: E402

NOT_COMPATIBLE = 9  # NVCV_ERROR_NOT_COMPATIBLE, nvcv/Status.h


def compare(got, want, exact_float, what):
    """B200 library: nearest bit-exact, uint8 within 1, float32 within 1e-5 (observed: equality). Reference operators:
    their own tests' bounds (+-1, 1e-4), because their kernels contract multiply-adds."""
    assert got.shape == want.shape and got.dtype == want.dtype, what
    if got.dtype == np.float32:
        d = float(np.abs(got.astype(np.float64) - want).max())
        assert d <= (1e-5 if exact_float else 1e-4 * max(1.0, float(np.abs(want).max()))), f"{what}: float diff {d}"
    else:
        d = int(np.abs(got.astype(np.int64) - want.astype(np.int64)).max())
        assert d <= 1, f"{what}: integer diff {d}"


def main(which: str) -> int:
    L = R.load(which)
    assert L is not None, "harness not built"
    assert L.h_which().decode() == {"b200": "b200", "ref": "reference"}[which]
    b200 = which == "b200"
    results = {}

    def run(name, fn):
        try:
            fn()
            results[name] = "ok"
        except Exception:  # noqa: BLE001 - reported to the parent
            results[name] = traceback.format_exc(limit=3)

    for idx in (0, 7, 10, 24, 30, 41, 45, 52, 57, 61):
        r = T.RCCR_ROWS[idx]

        def tensor_case(r=r, idx=idx):
            w, h, n = r.src
            src = np.random.default_rng(idx).integers(0, 256, (min(n, 2), h, w, 3), dtype=np.uint8)
            spec = O.ResizeSpec(resize=r.resize, crop=r.crop, out_size=r.out, interp=r.interp, src_cast=r.src_cast,
                                manip=r.manip, scale=r.scale, offset=r.offset)
            want = O.resize_crop(list(src), spec, r.dtype, r.planar, nthreads=4)
            got = R.rccr_tensor(L, src, r.resize, r.crop, r.out, r.interp, r.manip, r.scale, r.offset, r.src_cast, r.dtype,
                                r.planar)
            compare(got, want, b200, f"tensor row {idx}")
            if b200:
                assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"tensor row {idx}: expected bit-equality"
        run(f"rccr_tensor_{idx}", tensor_case)

    for idx, late in ((3, 0), (9, 1), (31, 0), (44, 2), (57, 1)):
        r = T.RCCR_ROWS[idx]

        def varshape_case(r=r, idx=idx, late=late):
            w, h, _ = r.src
            rng = np.random.default_rng(100 + idx)
            images = [rng.integers(0, 256, (int(h * s), int(w * s), 3), dtype=np.uint8) for s in (0.8, 1.0, 1.2, 0.9)]
            spec = O.ResizeSpec(resize=r.resize, crop=r.crop, out_size=r.out, interp=r.interp, src_cast=r.src_cast,
                                manip=r.manip, scale=r.scale, offset=r.offset)
            want = O.resize_crop(images, spec, r.dtype, r.planar, nthreads=4)
            got = R.rccr_varshape(L, images, r.resize, r.crop, r.out, r.interp, r.manip, r.scale, r.offset, r.src_cast, r.dtype,
                                  r.planar, push_late=late)
            compare(got, want, b200, f"var-shape row {idx}")
            if b200:
                assert np.array_equal(got.view(np.uint8), want.view(np.uint8)), f"var-shape row {idx}: expected bit-equality"
        run(f"rccr_varshape_{idx}_late{late}", varshape_case)

    for idx, row in enumerate(T.CFNR_ROWS):
        def cfnr_case(row=row, idx=idx):
            images, rects, flips, base, scale, osz = T.cfnr_case(row, seed=77 + idx)
            want = O.crop_flip_normalize(images, row.src_planar, rects, flips, osz, row.dst_dtype, row.dst_planar, row.border, 1.0,
                                         base, scale, row.gscale, row.gshift, row.eps, row.flags)
            got = R.cfnr(L, images, row.src_planar, rects, flips, osz, row.dst_dtype, row.dst_planar, row.border, 1.0, base, scale,
                         row.gscale, row.gshift, row.eps, row.flags)
            compare(got, want, b200, f"cfnr row {idx}")
        run(f"cfnr_{idx}", cfnr_case)

    def negative():
        src = np.zeros((1, 32, 32, 3), np.uint8)
        try:
            R.rccr_tensor(L, src, (16, 16), (0, 0), (16, 16), 1, 0, 1.0, 0.0, True, np.float16, True)
        except R.HarnessError as e:
            assert e.status == NOT_COMPATIBLE, f"float16 output: status {e.status} ({e})"
        else:
            raise AssertionError("float16 output was accepted by the stock entry point")
        try:  # crop window outside the resized image: INVALID_ARGUMENT (2)
            R.rccr_tensor(L, src, (16, 16), (8, 8), (16, 16), 1, 0, 1.0, 0.0, True, np.float32, True)
        except R.HarnessError as e:
            assert e.status == 2, f"bad crop: status {e.status} ({e})"
        else:
            raise AssertionError("a crop outside the resized image was accepted")
    run("negative_status_through_the_wrappers", negative)

    print("RESULTS " + json.dumps(results))
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
