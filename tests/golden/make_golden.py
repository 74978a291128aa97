"""Generates tests/golden/*.npz by running the REFERENCE's own golden functions (oracle/_ref/libref_golden.so,
compiled from the reference tree by oracle/build_oracle.py) on seeded inputs.

Run where the reference tree is available:  python tests/golden/make_golden.py
The fixtures pin the C restatement (and through it the CUDA kernels) on machines without the reference tree.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.dirname(HERE))

from oracle import build_oracle, oracle as O  # noqa: E402
import ref_tables as T  # noqa: E402


def rccr_cases():
    """Small seeded cases covering both interpolations, both layouts, both dtypes, swap, rescale and source cast."""
    rng = np.random.default_rng(1234)
    specs = [
        # (w, h, n), resize, interp, out, crop, scale, offset, manip, planar, dtype, cast
        ((64, 48, 2), (32, 32), 1, (28, 28), (2, 2), 1.0 / 255.0, 0.0, 1, True, np.float32, False),
        ((64, 48, 2), (32, 32), 1, (28, 28), (2, 2), 1.0, 0.0, 0, True, np.float32, True),
        ((37, 29, 3), (50, 41), 1, (50, 41), (0, 0), 1 / 127.5, -1.0, 1, False, np.float32, False),
        ((37, 29, 3), (50, 41), 1, (33, 20), (9, 11), 0.5, 3.0, 0, True, np.uint8, False),
        ((64, 48, 2), (32, 32), 0, (28, 28), (2, 2), 2.0, -255.0, 1, True, np.float32, False),
        ((37, 29, 3), (50, 41), 0, (33, 20), (9, 11), -1.0, 255.0, 1, False, np.uint8, True),
        ((120, 90, 1), (16, 12), 1, (16, 12), (0, 0), 1.0, 0.0, 0, False, np.uint8, True),
    ]
    out = {}
    for i, (s, rs, interp, osz, crop, sc, off, manip, planar, dt, cast) in enumerate(specs):
        w, h, n = s
        src = rng.integers(0, 256, (n, h, w, 3), dtype=np.uint8)
        ref = O.ref_rccr(src, rs, crop, osz, interp, manip, sc, off, cast, dt, planar)
        out[f"rccr{i}_src"] = src
        out[f"rccr{i}_ref"] = ref
        out[f"rccr{i}_par"] = np.array([rs[0], rs[1], interp, osz[0], osz[1], crop[0], crop[1], manip, int(planar),
                                        int(cast)], np.int32)
        out[f"rccr{i}_aff"] = np.array([sc, off], np.float32)
    out["rccr_count"] = np.array(len(specs))
    return out


def cfnr_cases():
    out = {}
    k = 0
    for ri, row in enumerate(T.CFNR_ROWS):
        small = row._replace(images=2, width=min(row.width, 17), height=min(row.height, 19))
        images, rects, flips, base, scale, osz = T.cfnr_case(small, seed=100 + ri)
        for i, im in enumerate(images):
            ref = O.ref_cfnr(im, small.src_planar, rects[i], int(flips[i]), osz, small.dst_dtype, small.dst_planar,
                             small.border, 1.0, base, scale, small.gscale, small.gshift, small.eps, small.flags)
            out[f"cfnr{k}_src"] = im
            out[f"cfnr{k}_ref"] = ref
            out[f"cfnr{k}_par"] = np.array([*rects[i], flips[i], osz[0], osz[1], int(small.src_planar),
                                            int(small.dst_planar), small.border, small.flags], np.int32)
            out[f"cfnr{k}_f"] = np.array([small.gscale, small.gshift, small.eps], np.float32)
            out[f"cfnr{k}_base"] = base
            out[f"cfnr{k}_scale"] = scale
            k += 1
    out["cfnr_count"] = np.array(k)
    return out


def resize_cases():
    """Stand-alone Resize golden (nearest / linear) on small seeded images of every element type and channel count."""
    rng = np.random.default_rng(4321)
    out = {}
    k = 0
    shapes = [((26, 30), (15, 16)), ((11, 13), (22, 26)), ((19, 9), (7, 20)), ((8, 8), (8, 8))]
    for (sw, sh), (dw, dh) in shapes:
        for dt in (np.uint8, np.uint16, np.int16, np.float32):
            for ch in (1, 3, 4):
                for interp in (0, 1):
                    if dt == np.float32:
                        im = rng.uniform(0.0, 300.0, (sh, sw, ch)).astype(np.float32)
                    else:
                        info = np.iinfo(dt)
                        im = rng.integers(info.min, info.max + 1, (sh, sw, ch)).astype(dt)
                    out[f"resize{k}_src"] = im
                    out[f"resize{k}_ref"] = O.ref_resize(im, (dw, dh), interp)
                    out[f"resize{k}_par"] = np.array([dw, dh, interp], np.int32)
                    k += 1
    out["resize_count"] = np.array(k)
    return out


def normalize_cases():
    """Stand-alone Normalize golden on small versions of the reference's table rows (one image each)."""
    out = {}
    for k, row in enumerate(T.NORMALIZE_ROWS):
        small = row._replace(images=1, width=min(row.width, 23), height=min(row.height, 17))
        images, base, scale = T.normalize_case(small, 900 + k)
        out[f"norm{k}_src"] = images[0]
        out[f"norm{k}_base"] = base
        out[f"norm{k}_scale"] = scale
        out[f"norm{k}_par"] = np.array([small.gscale, small.gshift, small.eps, small.flags], np.float32)
        out[f"norm{k}_ref"] = O.ref_normalize(images[0], base, scale, small.gscale, small.gshift, small.eps, small.flags)
    out["norm_count"] = np.array(len(T.NORMALIZE_ROWS))
    return out


def border_cases():
    """Stand-alone CopyMakeBorder golden (tensor form) on small versions of the reference's table rows plus every
    border rule on each element type."""
    out, k = {}, 0
    rng = np.random.default_rng(77)
    rows = [(12, 13, 2, 12, 16, 0, 3, 0, (12, 100, 245, 0), np.uint8, 3), (21, 11, 1, 0, 11, 5, 0, 0, (13, 5, 4, 0), np.uint8, 3),
            (23, 13, 2, 44, 55, 33, 22, 1, (0, 0, 0, 0), np.uint8, 3), (23, 13, 2, 33, 20, 41, 42, 2, (0, 0, 0, 0), np.uint8, 4),
            (23, 13, 2, 100, 85, 53, 62, 3, (0, 0, 0, 0), np.float32, 3), (24, 12, 2, 56, 123, 77, 98, 4, (0, 0, 0, 0), np.float32, 4)]
    for dt in (np.uint16, np.int16, np.int32):
        for border in range(5):
            rows.append((7, 5, 1, 6, 9, 11, 3, border, (1000, 20000, 300, 7), dt, 1 + border % 4))
    for (w, h, n, top, bottom, left, right, border, value, dt, ch) in rows:
        if dt == np.float32:
            src = (rng.integers(0, 256, (n, h, w, ch)) / 255.0).astype(np.float32)
        else:
            info = np.iinfo(dt)
            src = rng.integers(info.min, int(info.max) + 1, (n, h, w, ch)).astype(dt)
        out[f"border{k}_src"] = src
        out[f"border{k}_par"] = np.array([top, bottom, left, right, border], np.int32)
        out[f"border{k}_val"] = np.array(value, np.float32)
        out[f"border{k}_ref"] = O.ref_copy_make_border(src, (w + left + right, h + top + bottom), top, left, border, value)
        k += 1
    out["border_count"] = np.array(k)
    return out


def random_crop_cases():
    """Rectangle sequences of the reference test's GetCropParams (TestOpRandomResizedCrop.cpp:39-93): several seeds and
    parameter sets, image sizes of its table, including a set no random try can satisfy (the central-crop fallback)."""
    out, k = {}, 0
    sizes = [(42, 48), (113, 12), (421, 148), (313, 212), (42, 40), (21, 21), (420, 420), (210, 210), (1920, 1080), (5, 400)] * 4
    for seed in (1, 2, 77, 12345, 4000000000):
        for par in ((0.08, 1.0, 0.75, 4.0 / 3.0), (0.5, 0.9, 0.5, 2.0), (1.0, 1.0, 3.0, 4.0), (0.2, 1.0, 0.8, 1.3)):
            out[f"seq{k}_seed"] = np.array(seed, np.int64)
            out[f"seq{k}_par"] = np.array(par, np.float64)
            out[f"seq{k}_sizes"] = np.array(sizes, np.int32)
            out[f"seq{k}_rects"] = O.ref_random_crop_rects(seed, sizes, *par)
            k += 1
    out["count"] = np.array(k)
    return out


MEAN = (123.675, 116.28, 103.53)
INV_STD = tuple(float(np.float32(1.0) / np.float32(s)) for s in (58.395, 57.12, 57.375))


def fused_cases():
    """The fused passes of the benchmark configurations, scaled down, as CHAINS of the reference's own goldens
    (oracle.ref_resize_then_normalize / ref_crop_resize_flip_normalize / ref_letterbox): what the one-pass entry points
    must reproduce. Kinds: 0 = resize + crop + per-channel normalise (float32 / float16, nearest / linear),
    1 = rectangle + resize + flip + normalise (float16), 2 = letterbox."""
    rng = np.random.default_rng(2468)
    out, k = {}, 0
    for (w, h, n), rs, crop, osz, interp, dt in (((120, 68, 2), (32, 32), (2, 2), (28, 28), 1, np.float32),
                                                 ((120, 68, 2), (48, 48), (4, 4), (40, 40), 1, np.float16),
                                                 ((120, 68, 2), (48, 48), (4, 4), (40, 40), 0, np.float16),
                                                 ((61, 47, 1), (90, 70), (10, 5), (64, 48), 1, np.float32)):
        src = rng.integers(0, 256, (n, h, w, 3), dtype=np.uint8)
        out[f"fused{k}_kind"] = np.array(0)
        out[f"fused{k}_src"] = src
        out[f"fused{k}_par"] = np.array([*rs, *crop, *osz, interp], np.int32)
        out[f"fused{k}_ref"] = O.ref_resize_then_normalize(src, rs, crop, osz, interp, MEAN, INV_STD, dt)
        k += 1
    sizes = [(97, 71), (160, 45), (53, 120)]
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (w, h) in sizes]
    rects = np.array([(5, 7, 80, 60), (0, 0, 160, 45), (20, 30, 30, 41)], np.int32)
    flips = np.array([1, 2, 1], np.int32)
    out[f"fused{k}_kind"] = np.array(1)
    for i, im in enumerate(images):
        out[f"fused{k}_src{i}"] = im
    out[f"fused{k}_rects"], out[f"fused{k}_flips"] = rects, flips
    out[f"fused{k}_par"] = np.array([28, 28], np.int32)
    out[f"fused{k}_ref"] = O.ref_crop_resize_flip_normalize(images, rects, flips, (28, 28), MEAN, INV_STD, np.float16)
    k += 1
    src = rng.integers(0, 256, (2, 54, 96, 3), dtype=np.uint8)  # 96x54 -> 32x18 (factor 3, as 1080p -> 640x360) in 32x32
    out[f"fused{k}_kind"] = np.array(2)
    out[f"fused{k}_src"] = src
    out[f"fused{k}_par"] = np.array([32, 18, 32, 32, 0, 7, 114], np.int32)
    out[f"fused{k}_ref"] = O.ref_letterbox(src, (32, 18), (32, 32), (0, 7), 114, 1.0 / 255.0)
    k += 1
    out["fused_count"] = np.array(k)
    return out


CASES = {"rccr": rccr_cases, "cfnr": cfnr_cases, "resize": resize_cases, "normalize": normalize_cases, "border": border_cases,
         "random_crop": random_crop_cases, "fused": fused_cases}

if __name__ == "__main__":
    assert build_oracle.build_ref() is not None, "reference tree not available"
    for name in (sys.argv[1:] or list(CASES)):  # python tests/golden/make_golden.py [name ...]
        np.savez_compressed(os.path.join(HERE, f"{name}_golden.npz"), **CASES[name]())
    print("written", [f for f in os.listdir(HERE) if f.endswith(".npz")])
