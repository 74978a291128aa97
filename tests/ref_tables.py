"""Parameter tables of the reference's own system tests for the two operators, restated as data.

ResizeCropConvertReformat: the 63 positive rows and the negative rows of
tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:232-329 and :574-603.
CropFlipNormalizeReformat: the 18 rows of tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp:416-453.

Only the numbers are kept; image formats are reduced to what the operators look at
(element type, planar or interleaved, channel count, and whether source and destination order differ).
"""
from __future__ import annotations

from typing import NamedTuple

import os

import numpy as np

NEAREST, LINEAR = 0, 1


class RccrRow(NamedTuple):
    src: tuple  # (w, h, n)
    resize: tuple  # (w, h)
    interp: int
    out: tuple  # (w, h)
    crop: tuple  # (x, y)
    scale: float
    offset: float
    manip: int  # 1 when source and destination channel order differ (RGB <-> BGR)
    planar: bool  # destination layout: planar (NCHW) or interleaved (NHWC)
    dtype: type
    src_cast: bool


_S1 = ((313, 212, 4), (412, 336), (412, 336), (0, 0))
_S2 = ((1280, 960, 3), (300, 225), (250, 200), (15, 16))
_SMALL = [
    ((8, 8, 1), (8, 8), (6, 6), (1, 1)),
    ((8, 8, 1), (16, 16), (12, 12), (2, 2)),
    ((42, 48, 1), (23, 24), (15, 13), (0, 0)),
    ((42, 40, 3), (21, 20), (17, 13), (1, 1)),
    ((21, 21, 5), (42, 42), (32, 32), (10, 10)),
    ((113, 12, 7), (12, 36), (7, 13), (3, 11)),
    ((17, 151, 7), (48, 16), (32, 16), (4, 0)),
    _S1,
    ((1080, 1920, 13), (800, 600), (640, 480), (101, 64)),
    _S2,
]


def _row(shape, interp, scale, offset, manip, planar, dtype, cast=False):
    s, r, o, c = shape
    return RccrRow(s, r, interp, o, c, scale, offset, manip, planar, dtype, cast)


def _rccr_rows():
    f32, u8 = np.float32, np.uint8
    rows = []
    # 0-11: RGB -> BGR planar, linear
    rows += [_row(s, LINEAR, 1, 0, 1, True, f32) for s in _SMALL]
    rows += [_row(s, LINEAR, 1, 0, 1, True, u8) for s in (_S1, _S2)]
    # 12-15: RGB -> RGB planar; 16-19: BGR -> RGB planar; 20-23: BGR -> BGR planar
    for manip in (0, 1, 0):
        rows += [_row(s, LINEAR, 1, 0, manip, True, f32) for s in (_S1, _S2)]
        rows += [_row(s, LINEAR, 1, 0, manip, True, u8) for s in (_S1, _S2)]
    # 24-31: RGB -> BGR interleaved
    rows += [_row(s, LINEAR, 1, 0, 1, False, f32) for s in (_SMALL[0], _SMALL[1], _SMALL[5], _SMALL[6], _S1, _S2)]
    rows += [_row(s, LINEAR, 1, 0, 1, False, u8) for s in (_S1, _S2)]
    # 32-39: RGB -> RGB interleaved (the table lists this group twice)
    for _ in range(2):
        rows += [_row(s, LINEAR, 1, 0, 0, False, f32) for s in (_S1, _S2)]
        rows += [_row(s, LINEAR, 1, 0, 0, False, u8) for s in (_S1, _S2)]
    # 40-47: nearest, RGB -> BGR planar
    nn_shapes = [_SMALL[0], ((8, 8, 5), (16, 16), (12, 12), (2, 2)), _SMALL[2], _S1, _SMALL[8], _S2]
    rows += [_row(s, NEAREST, 1, 0, 1, True, f32) for s in nn_shapes]
    rows += [_row(s, NEAREST, 1, 0, 1, True, u8) for s in (_S1, _S2)]
    # 48-51: nearest, BGR -> RGB planar
    rows += [_row(s, NEAREST, 1, 0, 1, True, f32) for s in (_S1, _S2)]
    rows += [_row(s, NEAREST, 1, 0, 1, True, u8) for s in (_S1, _S2)]
    # 52-56: rescaling
    rows.append(_row(_S1, LINEAR, 1 / 127.5, -1, 1, True, f32))
    rows.append(_row(_S2, NEAREST, 2, -255, 1, True, f32))
    rows.append(_row(_S2, NEAREST, -1, 255, 1, False, u8))
    rows.append(_row(_S1, LINEAR, 0.5, 0, 1, True, u8))
    rows.append(_row(_S2, NEAREST, 2, 0, 1, True, u8))
    # 57-62: source cast
    rows.append(_row(((353, 450, 3), (256, 256), (224, 224), (16, 16)), LINEAR, 1, 0, 1, True, f32, True))
    rows.append(_row(_S1, LINEAR, 1 / 127.5, -1, 1, True, f32, True))
    rows.append(_row(_S2, NEAREST, 2, -255, 1, True, f32, True))
    rows.append(_row(_S2, NEAREST, -1, 255, 1, False, u8, True))
    rows.append(_row(_S1, LINEAR, 1, 0, 1, True, u8, True))
    rows.append(_row(_S2, NEAREST, 1, 0, 1, True, u8, True))
    return rows


RCCR_ROWS = _rccr_rows()
assert len(RCCR_ROWS) == 63


def ramp_batch(n: int, h: int, w: int) -> np.ndarray:
    """The reference test's deterministic input: value (x + y + c) & 255 (TestOp...Reformat.cpp:198-221)."""
    y, x, c = np.meshgrid(np.arange(h), np.arange(w), np.arange(3), indexing="ij")
    return np.broadcast_to(((x + y + c) & 255).astype(np.uint8), (n, h, w, 3)).copy()


# Negative rows: source is 32x32, resize to `resize`, crop size = out.  Status names are NVCVStatus members.
class RccrNegRow(NamedTuple):
    interp: int
    n_in: int
    n_out: int
    src_channels: int
    src_dtype: str
    src_planar: bool
    dst_channels: int
    dst_dtype: str
    out: tuple
    crop: tuple
    resize: tuple
    status: str


RCCR_NEGATIVE_ROWS = [
    RccrNegRow(2, 2, 2, 3, "u8", False, 3, "u8", (4, 4), (0, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),  # cubic
    RccrNegRow(3, 2, 2, 3, "u8", False, 3, "u8", (4, 4), (0, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),  # area
    RccrNegRow(4, 2, 2, 3, "u8", False, 3, "u8", (4, 4), (0, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),  # lanczos
    RccrNegRow(1, 1, 2, 3, "u8", False, 3, "u8", (4, 4), (0, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),  # batch sizes
    RccrNegRow(1, 2, 1, 3, "u8", False, 3, "u8", (4, 4), (0, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),
    RccrNegRow(1, 2, 2, 3, "u8", False, 4, "u8", (4, 4), (0, 0), (16, 16), "ERROR_NOT_COMPATIBLE"),  # channel mismatch
    RccrNegRow(1, 2, 2, 4, "u8", False, 4, "u8", (4, 4), (0, 0), (16, 16), "ERROR_NOT_COMPATIBLE"),  # not 3 channels
    RccrNegRow(1, 2, 2, 3, "f32", False, 3, "u8", (4, 4), (0, 0), (16, 16), "ERROR_NOT_COMPATIBLE"),  # input not uchar
    RccrNegRow(1, 2, 2, 3, "u8", False, 3, "f16", (4, 4), (0, 0), (16, 16), "ERROR_NOT_COMPATIBLE"),  # output f16
    RccrNegRow(1, 2, 2, 3, "u8", False, 3, "u8", (4, 4), (-1, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),  # crop range
    RccrNegRow(1, 2, 2, 3, "u8", False, 3, "u8", (4, 4), (0, -1), (16, 16), "ERROR_INVALID_ARGUMENT"),
    RccrNegRow(1, 2, 2, 3, "u8", False, 3, "u8", (32, 4), (0, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),
    RccrNegRow(1, 2, 2, 3, "u8", False, 3, "u8", (4, 32), (0, 0), (16, 16), "ERROR_INVALID_ARGUMENT"),
    RccrNegRow(1, 2, 2, 3, "u8", True, 3, "u8", (4, 4), (0, 0), (16, 16), "ERROR_NOT_COMPATIBLE"),  # planar input
    RccrNegRow(1, 2, 2, 3, "u8", False, 3, "u8", (4, 4), (0, 0), (0, 0), "ERROR_INVALID_ARGUMENT"),  # resize dim
]


class CfnrRow(NamedTuple):
    width: int
    height: int
    images: int
    scalar_base: bool
    scalar_scale: bool
    flags: int
    gscale: float
    gshift: float
    eps: float
    channels: int
    src_planar: bool
    dst_planar: bool
    border: int  # NVCVBorderType
    src_dtype: type
    dst_dtype: type


_C, _REP, _REF, _WRAP, _R101 = 0, 1, 2, 3, 4
_u8, _f32, _s32 = np.uint8, np.float32, np.int32

CFNR_ROWS = [
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 3, True, True, _C, _u8, _u8),
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 3, True, False, _C, _u8, _u8),
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 3, False, True, _C, _u8, _u8),
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 4, False, False, _C, _u8, _u8),
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 4, True, False, _C, _u8, _u8),
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 4, False, False, _REF, _u8, _u8),
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 4, False, False, _R101, _u8, _u8),
    CfnrRow(10, 10, 2, True, True, 0, 1.0, 0.0, 0.0, 3, False, False, _WRAP, _u8, _u8),
    CfnrRow(15, 15, 3, True, True, 0, 1.0, 0.0, 0.0, 1, False, False, _REP, _u8, _u8),
    CfnrRow(9, 13, 10, True, True, 0, 1.0, 0.0, 0.0, 4, True, False, _C, _u8, _f32),
    CfnrRow(15, 15, 10, True, True, 0, 1.0, 0.0, 0.0, 1, False, False, _REP, _f32, _f32),
    CfnrRow(15, 15, 3, True, True, 0, 1.0, 0.0, 0.0, 1, False, False, _REP, _u8, _u8),
    CfnrRow(15, 15, 2, True, True, 0, 1.0, 0.0, 0.0, 1, False, False, _REP, _s32, _f32),
    CfnrRow(15, 15, 2, True, True, 0, 1.0, 0.0, 0.0, 1, False, False, _REP, _s32, _s32),
    CfnrRow(51, 53, 10, True, False, 0, 1.234, 33.21, 0.0, 3, False, False, _REP, _f32, _f32),
    CfnrRow(51, 53, 10, True, True, 1, 1.1, 0.3, 1.23, 4, False, True, _REP, _f32, _f32),
    CfnrRow(51, 53, 10, False, False, 0, 1.0, 12.3, 0.0, 4, True, False, _REP, _f32, _f32),
    CfnrRow(51, 53, 10, False, True, 1, 1.1, 0.3, 1.23, 4, False, True, _REP, _f32, _f32),
]
assert len(CFNR_ROWS) == 18


def cfnr_case(row: CfnrRow, seed: int):
    """Random inputs drawn the way the reference test driver draws them
    (TestOpCropFlipNormalizeReformat.cpp:167-303): image sizes in [0.8, 1.1] x nominal, pixel values 0..255, flip code
    in [-1, 2], crop origin from -3, crop size close to the image size, base in [0, 255), scale in [0, 1).
    Returns (images, rects[N,4], flips[N], base, scale, (out_w, out_h))."""
    rng = np.random.default_rng(seed)
    images, rects = [], []
    for _ in range(row.images):
        w = int(rng.integers(int(row.width * 0.8), int(row.width * 1.1) + 1))
        h = int(rng.integers(int(row.height * 0.8), int(row.height * 1.1) + 1))
        shape = (row.channels, h, w) if row.src_planar else (h, w, row.channels)
        images.append(rng.integers(0, 256, shape).astype(row.src_dtype))
    flips = rng.integers(-1, 3, row.images).astype(np.int32)
    for im in images:
        h, w = (im.shape[1], im.shape[2]) if row.src_planar else (im.shape[0], im.shape[1])
        x = int(rng.integers(-3, min(10, w // 10) + 2))
        y = int(rng.integers(-3, min(10, h // 10) + 2))
        cw = int(rng.integers(max(int(w * 0.8), w - 10), w))
        ch = int(rng.integers(max(int(h * 0.8), h - 10), h))
        rects.append((x, y, cw, ch))
    base = rng.uniform(0, 255, 1 if row.scalar_base else 4).astype(np.float32)
    scale = rng.uniform(0, 1, 1 if row.scalar_scale else 4).astype(np.float32)
    sizes = [((im.shape[2], im.shape[1]) if row.src_planar else (im.shape[1], im.shape[0])) for im in images]
    out = (max(s[0] for s in sizes), max(s[1] for s in sizes))
    return images, np.array(rects, np.int32), flips, base, scale, out


# ------------------------------------------------------------------------------------------------ stand-alone Resize

class ResizeRow(NamedTuple):
    src_w: int
    src_h: int
    dst_w: int
    dst_h: int
    interp: int  # 0 nearest, 1 linear
    images: int
    channels: int
    dtype: type


def _resize_rows():
    """The nearest / linear rows of the reference's Resize table (tests/cvcuda/system/TestOpResize.cpp:49-91): same
    shapes, interpolations, image counts and formats. Its cubic and area rows (:60-69, :71-78 in part) are not covered:
    those interpolations are not implemented here. The variable-shape test draws each image's source and destination
    size from 0.8x to 1.1x of the row's (:211-226); test code here does the same with its own generator."""
    u8, u16, s16, f32 = np.uint8, np.uint16, np.int16, np.float32
    rows = [
        (42, 48, 23, 24, 0, 1, 4, u8), (113, 12, 12, 36, 0, 1, 4, u8), (421, 148, 223, 124, 0, 2, 4, u8),
        (313, 212, 412, 336, 0, 3, 4, u8), (42, 40, 21, 20, 1, 1, 4, u8), (21, 21, 42, 42, 1, 1, 4, u8),
        (420, 420, 210, 210, 1, 4, 4, u8), (210, 210, 420, 420, 1, 5, 4, u8), (1080, 1920, 720, 1280, 1, 1, 4, u8),
        (2160, 3840, 1080, 1920, 1, 1, 4, u8), (2160, 3840, 1440, 2560, 1, 1, 4, u8),
    ]
    for dt in (u8, u16, s16, f32):
        for ch in (1, 3, 4):
            rows.append((42, 48, 23, 24, 0, 1, ch, dt))
    return [ResizeRow(*r) for r in rows]


RESIZE_ROWS = _resize_rows()
assert len(RESIZE_ROWS) == 23


# ------------------------------------------------------------------------------------------------ stand-alone Normalize

class NormalizeRow(NamedTuple):
    width: int
    height: int
    images: int
    scalar_base: bool
    scalar_scale: bool
    flags: int
    gscale: float
    gshift: float
    eps: float


# tests/cvcuda/system/TestOpNormalize.cpp:84-98 (RGBA8 images; scalar parameters are 1x1x1 float32, the others
# RGBAf32 tensors of the image size, one per image)
NORMALIZE_ROWS = [NormalizeRow(*r) for r in [
    (32, 33, 1, True, True, 0, 0.0, 0.0, 0.0), (66, 55, 1, True, True, 0, 1.0, 0.0, 0.0),
    (122, 212, 2, True, True, 0, 1.234, 43.21, 0.0), (211, 102, 3, False, False, 0, 1.1, 0.1, 0.0),
    (21, 12, 5, True, True, 1, 1.2, 0.2, 0.0), (22, 12, 5, False, True, 1, 1.3, 0.3, 0.0),
    (55, 23, 5, True, False, 1, 1.2, 0.2, 0.0), (72, 88, 5, False, False, 1, 1.2, 0.2, 0.0),
    (63, 32, 7, False, True, 0, 1.3, 0.3, 0.0), (22, 13, 9, True, False, 0, 1.4, 0.4, 0.0),
    (55, 33, 2, True, False, 1, 2.1, 1.1, 1.23), (444, 222, 4, True, False, 1, 2.2, 2.2, 12.3),
]]
assert len(NORMALIZE_ROWS) == 12


def normalize_case(row: NormalizeRow, seed: int):
    """Images, base and scale of one table row: uint8 RGBA images, base ~U(0, 255), scale ~U(0, 1) as the reference's
    test draws them (TestOpNormalize.cpp:141-199), from this file's own generator."""
    rng = np.random.default_rng(seed)
    images = [rng.integers(0, 256, (row.height, row.width, 4), dtype=np.uint8) for _ in range(row.images)]
    bshape = (1, 1, 1, 1) if row.scalar_base else (row.images, row.height, row.width, 4)
    sshape = (1, 1, 1, 1) if row.scalar_scale else (row.images, row.height, row.width, 4)
    base = rng.uniform(0.0, 255.0, bshape).astype(np.float32)
    scale = rng.uniform(0.0, 1.0, sshape).astype(np.float32)
    return images, base, scale


# ------------------------------------------------------------------------------------------------ fused passes

MEAN = (123.675, 116.28, 103.53)
INV_STD = tuple(float(np.float32(1.0) / np.float32(s)) for s in (58.395, 57.12, 57.375))


def fused_fixture_cases():
    """(kind, inputs, parameters, expected) of tests/golden/fused_golden.npz: outputs of CHAINS of the reference's goldens."""
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "fused_golden.npz"))
    for k in range(int(z["fused_count"])):
        kind = int(z[f"fused{k}_kind"])
        if kind == 1:
            n = len(z[f"fused{k}_rects"])
            yield k, kind, ([z[f"fused{k}_src{i}"] for i in range(n)], z[f"fused{k}_rects"], z[f"fused{k}_flips"]), \
                z[f"fused{k}_par"], z[f"fused{k}_ref"]
        else:
            yield k, kind, z[f"fused{k}_src"], z[f"fused{k}_par"], z[f"fused{k}_ref"]
