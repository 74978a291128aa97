"""ctypes front-end of the CPU checkers (TEST INFRASTRUCTURE ONLY).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may import this module; the product
package never does. It wraps

* ``liboracle.so``        -- the C restatement (preproc_oracle.c), always available after build_oracle.py ran;
* ``_ref/libref_golden.so`` -- the reference project's own golden functions, when they were compiled.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

U8, S8, U16, S16, U32, S32, F32, F16 = range(8)
NP_DTYPES = {U8: np.uint8, S8: np.int8, U16: np.uint16, S16: np.int16, U32: np.uint32, S32: np.int32,
             F32: np.float32, F16: np.float16}
DTYPE_CODE = {np.dtype(v): k for k, v in NP_DTYPES.items()}

NEAREST, LINEAR = 0, 1
BORDER_CONSTANT, BORDER_REPLICATE, BORDER_REFLECT, BORDER_WRAP, BORDER_REFLECT101 = range(5)


class _Image(C.Structure):
    _fields_ = [("base", C.c_void_p), ("width", C.c_int32), ("height", C.c_int32),
                ("rowStride", C.c_int64), ("planeStride", C.c_int64)]


class _Dst(C.Structure):
    _fields_ = [("base", C.c_void_p), ("dtype", C.c_int32), ("width", C.c_int32), ("height", C.c_int32),
                ("sampleStride", C.c_int64), ("rowStride", C.c_int64), ("pixStride", C.c_int64),
                ("chanStride", C.c_int64)]


class _ResizeParams(C.Structure):
    _fields_ = [("resizeW", C.c_int32), ("resizeH", C.c_int32), ("cropX", C.c_int32), ("cropY", C.c_int32),
                ("interp", C.c_int32), ("srcCast", C.c_int32), ("manip", C.c_int32), ("epilogue", C.c_int32),
                ("scale", C.c_float), ("offset", C.c_float), ("base", C.c_float * 4), ("mul", C.c_float * 4),
                ("gscale", C.c_float), ("shift", C.c_float),
                ("dstX", C.c_int32), ("dstY", C.c_int32), ("regionW", C.c_int32), ("regionH", C.c_int32),
                ("padValue", C.c_float)]


class _SliceParams(C.Structure):
    _fields_ = [("srcType", C.c_int32), ("srcPlanar", C.c_int32), ("channels", C.c_int32), ("border", C.c_int32),
                ("borderValue", C.c_float), ("base", C.POINTER(C.c_float)), ("baseCh", C.c_int32),
                ("scale", C.POINTER(C.c_float)), ("scaleCh", C.c_int32),
                ("gscale", C.c_float), ("shift", C.c_float), ("epsilon", C.c_float), ("flags", C.c_uint32)]


_lib = None
_ref = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            from . import build_oracle  # noqa: WPS433
            build_oracle.build_oracle()
        L = C.CDLL(path)
        L.oracle_resize_crop.restype = C.c_int
        L.oracle_resize_crop.argtypes = [C.POINTER(_Image), C.c_int32, C.c_void_p, C.c_void_p,
                                         C.POINTER(_ResizeParams), C.POINTER(_Dst), C.c_int32]
        L.oracle_crop_flip_normalize.restype = C.c_int
        L.oracle_crop_flip_normalize.argtypes = [C.POINTER(_Image), C.c_int32, C.c_void_p, C.c_void_p,
                                                 C.POINTER(_SliceParams), C.POINTER(_Dst), C.c_int32]
        L.oracle_resize_source_bytes.restype = C.c_int64
        L.oracle_resize_source_bytes.argtypes = [C.c_int32, C.c_int32, C.c_int64, C.c_void_p,
                                                 C.POINTER(_ResizeParams)]
        L.oracle_resized_crop.restype = C.c_int
        L.oracle_resized_crop.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                          C.c_void_p]
        L.oracle_resize_plain.restype = C.c_int
        L.oracle_resize_plain.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
        L.oracle_normalize.restype = C.c_int
        L.oracle_normalize.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_void_p,
                                       C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_uint32]
        L.oracle_copy_make_border.restype = C.c_int
        L.oracle_copy_make_border.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                              C.c_int32, C.c_int32, C.c_void_p]
        L.oracle_sat_u8.restype = C.c_uint8
        L.oracle_sat_u8.argtypes = [C.c_float]
        L.oracle_sat_s16.restype = C.c_int16
        L.oracle_sat_s16.argtypes = [C.c_float]
        L.oracle_sat_s32.restype = C.c_int32
        L.oracle_sat_s32.argtypes = [C.c_float]
        L.oracle_f32_to_f16_bits.restype = C.c_uint16
        L.oracle_f32_to_f16_bits.argtypes = [C.c_float]
        _lib = L
    return _lib


def ref() -> Optional[C.CDLL]:
    """The reference's own golden functions, or None when they were not compiled."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libref_golden.so")
        if not os.path.exists(path):
            return None
        R = C.CDLL(path)
        R.ref_rccr.restype = C.c_int
        R.ref_rccr.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int]
        R.ref_cfnr.restype = C.c_int
        R.ref_cfnr.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int,
                               C.c_int, C.c_int, C.c_int, C.c_float, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                               C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float, C.c_uint32]
        if hasattr(R, "ref_resized_crop"):
            R.ref_resized_crop.restype = C.c_int
            R.ref_resized_crop.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                           C.c_int, C.c_int, C.c_void_p]
        if hasattr(R, "ref_resize"):
            R.ref_resize.restype = C.c_int
            R.ref_resize.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_int, C.c_int]
        if hasattr(R, "ref_normalize"):
            R.ref_normalize.restype = C.c_int
            R.ref_normalize.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                        C.c_int, C.c_float, C.c_float, C.c_float, C.c_uint32]
        if hasattr(R, "ref_copy_make_border"):
            R.ref_copy_make_border.restype = C.c_int
            R.ref_copy_make_border.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 10 + [C.c_void_p]
        for name, rt in (("ref_sat_u8_f32", C.c_uint8), ("ref_sat_s32_f32", C.c_int32), ("ref_sat_s16_f32", C.c_int16)):
            f = getattr(R, name)
            f.restype = rt
            f.argtypes = [C.c_float]
        _ref = R
    return _ref


# ------------------------------------------------------------------------------------------------ helpers

@dataclass
class ResizeSpec:
    """Parameters of the resize/crop/convert/reformat path (see preproc_oracle.h: OracleResizeParams)."""
    resize: tuple  # (w, h)
    crop: tuple = (0, 0)  # (x, y)
    out_size: tuple = (0, 0)  # region (w, h) = output size when there is no canvas
    interp: int = LINEAR
    src_cast: bool = True
    manip: int = 0
    scale: float = 1.0
    offset: float = 0.0
    base: Optional[Sequence[float]] = None  # per-channel normalisation: (v-base)*mul*gscale+shift
    mul: Optional[Sequence[float]] = None
    gscale: float = 1.0
    shift: float = 0.0
    canvas: Optional[tuple] = None  # (w, h) of the output when the region is placed inside a larger canvas
    dst_pos: tuple = (0, 0)
    pad_value: float = 0.0
    extra: dict = field(default_factory=dict)

    def to_c(self) -> _ResizeParams:
        p = _ResizeParams()
        p.resizeW, p.resizeH = self.resize
        p.cropX, p.cropY = self.crop
        p.interp, p.srcCast, p.manip = int(self.interp), int(bool(self.src_cast)), int(self.manip)
        p.epilogue = 0 if self.base is None else 1
        p.scale, p.offset = np.float32(self.scale), np.float32(self.offset)
        for i in range(4):
            p.base[i] = np.float32(self.base[i]) if self.base is not None and i < len(self.base) else 0.0
            p.mul[i] = np.float32(self.mul[i]) if self.mul is not None and i < len(self.mul) else 1.0
        p.gscale, p.shift = np.float32(self.gscale), np.float32(self.shift)
        p.dstX, p.dstY = self.dst_pos
        p.regionW, p.regionH = self.out_size
        p.padValue = np.float32(self.pad_value)
        return p

    @property
    def canvas_size(self) -> tuple:
        return self.canvas if self.canvas is not None else self.out_size


def _images_c(images: Sequence[np.ndarray], planar: bool = False):
    arr = (_Image * len(images))()
    for i, im in enumerate(images):
        if planar:  # C,H,W
            c, h, w = im.shape
            assert im.strides[2] == im.itemsize
            arr[i] = _Image(im.ctypes.data, w, h, im.strides[1], im.strides[0])
        else:  # H,W,C
            h, w, c = im.shape
            assert im.strides[2] == im.itemsize and im.strides[1] == im.itemsize * c
            arr[i] = _Image(im.ctypes.data, w, h, im.strides[0], 0)
    return arr


def _dst_c(out: np.ndarray, planar: bool) -> _Dst:
    """out is [N,C,H,W] when planar else [N,H,W,C]."""
    if planar:
        n, c, h, w = out.shape
        ss, cs, rs, ps = out.strides
    else:
        n, h, w, c = out.shape
        ss, rs, ps, cs = out.strides
    return _Dst(out.ctypes.data, DTYPE_CODE[out.dtype], w, h, ss, rs, ps, cs)


def resize_crop(images: Sequence[np.ndarray], spec: ResizeSpec, out_dtype=np.float32, planar: bool = True,
                roi: Optional[np.ndarray] = None, flip: Optional[np.ndarray] = None, nthreads: int = 1) -> np.ndarray:
    """Run the restated golden on a list of HxWx3 uint8 arrays (rows may be padded). Returns NCHW or NHWC."""
    n = len(images)
    cw, ch = spec.canvas_size
    out = np.empty((n, 3, ch, cw) if planar else (n, ch, cw, 3), dtype=out_dtype)
    imgs = _images_c(images)
    roi_p = flip_p = None
    if roi is not None:
        roi = np.ascontiguousarray(roi, dtype=np.int32)
        roi_p = roi.ctypes.data
    if flip is not None:
        flip = np.ascontiguousarray(flip, dtype=np.int32)
        flip_p = flip.ctypes.data
    p, d = spec.to_c(), _dst_c(out, planar)
    rc = lib().oracle_resize_crop(imgs, n, roi_p, flip_p, C.byref(p), C.byref(d), nthreads)
    if rc != 0:
        raise ValueError("oracle_resize_crop rejected its arguments")
    return out


def crop_flip_normalize(images: Sequence[np.ndarray], src_planar: bool, crop_rect: np.ndarray, flip: np.ndarray,
                        out_size: tuple, out_dtype, out_planar: bool, border: int, border_value: float,
                        base: np.ndarray, scale: np.ndarray, gscale: float = 1.0, shift: float = 0.0,
                        epsilon: float = 0.0, flags: int = 0, nthreads: int = 1) -> np.ndarray:
    """Restated CropFlipNormalizeReformat golden. images: HxWxC (interleaved) or CxHxW (planar) arrays."""
    n = len(images)
    ch = images[0].shape[0] if src_planar else images[0].shape[2]
    w, h = out_size
    out = np.empty((n, ch, h, w) if out_planar else (n, h, w, ch), dtype=out_dtype)
    imgs = _images_c(images, planar=src_planar)
    crop_rect = np.ascontiguousarray(crop_rect, dtype=np.int32)
    flip = np.ascontiguousarray(flip, dtype=np.int32)
    base = np.ascontiguousarray(base, dtype=np.float32)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    p = _SliceParams(DTYPE_CODE[images[0].dtype], int(src_planar), ch, border, border_value,
                     base.ctypes.data_as(C.POINTER(C.c_float)), base.size,
                     scale.ctypes.data_as(C.POINTER(C.c_float)), scale.size, gscale, shift, epsilon, flags)
    d = _dst_c(out, out_planar)
    rc = lib().oracle_crop_flip_normalize(imgs, n, crop_rect.ctypes.data, flip.ctypes.data, C.byref(p), C.byref(d),
                                          nthreads)
    if rc != 0:
        raise ValueError("oracle_crop_flip_normalize rejected its arguments")
    return out


def resize_source_bytes(src_w: int, src_h: int, row_stride: int, spec: ResizeSpec, roi=None) -> int:
    p = spec.to_c()
    roi_p = None
    if roi is not None:
        roi = np.ascontiguousarray(roi, dtype=np.int32)
        roi_p = roi.ctypes.data
    return int(lib().oracle_resize_source_bytes(src_w, src_h, row_stride, roi_p, C.byref(p)))


# ------------------------------------------------------------------------------------------------ reference golden

def ref_rccr(src: np.ndarray, resize, crop, out_size, interp, manip, scale, offset, src_cast, out_dtype,
             planar: bool) -> np.ndarray:
    """The reference's ResizeCropConvert on a packed [N,H,W,3] uint8 batch."""
    R = ref()
    assert R is not None
    src = np.ascontiguousarray(src, dtype=np.uint8)
    n, h, w, _ = src.shape
    ow, oh = out_size
    out = np.empty((n, 3, oh, ow) if planar else (n, oh, ow, 3), dtype=out_dtype)
    R.ref_rccr(out.ctypes.data, ow, oh, int(planar), int(np.dtype(out_dtype) == np.float32), src.ctypes.data, w, h, n,
               resize[0], resize[1], crop[0], crop[1], interp, manip, float(scale), float(offset), int(src_cast))
    return out


def ref_cfnr(image: np.ndarray, src_planar: bool, rect, flip: int, out_size, out_dtype, out_planar: bool, border: int,
             border_value: float, base, scale, gscale, shift, epsilon, flags) -> np.ndarray:
    """The reference's CropFlipNormalizeReformat golden on one packed image."""
    R = ref()
    assert R is not None
    image = np.ascontiguousarray(image)
    if src_planar:
        ch, h, w = image.shape
    else:
        h, w, ch = image.shape
    ow, oh = out_size
    out = np.empty((ch, oh, ow) if out_planar else (oh, ow, ch), dtype=out_dtype)
    base = np.ascontiguousarray(base, dtype=np.float32)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    rc = R.ref_cfnr(out.ctypes.data, DTYPE_CODE[out.dtype], int(out_planar), ow, oh, image.ctypes.data,
                    DTYPE_CODE[image.dtype], int(src_planar), w, h, ch, border, border_value, flip,
                    int(rect[0]), int(rect[1]), int(rect[2]), int(rect[3]), base.ctypes.data, base.size,
                    scale.ctypes.data, scale.size, gscale, shift, epsilon, flags)
    assert rc == 0
    return out


# ------------------------------------------------------------------------------------------------ stand-alone Resize

class _PlainImage(C.Structure):
    _fields_ = [("base", C.c_void_p), ("width", C.c_int32), ("height", C.c_int32), ("rowStride", C.c_int64)]


def resize_plain(images: Sequence[np.ndarray], out_sizes: Sequence[tuple], interp: int,
                 golden_float: bool = False, rects=None) -> list:
    """Stand-alone Resize restatement (resize_oracle.h) on packed HxWxC images (C = 1..4; uint8, uint16, int16 or
    float32); out_sizes are (w, h) per image; rects, if given, one (left, top, width, height) crop rectangle per image
    (the golden's crop arguments). Returns the resized images."""
    imgs = [np.ascontiguousarray(im) for im in images]
    n = len(imgs)
    dt = imgs[0].dtype
    ch = imgs[0].shape[2]
    outs = [np.empty((h, w, ch), dtype=dt) for (w, h) in out_sizes]
    S = (_PlainImage * n)()
    D = (_PlainImage * n)()
    for i in range(n):
        h, w, _ = imgs[i].shape
        S[i] = _PlainImage(imgs[i].ctypes.data, w, h, imgs[i].strides[0])
        D[i] = _PlainImage(outs[i].ctypes.data, out_sizes[i][0], out_sizes[i][1], outs[i].strides[0])
    r = None if rects is None else np.ascontiguousarray(np.asarray(rects, np.int32).reshape(n, 4))
    rc = lib().oracle_resized_crop(S, D, n, DTYPE_CODE[np.dtype(dt)], ch, interp, int(golden_float),
                                   None if r is None else r.ctypes.data)
    assert rc == 0
    return outs


def ref_resize(image: np.ndarray, out_size: tuple, interp: int, rect=None) -> np.ndarray:
    """The reference's own Resize golden (test::resizedCrop as test::Resize calls it, or with a (left, top, width,
    height) crop rectangle as test::ResizedCrop calls it) on one packed HxWxC image."""
    R = ref()
    assert R is not None and hasattr(R, "ref_resize")
    if rect is not None:
        image = np.ascontiguousarray(image)
        h, w, ch = image.shape
        ow, oh = out_size
        out = np.empty((oh, ow, ch), dtype=image.dtype)
        r = np.ascontiguousarray(np.asarray(rect, np.int32))
        rc = R.ref_resized_crop(out.ctypes.data, ow * ch, ow, oh, image.ctypes.data, w * ch, w, h, ch, DTYPE_CODE[image.dtype],
                                interp, r.ctypes.data)
        assert rc == 0
        return out
    image = np.ascontiguousarray(image)
    h, w, ch = image.shape
    ow, oh = out_size
    out = np.empty((oh, ow, ch), dtype=image.dtype)
    rc = R.ref_resize(out.ctypes.data, ow * ch, ow, oh, image.ctypes.data, w * ch, w, h, ch, DTYPE_CODE[image.dtype], interp)
    assert rc == 0
    return out


# ------------------------------------------------------------------------------------------------ stand-alone Normalize

def _broadcast_strides(t: np.ndarray):
    """Byte strides of a float32 [N, H, W, C] parameter tensor with 0 for every dimension of extent 1."""
    assert t.ndim == 4 and t.dtype == np.float32
    return (C.c_int64 * 4)(*[0 if t.shape[k] == 1 else t.strides[k] for k in range(4)])


def normalize(images: Sequence[np.ndarray], base: np.ndarray, scale: np.ndarray, out_dtype=None, gscale: float = 1.0,
              shift: float = 0.0, epsilon: float = 0.0, flags: int = 0) -> list:
    """Stand-alone Normalize restatement on packed HxWxC images; base / scale are float32 [N|1, H|1, W|1, C|1] (full
    extents only make sense when all images have the same size)."""
    imgs = [np.ascontiguousarray(im) for im in images]
    n = len(imgs)
    dt = imgs[0].dtype
    od = np.dtype(out_dtype or dt)
    ch = imgs[0].shape[2]
    outs = [np.empty(im.shape, dtype=od) for im in imgs]
    S = (_PlainImage * n)()
    D = (_PlainImage * n)()
    for i in range(n):
        h, w, _ = imgs[i].shape
        S[i] = _PlainImage(imgs[i].ctypes.data, w, h, imgs[i].strides[0])
        D[i] = _PlainImage(outs[i].ctypes.data, w, h, outs[i].strides[0])
    base = np.ascontiguousarray(base, dtype=np.float32)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    rc = lib().oracle_normalize(S, D, n, DTYPE_CODE[np.dtype(dt)], DTYPE_CODE[od], ch, base.ctypes.data,
                                _broadcast_strides(base), scale.ctypes.data, _broadcast_strides(scale), gscale, shift,
                                epsilon, flags)
    assert rc == 0
    return outs


def ref_normalize(image: np.ndarray, base: np.ndarray, scale: np.ndarray, gscale, shift, epsilon, flags) -> np.ndarray:
    """The reference's own Normalize golden on one packed uint8 HxWxC image; base / scale hold one value or HxWxC."""
    R = ref()
    assert R is not None and hasattr(R, "ref_normalize")
    image = np.ascontiguousarray(image, dtype=np.uint8)
    h, w, ch = image.shape
    base = np.ascontiguousarray(base, dtype=np.float32)
    scale = np.ascontiguousarray(scale, dtype=np.float32)
    out = np.empty_like(image)
    rc = R.ref_normalize(out.ctypes.data, image.ctypes.data, w, h, ch, base.ctypes.data, int(base.size > 1),
                         scale.ctypes.data, int(scale.size > 1), gscale, shift, epsilon, flags)
    assert rc == 0
    return out


# ------------------------------------------------------------------------------------------------ stand-alone ConvertTo

def convert_to(src: np.ndarray, out_dtype, alpha: float, beta: float) -> np.ndarray:
    """The reference test's expectation for ConvertTo, value by value (tests/cvcuda/system/TestOpConvertTo.cpp:118-133):
    ``SaturateCast<DstT>(alpha * val + beta)`` with double alpha / beta, i.e. product and sum in double precision, then
    round half to even and clamp for the integer types (cuda_tools/detail/SaturateCastImpl.hpp, host path) or a plain
    narrowing for float32."""
    v = np.float64(alpha) * src.astype(np.float64) + np.float64(beta)
    od = np.dtype(out_dtype)
    if od.kind == "f":
        return v.astype(od)
    info = np.iinfo(od)
    return np.clip(np.rint(v), info.min, info.max).astype(od)


# ------------------------------------------------------------------------------------------------ stand-alone CopyMakeBorder

def border_fill(value, dtype, channels: int) -> np.ndarray:
    """The per-channel constant border value converted to the element type the way the golden does
    (static_cast<T>(float), tests/cvcuda/system/TestOpCopyMakeBorder.cpp:69), as the low bytes of four 32-bit words."""
    v = np.zeros(4, np.float32)
    v[:len(value)] = np.asarray(value, np.float32)[:4]
    words = np.zeros(4, np.uint32)
    dt = np.dtype(dtype)
    for c in range(4):
        if dt.kind in "iu":  # inside the type's range a static_cast drops the fraction; outside it (undefined there): clamp
            info = np.iinfo(dt)
            elem = np.array([min(max(np.trunc(np.float64(v[c])), info.min), info.max)]).astype(dt)
        else:
            elem = np.array([v[c]]).astype(dt)
        words[c] = np.frombuffer(elem.tobytes().ljust(4, b"\0"), np.uint32)[0]
    return words


def copy_make_border(images: Sequence[np.ndarray], out_sizes: Sequence[tuple], top, left, border: int, value=(0, 0, 0, 0)) -> list:
    """Stand-alone CopyMakeBorder restatement on packed HxWxC images; out_sizes are (w, h) per image; top / left one
    int each, or one per image."""
    imgs = [np.ascontiguousarray(im) for im in images]
    n = len(imgs)
    dt, ch = imgs[0].dtype, imgs[0].shape[2]
    outs = [np.empty((h, w, ch), dtype=dt) for (w, h) in out_sizes]
    S = (_PlainImage * n)()
    D = (_PlainImage * n)()
    for i in range(n):
        h, w, _ = imgs[i].shape
        S[i] = _PlainImage(imgs[i].ctypes.data, w, h, imgs[i].strides[0])
        D[i] = _PlainImage(outs[i].ctypes.data, out_sizes[i][0], out_sizes[i][1], outs[i].strides[0])
    per = not np.isscalar(top)
    t = np.ascontiguousarray(np.atleast_1d(top), np.int32)
    l = np.ascontiguousarray(np.atleast_1d(left), np.int32)
    fill = border_fill(value, dt, ch)
    rc = lib().oracle_copy_make_border(S, D, n, dt.itemsize, ch, t.ctypes.data, l.ctypes.data, int(per), border, fill.ctypes.data)
    assert rc == 0
    return outs


def ref_copy_make_border(batch: np.ndarray, out_size: tuple, top: int, left: int, border: int, value=(0, 0, 0, 0)) -> np.ndarray:
    """The reference's own CopyMakeBorder golden (tensor form) on a packed [N, H, W, C] batch."""
    R = ref()
    assert R is not None and hasattr(R, "ref_copy_make_border")
    batch = np.ascontiguousarray(batch)
    n, h, w, ch = batch.shape
    ow, oh = out_size
    out = np.empty((n, oh, ow, ch), dtype=batch.dtype)
    v = np.zeros(4, np.float32)
    v[:len(value)] = np.asarray(value, np.float32)[:4]
    rc = R.ref_copy_make_border(out.ctypes.data, batch.ctypes.data, n, ow, oh, w, h, ch, DTYPE_CODE[batch.dtype], top, left,
                                border, v.ctypes.data)
    assert rc == 0
    return out


# ------------------------------------------------------------------------------------------------ RandomResizedCrop

def ref_random_crop_rects(seed: int, sizes, min_scale=0.08, max_scale=1.0, min_ratio=0.75, max_ratio=4.0 / 3.0) -> np.ndarray:
    """Rectangles (left, top, width, height) from the reference test's own GetCropParams for images of the given
    (width, height) sizes, one generator seeded with `seed` for the whole sequence."""
    R = ref()
    assert R is not None and hasattr(R, "ref_random_crop_rects")
    rc = np.ascontiguousarray(np.array([(h, w) for (w, h) in sizes], np.int32))
    out = np.empty((len(sizes), 4), np.int32)
    R.ref_random_crop_rects.restype = C.c_int
    R.ref_random_crop_rects.argtypes = [C.c_uint, C.c_double, C.c_double, C.c_double, C.c_double, C.c_void_p, C.c_int, C.c_void_p]
    assert R.ref_random_crop_rects(seed, min_scale, max_scale, min_ratio, max_ratio, rc.ctypes.data, len(sizes), out.ctypes.data) == 0
    return out


# ------------------------------------------------------------------------------------------------ composed references
# The fused entry points do in one pass what the reference needs a chain of operators for. Each function below builds
# the expected result of such a pass from the reference's OWN golden functions only (oracle/_ref), chained the way a user
# of the reference would chain its operators, so that the additions to the restatement in preproc_oracle.c (per-channel
# affine in the resize path, float16 store, region of interest + flip, letterbox) are pinned as well.

def ref_resize_then_normalize(batch: np.ndarray, resize, crop, out_size, interp, base, mul, out_dtype=np.float32) -> np.ndarray:
    """ResizeCropConvertReformat (scale 1, offset 0, float32, no rounding in between) followed by the per-channel
    (v - base) * mul of CropFlipNormalizeReformat on the float image (whole image, no flip), NCHW; float16 = that result
    rounded to nearest even. Goldens: tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp:76-172 and
    TestOpCropFlipNormalizeReformat.cpp:43-149 (its float32 -> float32 instance; the Normalize golden of
    TestOpNormalize.cpp:34-77 only exists for uint8 -> uint8 images)."""
    mid = ref_rccr(batch, resize, crop, out_size, interp, 0, 1.0, 0.0, False, np.float32, planar=False)
    ow, oh = out_size
    out = np.stack([ref_cfnr(im, False, (0, 0, ow, oh), 2, out_size, np.float32, True, 0, 0.0, base, mul, 1.0, 0.0, 0.0, 0)
                    for im in mid])
    return out if np.dtype(out_dtype) == np.float32 else out.astype(out_dtype)


def ref_crop_resize_flip_normalize(images: Sequence[np.ndarray], rects, flips, out_size, base, mul,
                                   out_dtype=np.float32) -> np.ndarray:
    """Per image: the rectangle cut out as an image of its own (CustomCrop), resized by ResizeCropConvertReformat's golden
    to uint8 (the intermediate a chain of operators has), then CropFlipNormalizeReformat's golden with the whole resized
    image as crop, the flip code and the per-channel constants, NCHW."""
    ow, oh = out_size
    outs = []
    for im, (x, y, w, h), f in zip(images, rects, flips):
        sub = np.ascontiguousarray(im[y:y + h, x:x + w])
        small = ref_rccr(sub[None], out_size, (0, 0), out_size, 1, 0, 1.0, 0.0, True, np.uint8, planar=False)[0]
        outs.append(ref_cfnr(small, False, (0, 0, ow, oh), int(f), out_size, np.float32, True, 0, 0.0, base, mul, 1.0, 0.0, 0.0, 0))
    out = np.stack(outs)
    return out if np.dtype(out_dtype) == np.float32 else out.astype(out_dtype)


def ref_letterbox(batch: np.ndarray, resize, canvas, dst_pos, pad_value: int, scale: float) -> np.ndarray:
    """Resize (stand-alone Resize golden, tests/cvcuda/system/ResizeUtils.cpp:189-300) -> CopyMakeBorder golden with a
    constant (TestOpCopyMakeBorder.cpp:40-97) -> ResizeCropConvertReformat's golden as an identity-sized nearest pass that
    reverses the channels, multiplies by `scale` and writes float32 NCHW (the ConvertTo + channel swap + Reformat tail)."""
    small = np.stack([ref_resize(im, resize, 1) for im in batch])
    cw, ch = canvas
    padded = ref_copy_make_border(small, canvas, dst_pos[1], dst_pos[0], 0, (pad_value,) * 4)
    return ref_rccr(padded, (cw, ch), (0, 0), (cw, ch), 0, 1, scale, 0.0, False, np.float32, planar=True)
