"""ctypes front-end of the harness over the reference's C++ API (oracle/_ref/libharness_b200.so / libharness_ref.so).

TEST / BASELINE INFRASTRUCTURE ONLY. ``load("b200")`` runs the reference's header-only wrappers, real tensors and real
image batches against the B200 library; ``load("ref")`` runs the same calls against the reference's own operators
compiled for sm_100a. Load only ONE of the two per process, and do not mix with the object-model test double of
tests/fake_nvcv in the same process: the B200 library binds the nvcv* functions it finds first, once.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
CODE = {np.dtype(np.uint8): 0, np.dtype(np.int8): 1, np.dtype(np.uint16): 2, np.dtype(np.int16): 3, np.dtype(np.uint32): 4,
        np.dtype(np.int32): 5, np.dtype(np.float32): 6, np.dtype(np.float16): 7}
_loaded = {}


def path(which: str) -> str:
    return os.path.join(_HERE, "_ref", {"b200": "libharness_b200.so", "ref": "libharness_ref.so"}[which])


def load(which: str) -> Optional[C.CDLL]:
    """The harness library, or None when it was not built."""
    if which not in _loaded:
        if not os.path.exists(path(which)):
            return None
        L = C.CDLL(path(which))
        L.h_last_message.restype = C.c_char_p
        L.h_which.restype = C.c_char_p
        for name in ("h_rccr_tensor", "h_rccr_varshape", "h_cfnr", "h_time_classify", "h_time_letterbox", "h_time_varshape", "h_time_cfnr", "h_time_classify_e2e_host", "h_time_single_op", "h_time_rccr_list"):
            getattr(L, name).restype = C.c_int
        _loaded[which] = L
    return _loaded[which]


class HarnessError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"status {status}: {message}")
        self.status = status


def _check(L, st):
    if st != 0:
        raise HarnessError(st, L.h_last_message().decode(errors="replace"))


def _image_args(images: Sequence[np.ndarray], planar: bool):
    imgs = [np.ascontiguousarray(im) for im in images]
    n = len(imgs)
    ptrs = (C.c_void_p * n)(*[im.ctypes.data for im in imgs])
    ws = (C.c_int * n)(*[(im.shape[2] if planar else im.shape[1]) for im in imgs])
    hs = (C.c_int * n)(*[(im.shape[1] if planar else im.shape[0]) for im in imgs])
    return imgs, ptrs, ws, hs


def rccr_tensor(L, src: np.ndarray, resize, crop, out_size, interp, manip, scale, offset, src_cast, out_dtype, planar):
    src = np.ascontiguousarray(src, np.uint8)
    n, h, w, _ = src.shape
    ow, oh = out_size
    out = np.empty((n, 3, oh, ow) if planar else (n, oh, ow, 3), out_dtype)
    _check(L, L.h_rccr_tensor(C.c_void_p(src.ctypes.data), n, h, w, C.c_void_p(out.ctypes.data), CODE[np.dtype(out_dtype)],
                              int(planar), ow, oh, resize[0], resize[1], int(interp), crop[0], crop[1], int(manip),
                              C.c_float(scale), C.c_float(offset), int(src_cast)))
    return out


def rccr_varshape(L, images, resize, crop, out_size, interp, manip, scale, offset, src_cast, out_dtype, planar,
                  push_late: int = 0):
    imgs, ptrs, ws, hs = _image_args(images, False)
    n = len(imgs)
    ow, oh = out_size
    out = np.empty((n, 3, oh, ow) if planar else (n, oh, ow, 3), out_dtype)
    _check(L, L.h_rccr_varshape(ptrs, ws, hs, n, C.c_void_p(out.ctypes.data), CODE[np.dtype(out_dtype)], int(planar), ow, oh,
                                resize[0], resize[1], int(interp), crop[0], crop[1], int(manip), C.c_float(scale),
                                C.c_float(offset), int(src_cast), int(push_late)))
    return out


def cfnr(L, images, src_planar, rects, flips, out_size, out_dtype, out_planar, border, border_value, base, scale, gscale, shift,
         epsilon, flags):
    imgs, ptrs, ws, hs = _image_args(images, src_planar)
    n = len(imgs)
    ch = imgs[0].shape[0] if src_planar else imgs[0].shape[2]
    ow, oh = out_size
    out = np.empty((n, ch, oh, ow) if out_planar else (n, oh, ow, ch), out_dtype)
    rects = np.ascontiguousarray(rects, np.int32)
    flips = np.ascontiguousarray(flips, np.int32)
    base = np.ascontiguousarray(base, np.float32)
    scale = np.ascontiguousarray(scale, np.float32)
    _check(L, L.h_cfnr(ptrs, ws, hs, n, CODE[imgs[0].dtype], ch, int(src_planar), C.c_void_p(out.ctypes.data),
                       CODE[np.dtype(out_dtype)], int(out_planar), ow, oh, C.c_void_p(rects.ctypes.data), int(border),
                       C.c_float(border_value), C.c_void_p(flips.ctypes.data), C.c_void_p(base.ctypes.data), base.size,
                       C.c_void_p(scale.ctypes.data), scale.size, C.c_float(gscale), C.c_float(shift), C.c_float(epsilon),
                       C.c_uint32(flags)))
    return out


def time_classify(L, n, h, w, resize, crop, out_size, interp, chain: bool, max_per_call: int, warmup: int, iters: int):
    """(ms per pass, launches per pass) of the classification-style pass on device-resident data."""
    ms, launches = C.c_float(), C.c_int()
    _check(L, L.h_time_classify(n, h, w, resize[0], resize[1], crop[0], crop[1], out_size[0], out_size[1], int(interp), int(chain),
                                int(max_per_call), warmup, iters, C.byref(ms), C.byref(launches)))
    return ms.value, launches.value


def time_rccr_list(L, n, h, w, resize, crop, out_size, interp, scale: float, warmup: int, iters: int):
    """ms per call of the stock variable-shape ResizeCropConvertReformat on a list of n equal-sized RGB8 images -> float32 NCHW."""
    ms = C.c_float()
    _check(L, L.h_time_rccr_list(n, h, w, resize[0], resize[1], crop[0], crop[1], out_size[0], out_size[1], int(interp),
                                 C.c_float(scale), warmup, iters, C.byref(ms)))
    return ms.value


def time_letterbox(L, n, h, w, resize, canvas, top, chain: bool, warmup: int, iters: int):
    ms, launches = C.c_float(), C.c_int()
    _check(L, L.h_time_letterbox(n, h, w, resize[0], resize[1], canvas[0], canvas[1], top, int(chain), warmup, iters,
                                 C.byref(ms), C.byref(launches)))
    return ms.value, launches.value


def time_varshape(L, sizes, out_size, rects, flips, chain: bool, warmup: int, iters: int):
    n = len(sizes)
    ws = (C.c_int * n)(*[s[0] for s in sizes])
    hs = (C.c_int * n)(*[s[1] for s in sizes])
    rects = np.ascontiguousarray(rects, np.int32)
    flips = np.ascontiguousarray(flips, np.int32)
    ms, launches = C.c_float(), C.c_int()
    _check(L, L.h_time_varshape(ws, hs, n, out_size[0], out_size[1], C.c_void_p(rects.ctypes.data), C.c_void_p(flips.ctypes.data),
                                int(chain), warmup, iters, C.byref(ms), C.byref(launches)))
    return ms.value, launches.value


def time_cfnr(L, n, h, w, warmup: int, iters: int):
    ms, launches = C.c_float(), C.c_int()
    _check(L, L.h_time_cfnr(n, h, w, warmup, iters, C.byref(ms), C.byref(launches)))
    return ms.value, launches.value


def time_classify_e2e_host(L, n, h, w, resize, crop, out_size, interp, warmup: int, iters: int):
    """ms per pass of the one-pass entry point on nvcv tensors that wrap page-locked host memory (B200 build only)."""
    ms = C.c_float()
    _check(L, L.h_time_classify_e2e_host(n, h, w, resize[0], resize[1], crop[0], crop[1], out_size[0], out_size[1], int(interp),
                                         warmup, iters, C.byref(ms)))
    return ms.value


def select_stage(L, stage: int) -> None:
    """Chain legs time the whole chain (stage < 0, the default) or only operator number `stage` of it."""
    L.h_select_stage(int(stage))


SINGLE_OPS = {"resize": 0, "normalize_u8_f32": 1, "convertto_u8_f32": 2, "reformat_f32": 3, "copymakeborder": 4}


def time_single_op(L, op: str, n, h, w, out_size=(0, 0), interp=1, warmup: int = 3, iters: int = 20):
    """ms per call of one stand-alone operator on a dense RGB batch (see h_time_single_op)."""
    ms = C.c_float()
    _check(L, L.h_time_single_op(SINGLE_OPS[op], n, h, w, out_size[0], out_size[1], int(interp), warmup, iters, C.byref(ms)))
    return ms.value
