"""ctypes front-end of the reference project's own CUDA kernels (oracle/_ref/libref_cuda_kernels.so).

TEST / BASELINE INFRASTRUCTURE ONLY: used by GPU tests as a cross-check of single kernels (the timed baseline is the
reference's whole operators, oracle/ref_ops.py). The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_PATH = os.path.join(_HERE, "_ref", "libref_cuda_kernels.so")
_lib = None


def lib() -> Optional[C.CDLL]:
    """The library, or None when it was not built (reference tree absent at build time)."""
    global _lib
    if _lib is None:
        if not os.path.exists(_PATH):
            return None
        L = C.CDLL(_PATH)
        L.refcuda_rccr_tensor.restype = C.c_int
        L.refcuda_rccr_tensor.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_longlong, C.c_longlong, C.c_void_p,
                                          C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_int, C.c_int, C.c_float, C.c_float, C.c_int, C.c_void_p]
        L.refcuda_rccr_varshape.restype = C.c_int
        L.refcuda_rccr_varshape.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int,
                                            C.c_void_p]
        L.refcuda_cfnr_u8.restype = C.c_int
        L.refcuda_cfnr_u8.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                      C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int,
                                      C.c_float, C.c_float, C.c_float, C.c_float, C.c_uint32, C.c_void_p]
        _lib = L
    return _lib


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what}: reference kernel launch returned {rc}")


def rccr_tensor(src: torch.Tensor, dst: torch.Tensor, planar: bool, resize, interp: int, crop, manip: int, scale: float,
                offset: float, src_cast: bool) -> torch.Tensor:
    """src: uint8 CUDA [N,H,W,3]; dst: packed uint8/float32 CUDA [N,3,h,w] (planar) or [N,h,w,3]."""
    n, h, w, _ = src.shape
    oh, ow = (dst.shape[2], dst.shape[3]) if planar else (dst.shape[1], dst.shape[2])
    assert dst.is_contiguous() and src.stride(3) == 1 and src.stride(2) == 3
    _check(lib().refcuda_rccr_tensor(src.data_ptr(), n, w, h, src.stride(1), src.stride(0), dst.data_ptr(),
                                     int(dst.dtype == torch.float32), int(planar), ow, oh, resize[0], resize[1], interp,
                                     crop[0], crop[1], manip, scale, offset, int(src_cast), _stream()), "rccr_tensor")
    return dst


def rccr_varshape(table: torch.Tensor, n: int, dst: torch.Tensor, planar: bool, resize, interp: int, crop, manip: int,
                  scale: float, offset: float, src_cast: bool) -> torch.Tensor:
    """table: the device descriptor table of an image batch (NVCVImageBufferStrided[n])."""
    oh, ow = (dst.shape[2], dst.shape[3]) if planar else (dst.shape[1], dst.shape[2])
    _check(lib().refcuda_rccr_varshape(table.data_ptr(), n, dst.data_ptr(), int(dst.dtype == torch.float32), int(planar),
                                       ow, oh, resize[0], resize[1], interp, crop[0], crop[1], manip, scale, offset,
                                       int(src_cast), _stream()), "rccr_varshape")
    return dst


def cfnr_u8(table: torch.Tensor, n: int, channels: int, dst: torch.Tensor, planar: bool, rect: torch.Tensor,
            flip: torch.Tensor, base: torch.Tensor, scale: torch.Tensor, border: int, border_value: float, gscale: float,
            shift: float, eps: float, flags: int) -> torch.Tensor:
    oh, ow = (dst.shape[2], dst.shape[3]) if planar else (dst.shape[1], dst.shape[2])
    _check(lib().refcuda_cfnr_u8(table.data_ptr(), n, channels, dst.data_ptr(), int(dst.dtype == torch.float32),
                                 int(planar), ow, oh, rect.data_ptr(), flip.data_ptr(), base.data_ptr(), base.numel(),
                                 scale.data_ptr(), scale.numel(), border, border_value, gscale, shift, eps, flags,
                                 _stream()), "cfnr_u8")
    return dst
