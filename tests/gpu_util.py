"""Helpers of the GPU parity tests: run the library on torch CUDA tensors and compare with the CPU oracle.

Tolerances (stated once, used everywhere): nearest-neighbour results bit-exact; uint8-domain results within 1 LSB;
float32 results within 1e-5 absolute; float16 within 1 unit in the last place.
"""
from __future__ import annotations

import contextlib

import numpy as np
import torch

F32_ATOL = 1e-5
U8_ATOL = 1


@contextlib.contextmanager
def kernel_path(pkg, path):
    prev = pkg.set_kernel_path(path)
    try:
        yield
    finally:
        pkg.set_kernel_path(prev)


def f16_ulp_diff(a: np.ndarray, b: np.ndarray) -> int:
    """Largest distance in float16 representable steps between two float16 arrays."""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, 0x8000 - u, u)  # monotone integer key of the float16 ordering
    return int(np.abs(key(a) - key(b)).max()) if a.size else 0


def assert_parity(got: np.ndarray, want: np.ndarray, *, exact: bool = False, what: str = ""):
    assert got.shape == want.shape and got.dtype == want.dtype, f"{what}: shape/dtype {got.shape}/{got.dtype} vs {want.shape}/{want.dtype}"
    if exact or got.dtype not in (np.uint8, np.float32, np.float16):
        bad = int((got.view(np.uint8) != want.view(np.uint8)).sum())
        assert bad == 0, f"{what}: {bad} differing bytes (bit-exact required)"
        return
    if got.dtype == np.uint8:
        d = int(np.abs(got.astype(np.int32) - want.astype(np.int32)).max()) if got.size else 0
        assert d <= U8_ATOL, f"{what}: uint8 max diff {d} > {U8_ATOL}"
    elif got.dtype == np.float32:
        d = float(np.abs(got.astype(np.float64) - want.astype(np.float64)).max()) if got.size else 0.0
        assert d <= F32_ATOL, f"{what}: float32 max abs diff {d} > {F32_ATOL}"
    else:
        d = f16_ulp_diff(got, want)
        assert d <= 1, f"{what}: float16 differs by {d} ULP"


def to_dev(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


_TORCH_DTYPE = {np.dtype(np.uint8): torch.uint8, np.dtype(np.int8): torch.int8, np.dtype(np.int16): torch.int16,
                np.dtype(np.int32): torch.int32, np.dtype(np.float32): torch.float32,
                np.dtype(np.float16): torch.float16}
for _np, _name in ((np.uint16, "uint16"), (np.uint32, "uint32")):
    if hasattr(torch, _name):
        _TORCH_DTYPE[np.dtype(_np)] = getattr(torch, _name)


def padded_images(images, pad_to: int = 32, offset: int = 0, planar: bool = False):
    """Copies numpy images (HxWxC, or CxHxW when planar) into CUDA tensors whose rows are padded to a multiple of
    `pad_to` bytes and whose first byte sits `offset` bytes after an aligned address; returns strided views."""
    out = []
    for im in images:
        es = im.itemsize
        if planar:
            c, h, w = im.shape
            row_bytes, rows = w * es, c * h
        else:
            h, w, c = im.shape
            row_bytes, rows = w * c * es, h
        pitch = (row_bytes + pad_to - 1) // pad_to * pad_to
        pitch = (pitch + es - 1) // es * es
        buf = torch.zeros(offset + rows * pitch + 64, dtype=torch.uint8, device="cuda")
        flat = buf[offset:offset + rows * pitch]
        host = torch.from_numpy(np.ascontiguousarray(im).view(np.uint8).reshape(rows, row_bytes))
        flat.view(rows, pitch)[:, :row_bytes].copy_(host.cuda())
        typed = flat.view(_TORCH_DTYPE[im.dtype])
        if planar:
            out.append(torch.as_strided(typed, (c, h, w), (h * pitch // es, pitch // es, 1)))
        else:
            out.append(torch.as_strided(typed, (h, w, c), (pitch // es, c, 1)))
    return out
