"""b200ppResizedCropNoAlloc against b200ppResizedCrop, through the C ABI.

The no-alloc entry point exists for callers that may not allocate device memory (a plug-in in a serving process whose
GPU memory is fully handed out, a GPU shared with a model that fills it): it keeps the per-image rectangle table in an
array built into the library and takes the rectangles from the host. Its results must be those of the ordinary entry
point, which reads the rectangles from a device table the caller allocated. Two calls in a row are compared, the second
with fewer images and other rectangles, because every call shares the one built-in table and finds the previous
call's rectangles in it. Integer results are bit-exact, so equality is the tolerance.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_RECTS = 4096  # B200PP_NO_ALLOC_MAX_RECTS in include/cvcuda_b200/preproc.h


def _bind(pkg):
    L = C.CDLL(pkg.lib_path())
    S = pkg.ops._ImageSet
    L.b200ppResizedCropNoAlloc.argtypes = [C.POINTER(S), C.POINTER(S), C.c_void_p, C.c_int32, C.c_void_p]
    L.b200ppResizedCropNoAlloc.restype = C.c_int
    L.b200ppResizedCrop.argtypes = [C.POINTER(S), C.POINTER(S), C.c_void_p, C.c_int32, C.c_void_p]
    L.b200ppResizedCrop.restype = C.c_int
    L.b200ppGetLastErrorMessage.restype = C.c_char_p
    return L, S


def _dense(S, t: torch.Tensor, dtype_code: int):
    n, h, w, c = t.shape
    s = S()
    s.base, s.imageList, s.dtype, s.channels, s.numSamples = t.data_ptr(), None, dtype_code, c, n
    s.width, s.height = w, h
    s.rowStride, s.sampleStride = t.stride(1) * t.element_size(), t.stride(0) * t.element_size()
    return s


def _rects(rng, n, w, h):
    out = np.empty((n, 4), np.int32)
    for i in range(n):
        cw, ch = int(rng.integers(2, w + 1)), int(rng.integers(2, h + 1))
        out[i] = (int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch)
    return out


@pytest.mark.parametrize("dt,code", [(torch.uint8, 0), (torch.int16, 3)], ids=["u8", "s16"])
def test_no_alloc_matches_the_ordinary_entry_point_on_two_calls_in_a_row(pkg, dt, code):
    L, S = _bind(pkg)
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(2024)
    info = torch.iinfo(dt)
    for call, (n, interp) in enumerate(((7, 1), (3, 0))):  # the second call reuses the table with fewer entries
        src = torch.from_numpy(rng.integers(info.min, info.max + 1, (n, 61, 83, 3)).astype(
            np.uint8 if dt == torch.uint8 else np.int16)).cuda()
        rects = _rects(rng, n, 83, 61)
        want = torch.zeros((n, 40, 52, 3), dtype=dt, device="cuda")
        got = torch.zeros_like(want)
        dev_rects = torch.from_numpy(rects).cuda()  # the ordinary entry point: a device table the caller allocated
        s, dw, dg = _dense(S, src, code), _dense(S, want, code), _dense(S, got, code)
        assert L.b200ppResizedCrop(C.byref(s), C.byref(dw), dev_rects.data_ptr(), interp, stream) == 0, \
            L.b200ppGetLastErrorMessage()
        assert L.b200ppResizedCropNoAlloc(C.byref(s), C.byref(dg), rects.ctypes.data, interp, stream) == 0, \
            L.b200ppGetLastErrorMessage()
        torch.cuda.synchronize()
        assert want.cpu().numpy().any()
        assert np.array_equal(got.cpu().numpy(), want.cpu().numpy()), f"call {call}"


def test_no_alloc_refuses_more_images_than_its_table_holds(pkg):
    L, S = _bind(pkg)
    src = torch.zeros((1, 4, 4, 3), dtype=torch.uint8, device="cuda")
    dst = torch.zeros((1, 4, 4, 3), dtype=torch.uint8, device="cuda")
    s, d = _dense(S, src, 0), _dense(S, dst, 0)
    s.numSamples = d.numSamples = MAX_RECTS + 1  # refused before anything is read
    rects = np.zeros((1, 4), np.int32)
    st = L.b200ppResizedCropNoAlloc(C.byref(s), C.byref(d), rects.ctypes.data, 1, torch.cuda.current_stream().cuda_stream)
    assert st == pkg.ops.Status.ERROR_INVALID_ARGUMENT
    assert b"at most" in L.b200ppGetLastErrorMessage()
    assert L.b200ppResizedCropNoAlloc(C.byref(s), C.byref(d), None, 1, None) == pkg.ops.Status.ERROR_INVALID_ARGUMENT
