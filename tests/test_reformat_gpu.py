"""GPU parity of the stand-alone Reformat. The reference's CPU golden is an element-wise copy
dst(b, y, x, c) = src(b, y, x, c) between layouts (tests/cvcuda/system/TestOpReformat.cpp:51-69), which for packed
arrays is numpy's transpose: results must be bit-equal. Rows of the reference's table (:76-86), other element types,
strided views, argument errors, and the reference's own operator symbols."""
import ctypes as C

import numpy as np
import pytest
import torch

import nvcv_fake as NF
from gpu_util import _TORCH_DTYPE, to_dev

pytestmark = pytest.mark.gpu

# width, height, batches, input planar?, output planar?, channels, element type   (TestOpReformat.cpp:76-86)
ROWS = [(176, 113, 1, False, False, 3, np.uint8), (23, 43, 23, True, True, 3, np.uint8), (7, 4, 7, False, False, 3, np.float32),
        (3, 2, 1, True, False, 3, np.uint8), (2, 3, 1, False, True, 3, np.uint8), (56, 49, 2, True, False, 4, np.uint8),
        (56, 49, 3, False, True, 3, np.uint8), (31, 30, 3, False, True, 4, np.float32), (30, 31, 3, True, False, 3, np.float32)]


def _data(rng, shape, dt):
    if np.dtype(dt).kind == "f":
        lim = 6e4 if np.dtype(dt) == np.float16 else 1e6
        return rng.uniform(-lim, lim, shape).astype(dt)
    info = np.iinfo(dt)
    return rng.integers(info.min, int(info.max) + 1, shape).astype(dt)


def _golden(src, src_layout, dst_layout):
    return np.ascontiguousarray(np.transpose(src, [src_layout.index(k) for k in dst_layout]))


@pytest.mark.parametrize("row", ROWS, ids=lambda r: f"{r[0]}x{r[1]}x{r[2]}-{'p' if r[3] else 'i'}to{'p' if r[4] else 'i'}-{r[5]}x{np.dtype(r[6]).name}")
def test_reformat_rows(pkg, row):
    w, h, n, pin, pout, ch, dt = row
    rng = np.random.default_rng(w * h)
    sl, dl = ("NCHW" if pin else "NHWC"), ("NCHW" if pout else "NHWC")
    src = _data(rng, (n, ch, h, w) if pin else (n, h, w, ch), dt)
    got = pkg.reformat(to_dev(src), dl, src_layout=sl)
    torch.cuda.synchronize()
    want = _golden(src, sl, dl)
    assert got.shape == want.shape and np.array_equal(got.cpu().numpy().view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("dt", [np.int8, np.uint16, np.int16, np.int32, np.float16, np.float32], ids=lambda d: np.dtype(d).name)
def test_reformat_types_rank3_and_views(pkg, dt):
    """Rank-3 layouts, 1 to 5 channels, int32 values beyond float32's exact range (the copy must not go through float),
    strided source and destination views."""
    rng = np.random.default_rng(3)
    for ch in (1, 2, 5):
        src = _data(rng, (21, 34, ch), dt)
        got = pkg.reformat(to_dev(src), "CHW", src_layout="HWC")
        torch.cuda.synchronize()
        assert np.array_equal(got.cpu().numpy().view(np.uint8), _golden(src, "HWC", "CHW").view(np.uint8))
    big = _data(rng, (2, 3, 9, 40), dt)
    tsrc = to_dev(big)[:, :, 1:8, 3:37]
    store = torch.zeros((2, 9, 40, 3), dtype=_TORCH_DTYPE[np.dtype(dt)], device="cuda")
    pkg.reformat_into(store[:, 1:8, 2:36], tsrc, src_layout="NCHW", dst_layout="NHWC")
    torch.cuda.synchronize()
    out = store.cpu().numpy()
    assert np.array_equal(out[:, 1:8, 2:36].view(np.uint8), _golden(big[:, :, 1:8, 3:37], "NCHW", "NHWC").view(np.uint8))
    out[:, 1:8, 2:36] = 0
    assert not out.view(np.uint8).any(), "wrote outside the destination view"


@pytest.mark.parametrize("dt", [np.uint8, np.float32, np.int32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("to_planar", [True, False], ids=["to-planar", "to-interleaved"])
def test_reformat_rgb_vector_kernels(pkg, to_planar, dt):
    """Three channels of 8 or 32 bits between packed interleaved and planar with every row on a 16-byte boundary take the
    vector kernels (16 or 4 pixels per thread); kernel path 1 keeps the word-per-channel kernel on the same data. Widths
    with and without a ragged end (views of wider storage keep the rows aligned), heights that end inside a thread's pair of rows."""
    from gpu_util import kernel_path
    rng = np.random.default_rng(11)
    TD = _TORCH_DTYPE[np.dtype(dt)]
    for (n, h, w, W) in ((2, 37, 528, 528), (3, 5, 16, 16), (2, 9, 45, 64), (1, 1, 7, 16), (2, 18, 1000, 1008)):
        data = _data(rng, (n, h, w, 3), dt)  # logical NHWC content
        if to_planar:
            src = torch.zeros((n, h, W, 3), dtype=TD, device="cuda")
            src[:, :, :w] = to_dev(data)
            src_view, sl, dl = src[:, :, :w], "NHWC", "NCHW"
            store = torch.zeros((n, 3, h, W), dtype=TD, device="cuda")
            dst_view = store[:, :, :, :w]
            want = np.transpose(data, (0, 3, 1, 2))
        else:
            src = torch.zeros((n, 3, h, W), dtype=TD, device="cuda")
            src[:, :, :, :w] = to_dev(np.ascontiguousarray(np.transpose(data, (0, 3, 1, 2))))
            src_view, sl, dl = src[:, :, :, :w], "NCHW", "NHWC"
            store = torch.zeros((n, h, W, 3), dtype=TD, device="cuda")
            dst_view = store[:, :, :w]
            want = data
        for path in (0, 1):
            store.zero_()
            with kernel_path(pkg, path):
                pkg.reformat_into(dst_view, src_view, src_layout=sl, dst_layout=dl)
            torch.cuda.synchronize()
            assert np.array_equal(dst_view.cpu().numpy().view(np.uint8), np.ascontiguousarray(want).view(np.uint8)), (n, h, w, W, path)
            rest = store.clone()
            if to_planar:
                rest[:, :, :, :w] = 0
            else:
                rest[:, :, :w] = 0
            assert not rest.any().item(), "wrote outside the destination view"


def test_reformat_errors(pkg):
    INVALID = pkg.ops.Status.ERROR_INVALID_ARGUMENT
    a = torch.zeros((2, 4, 5, 3), dtype=torch.uint8, device="cuda")
    for bad in (lambda: pkg.reformat_into(torch.zeros((2, 3, 4, 5), dtype=torch.int8, device="cuda"), a, dst_layout="NCHW"),
                lambda: pkg.reformat_into(torch.zeros((2, 3, 4, 6), dtype=torch.uint8, device="cuda"), a, dst_layout="NCHW"),
                lambda: pkg.reformat_into(torch.zeros((1, 3, 4, 5), dtype=torch.uint8, device="cuda"), a, dst_layout="NCHW"),
                lambda: pkg.reformat_into(torch.zeros((3, 4, 5), dtype=torch.uint8, device="cuda"), a, dst_layout="CHW"),
                lambda: pkg.reformat(a, "NWHC")):
        with pytest.raises(pkg.ops.Error) as e:
            bad()
        assert e.value.status == INVALID
    assert pkg.reformat(torch.empty((0, 4, 5, 3), dtype=torch.uint8, device="cuda"), "NCHW").shape == (0, 3, 4, 5)


def test_reformat_through_operator_symbols(pkg):
    ops = NF.bind_operators(pkg.lib_path())
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(8)
    src = _data(rng, (2, 4, 49, 56), np.uint8)
    tsrc, tdst = to_dev(src), torch.empty((2, 49, 56, 4), dtype=torch.uint8, device="cuda")
    h_op = C.c_void_p()
    assert ops.cvcudaReformatCreate(C.byref(h_op)) == 0
    st = ops.cvcudaReformatSubmit(h_op, stream, NF.tensor_handle(tsrc, "NCHW"), NF.tensor_handle(tdst, "NHWC"))
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    assert np.array_equal(tdst.cpu().numpy(), _golden(src, "NCHW", "NHWC"))
    # element types differ, ranks differ, another operator's handle
    f32 = torch.empty((2, 49, 56, 4), dtype=torch.float32, device="cuda")
    assert ops.cvcudaReformatSubmit(h_op, stream, NF.tensor_handle(tsrc, "NCHW"), NF.tensor_handle(f32, "NHWC")) == 2
    hwc = torch.empty((49, 56, 4), dtype=torch.uint8, device="cuda")
    assert ops.cvcudaReformatSubmit(h_op, stream, NF.tensor_handle(tsrc, "NCHW"), NF.tensor_handle(hwc, "HWC")) == 2
    other = C.c_void_p()
    assert ops.cvcudaNormalizeCreate(C.byref(other)) == 0
    assert ops.cvcudaReformatSubmit(other, stream, NF.tensor_handle(tsrc, "NCHW"), NF.tensor_handle(tdst, "NHWC")) == 9
    ops.nvcvOperatorDestroy(other)
    ops.nvcvOperatorDestroy(h_op)
