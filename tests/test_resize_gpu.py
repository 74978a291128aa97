"""GPU parity of the stand-alone Resize (nearest / linear) against the CPU oracle, through the plain-C entry point, the
Python mirror and the reference's own operator symbols: the nearest / linear rows of the reference's test table
(tensor and variable-shape forms), every element type x channel count, odd strides, degenerate sizes, and the
reference's negative table. Integer element types must be bit-exact (the kernel does the golden's double-precision
arithmetic); float32 is compared bit for bit with the oracle's un-rounded form."""
import ctypes as C

import numpy as np
import pytest
import torch

import nvcv_fake as NF
import ref_tables as T
from gpu_util import _TORCH_DTYPE, padded_images, to_dev

pytestmark = pytest.mark.gpu


def _image(rng, w, h, ch, dt):
    if dt == np.float32:
        return rng.uniform(0.0, 300.0, (h, w, ch)).astype(np.float32)
    info = np.iinfo(dt)
    return rng.integers(info.min, info.max + 1, (h, w, ch)).astype(dt)


def _same(a, b, what):
    assert a.shape == b.shape and a.dtype == b.dtype, what
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{what}: {int((a != b).sum())} differing elements"


def _row_id(r):
    return f"{r.src_w}x{r.src_h}-{r.dst_w}x{r.dst_h}-i{r.interp}-n{r.images}-{r.channels}x{np.dtype(r.dtype).name}"


@pytest.mark.parametrize("row", T.RESIZE_ROWS, ids=_row_id)
def test_resize_tensor_rows(pkg, oracle, row):
    rng = np.random.default_rng(11)
    images = [_image(rng, row.src_w, row.src_h, row.channels, row.dtype) for _ in range(row.images)]
    want = np.stack(oracle.resize_plain(images, [(row.dst_w, row.dst_h)] * row.images, row.interp))
    src = to_dev(np.stack(images))
    got = pkg.resize(src, (row.images, row.dst_h, row.dst_w, row.channels), row.interp)
    torch.cuda.synchronize()
    _same(got.cpu().numpy(), want, "tensor")


@pytest.mark.parametrize("row", T.RESIZE_ROWS, ids=_row_id)
def test_resize_varshape_rows(pkg, oracle, row):
    """Per-image source and destination sizes from 0.8x to 1.1x of the row's, as the reference's var-shape test draws
    them (tests/cvcuda/system/TestOpResize.cpp:211-226)."""
    rng = np.random.default_rng(13)
    n = max(row.images, 3)
    big = row.src_w * row.src_h > 500000
    div = 4 if big else 1  # the largest rows at a quarter of their size: the oracle is a plain double loop
    def draw(v):
        return int(rng.integers(max(1, int(v // div * 0.8)), max(2, int(v // div * 1.1)) + 1))
    images = [_image(rng, draw(row.src_w), draw(row.src_h), row.channels, row.dtype) for _ in range(n)]
    sizes = [(draw(row.dst_w), draw(row.dst_h)) for _ in range(n)]
    want = oracle.resize_plain(images, sizes, row.interp)
    src = pkg.ImageBatchVarShape(padded_images(images, pad_to=32))
    got = pkg.resize(src, sizes, row.interp)
    torch.cuda.synchronize()
    for i in range(n):
        _same(got[i].cpu().numpy(), want[i], f"image {i}")


@pytest.mark.parametrize("dt", [np.uint8, np.uint16, np.int16, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("ch", [1, 3, 4])
@pytest.mark.parametrize("interp", [0, 1])
def test_resize_types_channels_strides(pkg, oracle, dt, ch, interp):
    """Up- and down-scaling, rows padded to odd pitches and bases off any vector alignment, strided output views."""
    rng = np.random.default_rng(100 * ch + interp)
    images = [_image(rng, 37, 29, ch, dt), _image(rng, 64, 5, ch, dt), _image(rng, 3, 50, ch, dt)]
    sizes = [(50, 41), (9, 40), (31, 7)]
    want = oracle.resize_plain(images, sizes, interp)
    es = np.dtype(dt).itemsize
    src = pkg.ImageBatchVarShape(padded_images(images, pad_to=es, offset=es))
    dst_store = [torch.zeros((h + 2, w + 3, ch), dtype=_TORCH_DTYPE[np.dtype(dt)], device="cuda") for (w, h) in sizes]
    dst = pkg.ImageBatchVarShape([t[1:1 + h, 2:2 + w] for t, (w, h) in zip(dst_store, sizes)])
    pkg.resize_into(dst, src, interp)
    torch.cuda.synchronize()
    for i in range(3):
        _same(dst[i].cpu().numpy(), want[i], f"image {i}")
        frame = dst_store[i].cpu().numpy().copy()
        frame[1:1 + sizes[i][1], 2:2 + sizes[i][0]] = 0
        assert not frame.any(), "wrote outside the destination view"


def test_resize_negative_int16_keeps_its_sign(pkg, oracle):
    """Linear interpolation of negative int16 data gives negative results, as the reference's CUDA operators do
    (src/cvcuda/priv/OpResize.cu:228-262 saturate-cast the signed blend). The reference's CPU golden rounds |blend|
    (tests/cvcuda/system/ResizeUtils.cpp:226) and would answer +100 for an image of -100; its tests never run int16 with
    linear interpolation. Tensor and variable-shape forms, Resize and the resized crop of RandomResizedCrop."""
    rng = np.random.default_rng(17)
    flat = np.full((2, 20, 24, 3), -100, np.int16)
    got = pkg.resize(to_dev(flat), (2, 31, 45, 3), 1).cpu().numpy()
    assert np.all(got == -100)
    images = [rng.integers(-32768, 0, (h, w, 3)).astype(np.int16) for (w, h) in ((33, 21), (18, 40))]
    sizes = [(50, 30), (11, 17)]
    want = oracle.resize_plain(images, sizes, 1)
    assert all((w < 0).all() for w in want)
    got = pkg.resize(pkg.ImageBatchVarShape(padded_images(images, pad_to=32)), sizes, 1)
    torch.cuda.synchronize()
    for i in range(2):
        _same(got[i].cpu().numpy(), want[i], f"var-shape image {i}")
    same = [rng.integers(-32768, 0, (26, 35, 3)).astype(np.int16) for _ in range(2)]
    _same(pkg.resize(to_dev(np.stack(same)), (2, 40, 29, 3), 1).cpu().numpy(),
          np.stack(oracle.resize_plain(same, [(29, 40)] * 2, 1)), "tensor")
    rects = [(3, 2, 20, 15), (0, 5, 35, 11)]
    want = oracle.resize_plain(same, [(16, 12)] * 2, 1, rects=rects)
    assert all((w < 0).all() for w in want)
    out = torch.empty((2, 12, 16, 3), dtype=torch.int16, device="cuda")
    pkg.resized_crop_into(out, to_dev(np.stack(same)), to_dev(np.asarray(rects, np.int32)), 1)
    torch.cuda.synchronize()
    _same(out.cpu().numpy(), np.stack(want), "resized crop")


def test_resize_degenerate_sizes(pkg, oracle):
    """1x1 sources and destinations; identity; sources one pixel wide or high with linear interpolation, where the
    reference golden itself would read outside the image: the result must be the replicated pixel row / column."""
    rng = np.random.default_rng(5)
    one = _image(rng, 1, 1, 3, np.uint8)
    got = pkg.resize(to_dev(one[None]), (1, 7, 9, 3), 1)
    assert np.array_equal(got.cpu().numpy()[0], np.broadcast_to(one, (7, 9, 3)))
    got = pkg.resize(to_dev(one[None]), (1, 7, 9, 3), 0)
    assert np.array_equal(got.cpu().numpy()[0], np.broadcast_to(one, (7, 9, 3)))
    col = _image(rng, 1, 13, 4, np.uint8)
    got = pkg.resize(to_dev(col[None]), (1, 13, 5, 4), 1).cpu().numpy()[0]
    assert np.array_equal(got, np.broadcast_to(col, (13, 5, 4)))
    im = _image(rng, 40, 30, 3, np.uint16)
    for interp in (0, 1):
        got = pkg.resize(to_dev(im[None]), (1, 30, 40, 3), interp).cpu().numpy()[0]
        assert np.array_equal(got, im), "identity resize"
        tiny = pkg.resize(to_dev(im[None]), (1, 1, 1, 3), interp).cpu().numpy()[0]
        _same(tiny, oracle.resize_plain([im], [(1, 1)], interp)[0], "to 1x1")
    empty = pkg.resize(torch.empty((0, 8, 8, 3), dtype=torch.uint8, device="cuda"), (0, 4, 4, 3), 1)
    assert empty.shape == (0, 4, 4, 3)


def test_resize_negative_table(pkg):
    """Status codes of the reference's negative table (tests/cvcuda/system/TestOpResize.cpp:317-356): all
    NVCV_ERROR_INVALID_ARGUMENT; cubic and area are refused as not implemented."""
    u8 = torch.zeros((1, 8, 8, 3), dtype=torch.uint8, device="cuda")
    def status(fn):
        with pytest.raises(pkg.ops.Error) as e:
            fn()
        return e.value.status
    INVALID = pkg.ops.Status.ERROR_INVALID_ARGUMENT
    assert status(lambda: pkg.resize_into(torch.zeros((1, 4, 4, 3), dtype=torch.int16, device="cuda"), u8, 0)) == INVALID
    assert status(lambda: pkg.resize_into(torch.zeros((2, 4, 4, 3), dtype=torch.uint8, device="cuda"), u8, 0)) == INVALID
    assert status(lambda: pkg.resize_into(torch.zeros((1, 4, 4, 1), dtype=torch.uint8, device="cuda"), u8, 0)) == INVALID
    assert status(lambda: pkg.resize_into(torch.zeros((1, 4, 4, 2), dtype=torch.uint8, device="cuda"),
                                          torch.zeros((1, 8, 8, 2), dtype=torch.uint8, device="cuda"), 0)) == INVALID
    f16 = torch.zeros((1, 8, 8, 3), dtype=torch.float16, device="cuda")
    assert status(lambda: pkg.resize_into(torch.zeros((1, 4, 4, 3), dtype=torch.float16, device="cuda"), f16, 0)) == INVALID
    assert status(lambda: pkg.resize_into(torch.zeros((1, 4, 4, 3), dtype=torch.uint8, device="cuda"), u8, 7)) == INVALID
    for interp in (2, 3):
        assert status(lambda: pkg.resize_into(torch.zeros((1, 4, 4, 3), dtype=torch.uint8, device="cuda"), u8, interp)) \
            == pkg.ops.Status.ERROR_NOT_IMPLEMENTED


def test_resize_through_operator_symbols(pkg, oracle):
    """cvcudaResizeCreate / Submit / VarShapeSubmit on handles of the object-model test double."""
    ops = NF.bind_operators(pkg.lib_path())
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(21)
    h_op = C.c_void_p()
    assert ops.cvcudaResizeCreate(C.byref(h_op)) == 0
    images = [_image(rng, 42, 48, 4, np.uint8) for _ in range(2)]
    src, dst = to_dev(np.stack(images)), torch.empty((2, 24, 23, 4), dtype=torch.uint8, device="cuda")
    for interp in (0, 1):
        st = ops.cvcudaResizeSubmit(h_op, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(dst, "NHWC"), interp)
        assert st == 0, NF.fake().fakeLastMessage()
        torch.cuda.synchronize()
        _same(dst.cpu().numpy(), np.stack(oracle.resize_plain(images, [(23, 24)] * 2, interp)), "tensor handles")
    # layouts differ, data types differ, another operator's handle, NULL handle
    chw = torch.empty((2, 4, 24, 23), dtype=torch.uint8, device="cuda")
    assert ops.cvcudaResizeSubmit(h_op, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(chw, "NCHW"), 1) == 2
    s16 = torch.empty((2, 24, 23, 4), dtype=torch.int16, device="cuda")
    assert ops.cvcudaResizeSubmit(h_op, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(s16, "NHWC"), 1) == 2
    assert ops.cvcudaResizeSubmit(None, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(dst, "NHWC"), 1) == 2
    other = C.c_void_p()
    assert ops.cvcudaCropFlipNormalizeReformatCreate(C.byref(other)) == 0
    assert ops.cvcudaResizeSubmit(other, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(dst, "NHWC"), 1) == 9
    ops.nvcvOperatorDestroy(other)

    sizes = [(30, 17), (8, 40)]
    batch_in = pkg.ImageBatchVarShape(padded_images(images))
    batch_out = pkg.ImageBatchVarShape([torch.empty((h, w, 4), dtype=torch.uint8, device="cuda") for (w, h) in sizes])
    st = ops.cvcudaResizeVarShapeSubmit(h_op, stream, NF.image_batch_handle(batch_in), NF.image_batch_handle(batch_out), 1)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    want = oracle.resize_plain(images, sizes, 1)
    for i in range(2):
        _same(batch_out[i].cpu().numpy(), want[i], f"batch handles, image {i}")
    ops.nvcvOperatorDestroy(h_op)
