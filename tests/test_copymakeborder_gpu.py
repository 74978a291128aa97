"""GPU parity of the stand-alone CopyMakeBorder against the CPU restatement of the reference's golden
(tests/cvcuda/system/TestOpCopyMakeBorder.cpp:40-97, border index rules tests/common/BorderUtils.cpp): the reference's own
parameter table in its three forms (tensor, variable-shape batch, variable-shape batch stacked into a tensor), every border
rule on every element type and channel count with rows off any word alignment, degenerate sizes, the reference's
negative table, and its operator symbols. Results are bit-exact: the operator copies elements."""
import ctypes as C

import numpy as np
import pytest
import torch

import nvcv_fake as NF
from gpu_util import _TORCH_DTYPE, padded_images, to_dev

pytestmark = pytest.mark.gpu

CONSTANT, REPLICATE, REFLECT, WRAP, REFLECT101 = range(5)
# srcWidth, srcHeight, batch, top, bottom, left, right, border, value, dtype, channels (TestOpCopyMakeBorder.cpp:230-243)
REF_ROWS = [
    (212, 113, 1, 0, 0, 0, 0, CONSTANT, (0, 0, 0, 0), np.uint8, 3),
    (12, 13, 2, 12, 16, 0, 3, CONSTANT, (12, 100, 245, 0), np.uint8, 3),
    (212, 113, 3, 0, 113, 5, 0, CONSTANT, (13, 5, 4, 0), np.uint8, 3),
    (212, 613, 4, 19, 20, 7, 7, CONSTANT, (255, 255, 255, 0), np.uint8, 3),
    (234, 131, 2, 44, 55, 33, 22, REPLICATE, (0, 0, 0, 0), np.uint8, 3),
    (234, 131, 2, 33, 20, 41, 42, REFLECT, (0, 0, 0, 0), np.uint8, 4),
    (234, 131, 2, 100, 85, 53, 62, WRAP, (0, 0, 0, 0), np.float32, 3),
    (243, 123, 2, 56, 123, 77, 98, REFLECT101, (0, 0, 0, 0), np.float32, 4),
]


def _image(rng, w, h, ch, dt):
    if dt == np.float32:
        return (rng.integers(0, 256, (h, w, ch)) / 255.0).astype(np.float32)
    info = np.iinfo(dt)
    return rng.integers(info.min, int(info.max) + 1, (h, w, ch)).astype(dt)


def _same(a, b, what):
    assert a.shape == b.shape and a.dtype == b.dtype, what
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{what}: {int((a != b).sum())} differing elements"


def _row_id(r):
    return f"{r[0]}x{r[1]}n{r[2]}-t{r[3]}b{r[4]}l{r[5]}r{r[6]}-m{r[7]}-{np.dtype(r[9]).name}x{r[10]}"


@pytest.mark.parametrize("row", REF_ROWS, ids=_row_id)
def test_reference_table_tensor(pkg, oracle, row):
    w, h, n, top, bottom, left, right, border, value, dt, ch = row
    rng = np.random.default_rng(0)
    batch = np.stack([_image(rng, w, h, ch, dt) for _ in range(n)])
    want = np.stack(oracle.copy_make_border(list(batch), [(w + left + right, h + top + bottom)] * n, top, left, border, value))
    got = pkg.copymakeborder(to_dev(batch), border, value, top=top, bottom=bottom, left=left, right=right)
    torch.cuda.synchronize()
    _same(got.cpu().numpy(), want, "tensor form")


@pytest.mark.parametrize("row", REF_ROWS, ids=_row_id)
def test_reference_table_varshape_and_stack(pkg, oracle, row):
    """The variable-shape tests of the reference draw each image's size below the row's size and each top / left inside
    the padding (TestOpCopyMakeBorder.cpp:330-420, :480-570); same here with this file's generator."""
    w, h, n, top, bottom, left, right, border, value, dt, ch = row
    rng = np.random.default_rng(1)
    ow, oh = w + left + right, h + top + bottom
    images = [_image(rng, int(rng.integers(max(1, w // 2), w + 1)), int(rng.integers(max(1, h // 2), h + 1)), ch, dt)
              for _ in range(n)]
    tops = np.array([int(rng.integers(0, oh - im.shape[0] + 1)) for im in images], np.int32)
    lefts = np.array([int(rng.integers(0, ow - im.shape[1] + 1)) for im in images], np.int32)
    src = pkg.ImageBatchVarShape(padded_images(images, pad_to=32))
    ttop, tleft = to_dev(tops), to_dev(lefts)
    # stacked into one tensor
    want = oracle.copy_make_border(images, [(ow, oh)] * n, tops, lefts, border, value)
    got = pkg.copymakeborderstack(src, border, value, top=ttop, left=tleft, out_height=oh, out_width=ow)
    torch.cuda.synchronize()
    _same(got.cpu().numpy(), np.stack(want), "stack form")
    # into a variable-shape batch with its own sizes
    sizes = [(int(rng.integers(im.shape[1] + l, ow + 1)), int(rng.integers(im.shape[0] + t, oh + 1)))
             for im, t, l in zip(images, tops, lefts)]
    want = oracle.copy_make_border(images, sizes, tops, lefts, border, value)
    got = pkg.copymakeborder(src, border, value, top=ttop, left=tleft, out_heights=[s[1] for s in sizes],
                             out_widths=[s[0] for s in sizes])
    torch.cuda.synchronize()
    for i in range(n):
        _same(got[i].cpu().numpy(), want[i], f"var-shape image {i}")


@pytest.mark.parametrize("dt", [np.uint8, np.int8, np.uint16, np.int16, np.int32, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("ch", [1, 2, 3, 4])
@pytest.mark.parametrize("border", [CONSTANT, REPLICATE, REFLECT, WRAP, REFLECT101])
def test_types_channels_borders_alignment(pkg, oracle, dt, ch, border):
    """Borders several times wider than the image (the index rules wrap more than once), images one pixel wide or high,
    source rows at odd pitches and bases, destination views inside larger buffers (nothing outside may change)."""
    rng = np.random.default_rng(10 * ch + border)
    images = [_image(rng, 37, 29, ch, dt), _image(rng, 5, 3, ch, dt), _image(rng, 1, 9, ch, dt), _image(rng, 11, 1, ch, dt)]
    sizes = [(61, 40), (33, 31), (7, 20), (40, 6)]
    tops = np.array([4, 13, 5, 2], np.int32)
    lefts = np.array([9, 14, 3, 17], np.int32)
    value = (3.7, 250.2, -20.5, 99.0)
    want = oracle.copy_make_border(images, sizes, tops, lefts, border, value)
    es = np.dtype(dt).itemsize
    for pad, off in ((32, 0), (es, es)):
        src = pkg.ImageBatchVarShape(padded_images(images, pad_to=pad, offset=off))
        store = [torch.zeros((h + 2, w + 3, ch), dtype=_TORCH_DTYPE[np.dtype(dt)], device="cuda") for (w, h) in sizes]
        dst = pkg.ImageBatchVarShape([t[1:1 + h, 2:2 + w] for t, (w, h) in zip(store, sizes)])
        pkg.copymakeborder_into(dst, src, border, value, top=to_dev(tops), left=to_dev(lefts))
        torch.cuda.synchronize()
        for i in range(len(images)):
            _same(dst[i].cpu().numpy(), want[i], f"image {i} (pad {pad}, offset {off})")
            frame = store[i].cpu().numpy().copy()
            frame[1:1 + sizes[i][1], 2:2 + sizes[i][0]] = 0
            assert not frame.view(np.uint8).any(), "wrote outside the destination view"


def test_offsets_outside_and_empty(pkg, oracle):
    """Per-sample top / left may place the image partly or wholly outside the destination (the variable-shape forms of
    the reference do not check them): the visible part is copied, the rest follows the border rule. Empty batches and
    rank-3 tensors are accepted."""
    rng = np.random.default_rng(3)
    images = [_image(rng, 20, 10, 3, np.uint8) for _ in range(4)]
    tops = np.array([-3, 8, -30, 40], np.int32)
    lefts = np.array([-5, 15, 2, -60], np.int32)
    src = pkg.ImageBatchVarShape(padded_images(images, pad_to=4))
    for border in (CONSTANT, REPLICATE, REFLECT, WRAP, REFLECT101):
        want = oracle.copy_make_border(images, [(24, 16)] * 4, tops, lefts, border, (9, 8, 7, 0))
        got = pkg.copymakeborderstack(src, border, (9, 8, 7), top=to_dev(tops), left=to_dev(lefts), out_height=16, out_width=24)
        torch.cuda.synchronize()
        _same(got.cpu().numpy(), np.stack(want), f"border {border}")
    hwc = _image(rng, 9, 7, 4, np.int16)
    got = pkg.copymakeborder(to_dev(hwc), REFLECT101, top=2, bottom=3, left=4, right=1)
    _same(got.cpu().numpy(), oracle.copy_make_border([hwc], [(14, 12)], 2, 4, REFLECT101)[0], "rank 3")
    empty = pkg.copymakeborder(torch.empty((0, 4, 4, 3), dtype=torch.uint8, device="cuda"), top=1, bottom=1, left=1, right=1)
    assert empty.shape == (0, 6, 6, 3)
    # border values outside the element range saturate; fractions drop toward zero
    one = np.zeros((1, 1, 1, 4), np.uint8)
    got = pkg.copymakeborder(to_dev(one), CONSTANT, (300.0, -4.0, 7.9, 255.5), top=1, bottom=0, left=0, right=0).cpu().numpy()
    assert got[0, 0, 0].tolist() == [255, 0, 7, 255]


def test_negative_table(pkg):
    """Status codes of the reference's negative table (TestOpCopyMakeBorder.cpp:654-664): all NVCV_ERROR_INVALID_ARGUMENT."""
    INVALID = pkg.ops.Status.ERROR_INVALID_ARGUMENT

    def status(fn):
        with pytest.raises(pkg.ops.Error) as e:
            fn()
        return e.value.status

    u8 = torch.zeros((1, 24, 24, 1), dtype=torch.uint8, device="cuda")
    out = torch.zeros((1, 24, 24, 1), dtype=torch.uint8, device="cuda")
    assert status(lambda: pkg.copymakeborder_into(torch.zeros((1, 24, 24, 1), dtype=torch.int16, device="cuda"), u8,
                                                  top=0, left=0)) == INVALID
    f16 = torch.zeros((1, 24, 24, 1), dtype=torch.float16, device="cuda")
    assert status(lambda: pkg.copymakeborder_into(torch.zeros_like(f16), f16, top=0, left=0)) == INVALID
    assert status(lambda: pkg.copymakeborder_into(out, u8, 255, top=0, left=0)) == INVALID
    assert status(lambda: pkg.copymakeborder_into(out, u8, top=-1, left=0)) == INVALID
    assert status(lambda: pkg.copymakeborder_into(out, u8, top=0, left=-1)) == INVALID
    assert status(lambda: pkg.copymakeborder_into(out, u8, top=1, left=0)) == INVALID  # bottom would be negative
    assert status(lambda: pkg.copymakeborder_into(torch.zeros((2, 24, 24, 1), dtype=torch.uint8, device="cuda"), u8,
                                                  top=0, left=0)) == INVALID
    assert status(lambda: pkg.copymakeborder_into(torch.zeros((1, 24, 24, 3), dtype=torch.uint8, device="cuda"), u8,
                                                  top=0, left=0)) == INVALID
    assert status(lambda: pkg.copymakeborder_into(out, u8, 0, (1, 2, 3, 4, 5), top=0, left=0)) == INVALID
    batch = pkg.ImageBatchVarShape([u8[0]])
    zero = torch.zeros(1, dtype=torch.int32, device="cuda")
    assert status(lambda: pkg.copymakeborder_into(out, batch, top=zero.float(), left=zero)) == INVALID
    assert status(lambda: pkg.copymakeborder_into(batch, u8, top=0, left=0)) == INVALID


def test_through_operator_symbols(pkg, oracle):
    """cvcudaCopyMakeBorderCreate / Submit / VarShapeSubmit / VarShapeStackSubmit on handles of the object-model test
    double; top / left tensors as the reference's tests build them ([1, 1, N, 1] int32 NHWC)."""
    ops = NF.bind_operators(pkg.lib_path())
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(8)
    h_op = C.c_void_p()
    assert ops.cvcudaCopyMakeBorderCreate(None) == 2
    assert ops.cvcudaCopyMakeBorderCreate(C.byref(h_op)) == 0
    value = NF.Float4(12.0, 100.0, 245.0, 0.0)
    batch = np.stack([_image(rng, 30, 20, 3, np.uint8) for _ in range(2)])
    tsrc, tdst = to_dev(batch), torch.empty((2, 31, 40, 3), dtype=torch.uint8, device="cuda")
    st = ops.cvcudaCopyMakeBorderSubmit(h_op, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), 4, 6,
                                        CONSTANT, value)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    _same(tdst.cpu().numpy(), np.stack(oracle.copy_make_border(list(batch), [(40, 31)] * 2, 4, 6, CONSTANT, (12, 100, 245, 0))),
          "tensor handles")
    # negative rows: planar layouts, mismatched types, bad border, negative top / left
    chw = torch.empty((2, 3, 20, 30), dtype=torch.uint8, device="cuda")
    assert ops.cvcudaCopyMakeBorderSubmit(h_op, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(chw, "NCHW"), 0, 0,
                                          CONSTANT, value) == 2
    assert ops.cvcudaCopyMakeBorderSubmit(h_op, stream, NF.tensor_handle(chw, "NCHW"), NF.tensor_handle(chw, "NCHW"), 0, 0,
                                          CONSTANT, value) == 2
    assert ops.cvcudaCopyMakeBorderSubmit(h_op, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), 0, 0,
                                          255, value) == 2
    assert ops.cvcudaCopyMakeBorderSubmit(h_op, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), -1, 0,
                                          CONSTANT, value) == 2

    images = [_image(rng, 17, 23, 4, np.uint8), _image(rng, 40, 9, 4, np.uint8), _image(rng, 8, 8, 4, np.uint8)]
    tops, lefts = np.array([3, 0, 11], np.int32), np.array([5, 2, 0], np.int32)
    bin_ = pkg.ImageBatchVarShape(padded_images(images, pad_to=32))
    ttop = to_dev(tops).reshape(1, 1, 3, 1)
    tleft = to_dev(lefts).reshape(1, 1, 3, 1)
    stack = torch.empty((3, 30, 44, 4), dtype=torch.uint8, device="cuda")
    st = ops.cvcudaCopyMakeBorderVarShapeStackSubmit(h_op, stream, NF.image_batch_handle(bin_), NF.tensor_handle(stack, "NHWC"),
                                                     NF.tensor_handle(ttop, "NHWC"), NF.tensor_handle(tleft, "NHWC"), WRAP, value)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    _same(stack.cpu().numpy(), np.stack(oracle.copy_make_border(images, [(44, 30)] * 3, tops, lefts, WRAP)), "stack handles")
    sizes = [(25, 30), (44, 12), (9, 20)]
    bout = pkg.ImageBatchVarShape([torch.empty((h, w, 4), dtype=torch.uint8, device="cuda") for (w, h) in sizes])
    st = ops.cvcudaCopyMakeBorderVarShapeSubmit(h_op, stream, NF.image_batch_handle(bin_), NF.image_batch_handle(bout),
                                                NF.tensor_handle(ttop, "NHWC"), NF.tensor_handle(tleft, "NHWC"), REFLECT, value)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    want = oracle.copy_make_border(images, sizes, tops, lefts, REFLECT)
    for i in range(3):
        _same(bout[i].cpu().numpy(), want[i], f"var-shape handles, image {i}")
    # top / left of the wrong element type
    ftop = ttop.float()
    assert ops.cvcudaCopyMakeBorderVarShapeSubmit(h_op, stream, NF.image_batch_handle(bin_), NF.image_batch_handle(bout),
                                                  NF.tensor_handle(ftop, "NHWC"), NF.tensor_handle(tleft, "NHWC"), REFLECT,
                                                  value) == 2
    other = C.c_void_p()
    assert ops.cvcudaReformatCreate(C.byref(other)) == 0
    assert ops.cvcudaCopyMakeBorderSubmit(other, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), 4, 6,
                                          CONSTANT, value) == 9
    ops.nvcvOperatorDestroy(other)
    ops.nvcvOperatorDestroy(h_op)
