"""GPU parity through the reference's own operator symbols (cvcuda...Create / Submit, nvcvOperatorDestroy): handles are
unpacked by the object-model test double, values come from the CUDA kernels and are compared with the CPU oracle."""
import ctypes as C

import numpy as np
import pytest
import torch

import nvcv_fake as NF
import ref_tables as T
from gpu_util import _TORCH_DTYPE, assert_parity, padded_images, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops(pkg):
    return NF.bind_operators(pkg.lib_path())


def _stream():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("idx", [0, 7, 10, 24, 30, 41, 45, 52, 54, 57, 60, 61])
def test_rccr_tensor_submit(ops, oracle, idx):
    r = T.RCCR_ROWS[idx]
    w, h, n = r.src
    n = min(n, 2)
    src = np.random.default_rng(idx).integers(0, 256, (n, h, w, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=r.resize, crop=r.crop, out_size=r.out, interp=r.interp, src_cast=r.src_cast,
                             manip=r.manip, scale=r.scale, offset=r.offset)
    want = oracle.resize_crop(list(src), spec, r.dtype, r.planar, nthreads=4)
    tsrc = to_dev(src)
    shape = (n, 3, r.out[1], r.out[0]) if r.planar else (n, r.out[1], r.out[0], 3)
    tdst = torch.empty(shape, dtype=_TORCH_DTYPE[np.dtype(r.dtype)], device="cuda")
    h_op = C.c_void_p()
    assert ops.cvcudaResizeCropConvertReformatCreate(C.byref(h_op)) == 0
    hi, ho = NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NCHW" if r.planar else "NHWC")
    st = ops.cvcudaResizeCropConvertReformatSubmit(h_op, _stream(), hi, ho, NF.Size2D(*r.resize), r.interp,
                                                   NF.Int2(*r.crop), r.manip, r.scale, r.offset, r.src_cast)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    assert_parity(tdst.cpu().numpy(), want, exact=(r.interp == 0), what=f"row {idx}")
    ops.nvcvOperatorDestroy(h_op)


@pytest.mark.parametrize("idx", [3, 9, 31, 44, 57])
def test_rccr_varshape_submit(pkg, ops, oracle, idx):
    r = T.RCCR_ROWS[idx]
    w, h, n = r.src
    rng = np.random.default_rng(idx)
    images = [rng.integers(0, 256, (int(h * s), int(w * s), 3), dtype=np.uint8) for s in (0.8, 1.0, 1.2)]
    spec = oracle.ResizeSpec(resize=r.resize, crop=r.crop, out_size=r.out, interp=r.interp, src_cast=r.src_cast,
                             manip=r.manip, scale=r.scale, offset=r.offset)
    want = oracle.resize_crop(images, spec, r.dtype, r.planar, nthreads=4)
    batch = pkg.ImageBatchVarShape(padded_images(images))
    shape = (3, 3, r.out[1], r.out[0]) if r.planar else (3, r.out[1], r.out[0], 3)
    tdst = torch.empty(shape, dtype=_TORCH_DTYPE[np.dtype(r.dtype)], device="cuda")
    h_op = C.c_void_p()
    assert ops.cvcudaResizeCropConvertReformatCreate(C.byref(h_op)) == 0
    hb, ho = NF.image_batch_handle(batch), NF.tensor_handle(tdst, "NCHW" if r.planar else "NHWC")
    st = ops.cvcudaResizeCropConvertReformatVarShapeSubmit(h_op, _stream(), hb, ho, NF.Size2D(*r.resize), r.interp,
                                                           NF.Int2(*r.crop), r.manip, r.scale, r.offset, r.src_cast)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    assert_parity(tdst.cpu().numpy(), want, exact=(r.interp == 0), what=f"row {idx}")
    ops.nvcvOperatorDestroy(h_op)


@pytest.mark.parametrize("idx", range(len(T.CFNR_ROWS)))
def test_cfnr_submit(pkg, ops, oracle, idx):
    row = T.CFNR_ROWS[idx]
    if np.dtype(row.src_dtype) not in _TORCH_DTYPE or np.dtype(row.dst_dtype) not in _TORCH_DTYPE:
        pytest.skip("no such torch tensor type")
    images, rects, flips, base, scale, osz = T.cfnr_case(row, seed=77 + idx)
    want = oracle.crop_flip_normalize(images, row.src_planar, rects, flips, osz, row.dst_dtype, row.dst_planar,
                                      row.border, 1.0, base, scale, row.gscale, row.gshift, row.eps, row.flags)
    n = len(images)
    batch = pkg.ImageBatchVarShape(padded_images(images, planar=row.src_planar), planar=row.src_planar)
    shape = (n, row.channels, osz[1], osz[0]) if row.dst_planar else (n, osz[1], osz[0], row.channels)
    tdst = torch.empty(shape, dtype=_TORCH_DTYPE[np.dtype(row.dst_dtype)], device="cuda")
    trect = to_dev(rects.reshape(n, 1, 1, 4))
    tflip = to_dev(flips)
    tbase, tscale = to_dev(base.reshape(1, 1, 1, -1)), to_dev(scale.reshape(1, 1, 1, -1))
    kind = "f" if np.dtype(row.src_dtype).kind == "f" else ("u" if np.dtype(row.src_dtype).kind == "u" else "i")
    h_op = C.c_void_p()
    assert ops.cvcudaCropFlipNormalizeReformatCreate(C.byref(h_op)) == 0
    st = ops.cvcudaCropFlipNormalizeReformatSubmit(
        h_op, _stream(), NF.image_batch_handle(batch, kind, np.dtype(row.src_dtype).itemsize * 8),
        NF.tensor_handle(tdst, "NCHW" if row.dst_planar else "NHWC"), NF.tensor_handle(trect, "NHWC"), row.border, 1.0,
        NF.tensor_handle(tflip, "N"), NF.tensor_handle(tbase, "NHWC"), NF.tensor_handle(tscale, "NHWC"), row.gscale,
        row.gshift, row.eps, row.flags)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    assert_parity(tdst.cpu().numpy(), want, what=f"row {idx}")
    ops.nvcvOperatorDestroy(h_op)


def test_cfnr_submit_refuses_tensors_it_would_overrun_or_misread(pkg, ops):
    """An output with fewer samples or channels than the batch, flipCode / cropRect that are not int32 or hold too few
    entries, base / scale that are not float32: INVALID_ARGUMENT before anything is launched. (The reference's typed
    accessors would read or write past the tensors, src/cvcuda/priv/OpCropFlipNormalizeReformat.cu:208-215,264-267.)"""
    rng = np.random.default_rng(3)
    images = [rng.integers(0, 256, (20, 24, 3), dtype=np.uint8) for _ in range(3)]
    batch = pkg.ImageBatchVarShape(padded_images(images))
    good = dict(out=torch.zeros((3, 3, 16, 16), dtype=torch.float32, device="cuda"),
                rect=to_dev(np.tile(np.asarray([0, 0, 16, 16], np.int32), (3, 1)).reshape(3, 1, 1, 4)),
                flip=to_dev(np.zeros(3, np.int32)), base=to_dev(np.zeros((1, 1, 1, 3), np.float32)),
                scale=to_dev(np.ones((1, 1, 1, 3), np.float32)))
    h_op = C.c_void_p()
    assert ops.cvcudaCropFlipNormalizeReformatCreate(C.byref(h_op)) == 0

    def submit(**over):
        a = dict(good, **over)
        st = ops.cvcudaCropFlipNormalizeReformatSubmit(
            h_op, _stream(), NF.image_batch_handle(batch, "u", 8), NF.tensor_handle(a["out"], "NCHW"),
            NF.tensor_handle(a["rect"], "NHWC"), 0, 0.0, NF.tensor_handle(a["flip"], "N"), NF.tensor_handle(a["base"], "NHWC"),
            NF.tensor_handle(a["scale"], "NHWC"), 1.0, 0.0, 0.0, 0)
        torch.cuda.synchronize()
        return st

    assert submit() == 0, NF.fake().fakeLastMessage()
    bad = [dict(out=torch.zeros((2, 3, 16, 16), dtype=torch.float32, device="cuda")),
           dict(out=torch.zeros((3, 2, 16, 16), dtype=torch.float32, device="cuda")),
           dict(flip=to_dev(np.zeros(2, np.int32))),
           dict(flip=to_dev(np.zeros(3, np.float32))),
           dict(rect=to_dev(np.zeros((2, 1, 1, 4), np.int32))),
           dict(rect=to_dev(np.zeros((3, 1, 1, 2), np.int32))),
           dict(rect=to_dev(np.zeros((3, 1, 1, 4), np.float32))),
           dict(base=to_dev(np.zeros((1, 1, 1, 3), np.int32))),
           dict(scale=to_dev(np.zeros((1, 1, 1, 3), np.uint8)))]
    for over in bad:
        assert submit(**over) == 2, f"accepted {list(over)}"
    ops.nvcvOperatorDestroy(h_op)
