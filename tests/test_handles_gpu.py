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
