"""CPU: the handle-based operator entry points (the reference's exported symbols) -- creation, destruction, handle
checks and argument validation, which all happen before any CUDA call -- against an object-model test double."""
import ctypes as C
import os
import subprocess

import pytest
import torch

import nvcv_fake as NF

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INVALID_ARGUMENT, NOT_COMPATIBLE = 2, 9


@pytest.fixture(scope="module")
def ops(pkg):
    return NF.bind_operators(pkg.lib_path())


def _cpu_tensor(shape, dtype):
    return torch.zeros(shape, dtype=dtype)


def test_create_with_null_pointer_is_invalid_argument(ops):
    """TestOpResizeCropConvertReformat.cpp:608-611 (createWillNullPtr)."""
    assert ops.cvcudaResizeCropConvertReformatCreate(None) == INVALID_ARGUMENT
    assert ops.cvcudaCropFlipNormalizeReformatCreate(None) == INVALID_ARGUMENT
    assert NF.fake().fakeLastStatus() == INVALID_ARGUMENT


def test_create_destroy_and_handle_kind(ops):
    h1, h2 = C.c_void_p(), C.c_void_p()
    assert ops.cvcudaResizeCropConvertReformatCreate(C.byref(h1)) == 0 and h1.value
    assert ops.cvcudaCropFlipNormalizeReformatCreate(C.byref(h2)) == 0 and h2.value
    t = NF.tensor_handle(_cpu_tensor((1, 8, 8, 3), torch.uint8), "NHWC")
    args = (None, t, t, NF.Size2D(16, 16), 1, NF.Int2(0, 0), 0, 1.0, 0.0, True)
    # NULL handle -> INVALID_ARGUMENT; a handle of the other operator -> NOT_COMPATIBLE (priv/IOperator.hpp:56-73)
    assert ops.cvcudaResizeCropConvertReformatSubmit(None, *args) == INVALID_ARGUMENT
    assert ops.cvcudaResizeCropConvertReformatSubmit(h2, *args) == NOT_COMPATIBLE
    assert b"requested object" in NF.fake().fakeLastMessage()
    ops.nvcvOperatorDestroy(h1)
    ops.nvcvOperatorDestroy(h2)
    ops.nvcvOperatorDestroy(None)


@pytest.mark.parametrize("in_layout,out_layout,in_dtype,out_dtype,in_shape,out_shape,status", [
    ("NCHW", "NHWC", torch.uint8, torch.uint8, (2, 3, 32, 32), (2, 4, 4, 3), NOT_COMPATIBLE),  # planar input layout
    ("NHWC", "NHWC", torch.uint8, torch.uint8, (1, 32, 32, 3), (2, 4, 4, 3), INVALID_ARGUMENT),  # batch mismatch
    ("NHWC", "NHWC", torch.uint8, torch.uint8, (2, 32, 32, 3), (2, 4, 4, 4), NOT_COMPATIBLE),  # channel mismatch
    ("NHWC", "NHWC", torch.uint8, torch.uint8, (2, 32, 32, 4), (2, 4, 4, 4), NOT_COMPATIBLE),  # not 3 channels
    ("NHWC", "NHWC", torch.float32, torch.uint8, (2, 32, 32, 3), (2, 4, 4, 3), NOT_COMPATIBLE),  # input not uchar
    ("NHWC", "NHWC", torch.uint8, torch.float16, (2, 32, 32, 3), (2, 4, 4, 3), NOT_COMPATIBLE),  # f16 output refused
    ("NHWC", "NWHC", torch.uint8, torch.uint8, (2, 32, 32, 3), (2, 4, 4, 3), NOT_COMPATIBLE),  # output layout
])
def test_tensor_submit_validation(ops, in_layout, out_layout, in_dtype, out_dtype, in_shape, out_shape, status):
    h = C.c_void_p()
    assert ops.cvcudaResizeCropConvertReformatCreate(C.byref(h)) == 0
    src, dst = _cpu_tensor(in_shape, in_dtype), _cpu_tensor(out_shape, out_dtype)
    ti, to = NF.tensor_handle(src, in_layout), NF.tensor_handle(dst, out_layout)
    got = ops.cvcudaResizeCropConvertReformatSubmit(h, None, ti, to, NF.Size2D(16, 16), 1, NF.Int2(0, 0), 0, 1.0, 0.0, True)
    assert got == status and NF.fake().fakeLastStatus() == status
    ops.nvcvOperatorDestroy(h)


@pytest.mark.parametrize("interp,crop,out_wh,resize", [
    (2, (0, 0), (4, 4), (16, 16)), (3, (0, 0), (4, 4), (16, 16)), (4, (0, 0), (4, 4), (16, 16)),
    (1, (-1, 0), (4, 4), (16, 16)), (1, (0, -1), (4, 4), (16, 16)), (1, (0, 0), (32, 4), (16, 16)),
    (1, (0, 0), (4, 32), (16, 16)), (1, (0, 0), (4, 4), (0, 0)),
])
def test_geometry_validation_is_invalid_argument(ops, interp, crop, out_wh, resize):
    """Interpolation, crop range and resize-dimension rows of the reference's negative table (:578-602)."""
    h = C.c_void_p()
    assert ops.cvcudaResizeCropConvertReformatCreate(C.byref(h)) == 0
    src = _cpu_tensor((2, 32, 32, 3), torch.uint8)
    dst = _cpu_tensor((2, out_wh[1], out_wh[0], 3), torch.uint8)
    ti, to = NF.tensor_handle(src, "NHWC"), NF.tensor_handle(dst, "NHWC")
    got = ops.cvcudaResizeCropConvertReformatSubmit(h, None, ti, to, NF.Size2D(*resize), interp, NF.Int2(*crop), 0, 1.0,
                                                    0.0, True)
    assert got == INVALID_ARGUMENT
    ops.nvcvOperatorDestroy(h)


def test_struct_layouts_match_the_reference_headers():
    """sizeof/offsetof of the restated object-model structs against the reference's own headers (when present)."""
    ref = os.environ.get("CVCUDA_REFERENCE_ROOT", "/root/reference")
    inc = os.path.join(ref, "src/nvcv/src/include")
    if not os.path.exists(os.path.join(inc, "nvcv/TensorData.h")):
        pytest.skip("reference headers not available on this machine")
    body = r'''
#include <stddef.h>
#include <stdio.h>
int main(void) {
  printf("%zu %zu %zu %zu %zu %zu %zu\n", sizeof(NVCVTensorData), offsetof(NVCVTensorData, layout), offsetof(NVCVTensorData, rank),
         offsetof(NVCVTensorData, shape), offsetof(NVCVTensorData, bufferType), OFF_STRIDES, OFF_BASE);
  printf("%zu %zu %zu %zu %zu\n", sizeof(NVCVImageBatchData), OFF_FMT, OFF_MAXW, OFF_HOSTFMT, OFF_LIST);
  printf("%zu %zu %zu %zu\n", sizeof(IMGBUF), offsetof(IMGBUF, planes), sizeof(IMGPLANE), offsetof(IMGPLANE, basePtr));
  printf("%zu %zu\n", sizeof(NVCVSize2D), sizeof(NVCVTensorLayout));
  return 0; }'''
    theirs = ('#include <nvcv/TensorData.h>\n#include <nvcv/ImageBatchData.h>\n#include <nvcv/Size.h>\n'
              '#define OFF_STRIDES offsetof(NVCVTensorData, buffer.strided.strides)\n'
              '#define OFF_BASE offsetof(NVCVTensorData, buffer.strided.basePtr)\n'
              '#define OFF_FMT offsetof(NVCVImageBatchData, buffer.varShapeStrided.uniqueFormat)\n'
              '#define OFF_MAXW offsetof(NVCVImageBatchData, buffer.varShapeStrided.maxWidth)\n'
              '#define OFF_HOSTFMT offsetof(NVCVImageBatchData, buffer.varShapeStrided.hostFormatList)\n'
              '#define OFF_LIST offsetof(NVCVImageBatchData, buffer.varShapeStrided.imageList)\n'
              '#define IMGBUF NVCVImageBufferStrided\n#define IMGPLANE NVCVImagePlaneStrided\n')
    ours = ('#include <cvcuda_b200/cvcuda_ops.h>\n'
            '#define OFF_STRIDES offsetof(NVCVTensorData, strided.strides)\n'
            '#define OFF_BASE offsetof(NVCVTensorData, strided.basePtr)\n'
            '#define OFF_FMT offsetof(NVCVImageBatchData, varShapeStrided.uniqueFormat)\n'
            '#define OFF_MAXW offsetof(NVCVImageBatchData, varShapeStrided.maxWidth)\n'
            '#define OFF_HOSTFMT offsetof(NVCVImageBatchData, varShapeStrided.hostFormatList)\n'
            '#define OFF_LIST offsetof(NVCVImageBatchData, varShapeStrided.imageList)\n'
            '#define IMGBUF B200ppImageBuffer\n#define IMGPLANE B200ppImagePlane\n')
    outs = []
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        for name, head, incs in (("theirs", theirs, [inc]), ("ours", ours, [os.path.join(ROOT, "include")])):
            src = os.path.join(tmp, name + ".c")
            exe = os.path.join(tmp, name)
            open(src, "w").write(head + body)
            subprocess.check_call(["gcc", "-std=c11", *("-I" + i for i in incs), "-o", exe, src])
            outs.append(subprocess.check_output([exe], text=True))
    assert outs[0] == outs[1], f"reference:\n{outs[0]}\nthis library:\n{outs[1]}"
