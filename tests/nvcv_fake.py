"""Test helper: builds and loads the object-model test double (tests/fake_nvcv) and wraps torch tensors / image
batches in handles the way the reference's libnvcv_types would export them."""
import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
SRC = os.path.join(HERE, "fake_nvcv", "fake_nvcv_types.cpp")
LIB = os.path.join(HERE, "fake_nvcv", "libfake_nvcv_types.so")

KIND = {"u": 0, "i": 1, "f": 2}


class TensorLayout(C.Structure):
    _fields_ = [("data", C.c_char * 16), ("rank", C.c_int32)]


class Strided(C.Structure):
    _fields_ = [("strides", C.c_int64 * 15), ("basePtr", C.c_void_p)]


class TensorData(C.Structure):
    _fields_ = [("dtype", C.c_uint64), ("layout", TensorLayout), ("rank", C.c_int32), ("shape", C.c_int64 * 15),
                ("bufferType", C.c_int32), ("strided", Strided)]


class VarShape(C.Structure):
    _fields_ = [("uniqueFormat", C.c_uint64), ("maxWidth", C.c_int32), ("maxHeight", C.c_int32),
                ("formatList", C.c_void_p), ("hostFormatList", C.c_void_p), ("imageList", C.c_void_p)]


class ImageBatchData(C.Structure):
    _fields_ = [("numImages", C.c_int32), ("bufferType", C.c_int32), ("varShapeStrided", VarShape)]


class Size2D(C.Structure):
    _fields_ = [("w", C.c_int32), ("h", C.c_int32)]


class Int2(C.Structure):
    _fields_ = [("x", C.c_int), ("y", C.c_int)]


assert C.sizeof(TensorData) == 288 and C.sizeof(ImageBatchData) == 48

_fake = None


class Float4(C.Structure):
    _fields_ = [("x", C.c_float), ("y", C.c_float), ("z", C.c_float), ("w", C.c_float)]


def fake():
    global _fake
    if _fake is None:
        if not os.path.exists(LIB) or os.path.getmtime(LIB) < os.path.getmtime(SRC):
            subprocess.check_call(["g++", "-std=c++17", "-O1", "-fPIC", "-shared", "-fvisibility=hidden",
                                   "-I" + os.path.join(ROOT, "include"), "-o", LIB, SRC])
        F = C.CDLL(LIB, mode=C.RTLD_GLOBAL)  # global: the operator library looks the nvcv* symbols up in the process
        F.fakeTensorCreate.restype = C.c_void_p
        F.fakeTensorCreate.argtypes = [C.POINTER(TensorData)]
        F.fakeTensorDestroy.argtypes = [C.c_void_p]
        F.fakeImageBatchCreate.restype = C.c_void_p
        F.fakeImageBatchCreate.argtypes = [C.POINTER(ImageBatchData)]
        F.fakeImageBatchCreateSized.restype = C.c_void_p
        F.fakeImageBatchCreateSized.argtypes = [C.POINTER(ImageBatchData), C.POINTER(C.c_int32)]
        F.fakeImageBatchDestroy.argtypes = [C.c_void_p]
        F.fakeLastStatus.restype = C.c_int
        F.fakeLastMessage.restype = C.c_char_p
        _fake = F
    return _fake


def dtype_code(kind: str, bits: int, channels: int = 1) -> int:
    return KIND[kind] | bits << 8 | channels << 16


def format_code(kind: str, bits: int, channels: int, planes: int) -> int:
    return KIND[kind] | bits << 8 | channels << 16 | planes << 24


def _kind_bits(t):
    import torch
    kind = "f" if t.dtype.is_floating_point else ("u" if t.dtype in (torch.uint8, getattr(torch, "uint16", None),
                                                                   getattr(torch, "uint32", None)) else "i")
    return kind, t.element_size() * 8


def tensor_handle(t, layout: str):
    """Handle of a torch tensor with the given layout string (e.g. "NHWC"); a raw address works for CPU-only checks."""
    d = TensorData()
    kind, bits = _kind_bits(t)
    d.dtype = dtype_code(kind, bits)
    d.layout.data = layout.encode()
    d.layout.rank = len(layout)
    d.rank = t.dim()
    for i in range(t.dim()):
        d.shape[i] = t.shape[i]
        d.strided.strides[i] = t.stride(i) * t.element_size()
    d.bufferType = 1
    d.strided.basePtr = t.data_ptr()
    return fake().fakeTensorCreate(C.byref(d))


def image_batch_handle(batch, kind="u", bits=8):
    """Handle of a package ImageBatchVarShape (its device descriptor table is what the real library would export)."""
    d = ImageBatchData()
    d.numImages = len(batch)
    d.bufferType = 1
    planes = batch.channels if batch.planar and batch.channels > 1 else 1
    d.varShapeStrided.uniqueFormat = format_code(kind, bits, batch.channels, planes)
    d.varShapeStrided.maxWidth, d.varShapeStrided.maxHeight = batch.max_size
    d.varShapeStrided.imageList = batch.descriptor_table().data_ptr()
    wh = [(im.shape[2], im.shape[1]) if batch.planar else (im.shape[1], im.shape[0]) for im in batch._images]
    sizes = (C.c_int32 * (2 * max(1, len(batch))))(*[v for pair in wh for v in pair])
    return fake().fakeImageBatchCreateSized(C.byref(d), sizes)


def bind_operators(lib_path: str):
    """The handle-based entry points of the operator library, with ctypes signatures."""
    fake()
    L = C.CDLL(lib_path)
    H = C.c_void_p
    L.cvcudaResizeCropConvertReformatCreate.restype = C.c_int
    L.cvcudaResizeCropConvertReformatCreate.argtypes = [C.POINTER(H)]
    L.cvcudaCropFlipNormalizeReformatCreate.restype = C.c_int
    L.cvcudaCropFlipNormalizeReformatCreate.argtypes = [C.POINTER(H)]
    L.nvcvOperatorDestroy.restype = None
    L.nvcvOperatorDestroy.argtypes = [H]
    for name in ("cvcudaResizeCropConvertReformatSubmit", "cvcudaResizeCropConvertReformatVarShapeSubmit"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [H, C.c_void_p, H, H, Size2D, C.c_int, Int2, C.c_int, C.c_float, C.c_float, C.c_bool]
    L.cvcudaResizeCreate.restype = C.c_int
    L.cvcudaResizeCreate.argtypes = [C.POINTER(H)]
    for name in ("cvcudaResizeSubmit", "cvcudaResizeVarShapeSubmit"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [H, C.c_void_p, H, H, C.c_int]
    L.cvcudaConvertToCreate.restype = C.c_int
    L.cvcudaConvertToCreate.argtypes = [C.POINTER(H)]
    L.cvcudaConvertToSubmit.restype = C.c_int
    L.cvcudaConvertToSubmit.argtypes = [H, C.c_void_p, H, H, C.c_double, C.c_double]
    L.cvcudaCopyMakeBorderCreate.restype = C.c_int
    L.cvcudaCopyMakeBorderCreate.argtypes = [C.POINTER(H)]
    L.cvcudaCopyMakeBorderSubmit.restype = C.c_int
    L.cvcudaCopyMakeBorderSubmit.argtypes = [H, C.c_void_p, H, H, C.c_int32, C.c_int32, C.c_int, Float4]
    for name in ("cvcudaCopyMakeBorderVarShapeSubmit", "cvcudaCopyMakeBorderVarShapeStackSubmit"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [H, C.c_void_p, H, H, H, H, C.c_int, Float4]
    L.cvcudaRandomResizedCropCreate.restype = C.c_int
    L.cvcudaRandomResizedCropCreate.argtypes = [C.POINTER(H), C.c_double, C.c_double, C.c_double, C.c_double, C.c_int32, C.c_uint32]
    for name in ("cvcudaRandomResizedCropSubmit", "cvcudaRandomResizedCropVarShapeSubmit"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [H, C.c_void_p, H, H, C.c_int]
    L.cvcudaReformatCreate.restype = C.c_int
    L.cvcudaReformatCreate.argtypes = [C.POINTER(H)]
    L.cvcudaReformatSubmit.restype = C.c_int
    L.cvcudaReformatSubmit.argtypes = [H, C.c_void_p, H, H]
    L.cvcudaNormalizeCreate.restype = C.c_int
    L.cvcudaNormalizeCreate.argtypes = [C.POINTER(H)]
    for name in ("cvcudaNormalizeSubmit", "cvcudaNormalizeVarShapeSubmit"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [H, C.c_void_p, H, H, H, H, C.c_float, C.c_float, C.c_float, C.c_uint32]
    L.cvcudaCropFlipNormalizeReformatSubmit.restype = C.c_int
    L.cvcudaCropFlipNormalizeReformatSubmit.argtypes = [H, C.c_void_p, H, H, H, C.c_int, C.c_float, H, H, H, C.c_float,
                                                        C.c_float, C.c_float, C.c_uint32]
    return L
