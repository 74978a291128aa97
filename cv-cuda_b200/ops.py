"""Host-side mirror of the reference's Python operator interface for the fused pre-processing path.

Function names, argument names and meaning follow the reference binding
(python/mod_cvcuda/OpResizeCropConvertReformat.cpp:207-420, python/mod_cvcuda/OpCropFlipNormalizeReformat.cpp:86-165);
tensors are ``torch`` CUDA tensors instead of ``nvcv.Tensor`` objects, and a variable-shape batch is an
:class:`ImageBatchVarShape` of CUDA tensors. PyTorch only provides device memory and streams here: every value is
computed by ``libcvcuda_b200.so`` through its plain-C entry points (``include/cvcuda_b200/preproc.h``).
"""
from __future__ import annotations

import ctypes as C
import enum
import os
from typing import List, NamedTuple, Optional, Sequence, Tuple, Union

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_NAME = "libcvcuda_b200.so"


# ------------------------------------------------------------------------------------------------ enums / small types

class Interp(enum.IntEnum):
    """NVCVInterpolationType (src/cvcuda/include/cvcuda/Types.h:39-51)."""
    NEAREST = 0
    LINEAR = 1
    CUBIC = 2
    AREA = 3
    LANCZOS = 4


class ChannelManip(enum.IntEnum):
    """NVCVChannelManip (Types.h:63-67)."""
    NO_OP = 0
    REVERSE = 1


class Border(enum.IntEnum):
    """NVCVBorderType (src/nvcv/src/include/nvcv/BorderType.h:36-43)."""
    CONSTANT = 0
    REPLICATE = 1
    REFLECT = 2
    WRAP = 3
    REFLECT101 = 4


NORMALIZE_SCALE_IS_STDDEV = 1


class RectI(NamedTuple):
    """nvcv.RectI: x, y, width, height."""
    x: int
    y: int
    width: int
    height: int


class Status(enum.IntEnum):
    SUCCESS = 0
    ERROR_NOT_IMPLEMENTED = 1
    ERROR_INVALID_ARGUMENT = 2
    ERROR_INVALID_IMAGE_FORMAT = 3
    ERROR_INTERNAL = 8
    ERROR_NOT_COMPATIBLE = 9
    ERROR_OVERFLOW = 10


class Error(RuntimeError):
    """A failed operator call; ``status`` holds the NVCVStatus code the C entry point returned."""

    def __init__(self, status: int, message: str):
        try:
            name = Status(status).name
        except ValueError:
            name = str(status)
        super().__init__(f"NVCV_{name}: {message}")
        self.status = status
        self.message = message


# ------------------------------------------------------------------------------------------------ C structs

class _ImagePlane(C.Structure):
    _fields_ = [("width", C.c_int32), ("height", C.c_int32), ("rowStride", C.c_int32), ("basePtr", C.c_void_p)]


class _ImageBuffer(C.Structure):
    _fields_ = [("numPlanes", C.c_int32), ("planes", _ImagePlane * 6)]


class _Source(C.Structure):
    _fields_ = [("dtype", C.c_int32), ("channels", C.c_int32), ("planar", C.c_int32), ("numSamples", C.c_int32),
                ("base", C.c_void_p), ("sampleStride", C.c_int64), ("rowStride", C.c_int64),
                ("planeStride", C.c_int64), ("width", C.c_int32), ("height", C.c_int32),
                ("imageList", C.c_void_p), ("maxWidth", C.c_int32), ("maxHeight", C.c_int32)]


class _Dest(C.Structure):
    _fields_ = [("base", C.c_void_p), ("dtype", C.c_int32), ("channels", C.c_int32), ("width", C.c_int32),
                ("height", C.c_int32), ("sampleStride", C.c_int64), ("rowStride", C.c_int64),
                ("pixStride", C.c_int64), ("chanStride", C.c_int64)]


class _ResizeOp(C.Structure):
    _fields_ = [("resizeW", C.c_int32), ("resizeH", C.c_int32), ("cropX", C.c_int32), ("cropY", C.c_int32),
                ("interp", C.c_int32), ("srcCast", C.c_int32), ("manip", C.c_int32), ("perChannel", C.c_int32),
                ("scale", C.c_float), ("offset", C.c_float), ("base", C.c_float * 4), ("mul", C.c_float * 4),
                ("gscale", C.c_float), ("shift", C.c_float),
                ("dstX", C.c_int32), ("dstY", C.c_int32), ("regionW", C.c_int32), ("regionH", C.c_int32),
                ("padValue", C.c_float),
                ("roi", C.c_void_p), ("roiStride", C.c_int64), ("flipCode", C.c_void_p)]


class _SliceOp(C.Structure):
    _fields_ = [("cropRect", C.c_void_p), ("cropRectStride", C.c_int64), ("flipCode", C.c_void_p),
                ("border", C.c_int32), ("borderValue", C.c_float),
                ("base", C.c_void_p), ("baseChannels", C.c_int32), ("baseChanStride", C.c_int64),
                ("scale", C.c_void_p), ("scaleChannels", C.c_int32), ("scaleChanStride", C.c_int64),
                ("gscale", C.c_float), ("shift", C.c_float), ("epsilon", C.c_float), ("flags", C.c_uint32)]


class _ImageSet(C.Structure):
    _fields_ = [("base", C.c_void_p), ("imageList", C.c_void_p), ("dtype", C.c_int32), ("channels", C.c_int32),
                ("numSamples", C.c_int32), ("width", C.c_int32), ("height", C.c_int32), ("maxWidth", C.c_int32),
                ("maxHeight", C.c_int32), ("rowStride", C.c_int64), ("sampleStride", C.c_int64)]


class _NormalizeOp(C.Structure):
    _fields_ = [("base", C.c_void_p), ("baseStride", C.c_int64 * 4), ("scale", C.c_void_p), ("scaleStride", C.c_int64 * 4),
                ("gscale", C.c_float), ("shift", C.c_float), ("epsilon", C.c_float), ("flags", C.c_uint32)]


assert C.sizeof(_ImagePlane) == 24 and C.sizeof(_ImageBuffer) == 152  # NVCVImageBufferStrided layout

_DTYPE_CODE = {torch.uint8: 0, torch.int8: 1, torch.int16: 3, torch.int32: 5, torch.float32: 6, torch.float16: 7}
for _name, _code in (("uint16", 2), ("uint32", 4)):
    if hasattr(torch, _name):
        _DTYPE_CODE[getattr(torch, _name)] = _code


# ------------------------------------------------------------------------------------------------ library

_lib: Optional[C.CDLL] = None


def lib_path() -> str:
    return os.path.join(_HERE, _LIB_NAME)


def lib() -> C.CDLL:
    """The CUDA library. Raises if it has not been built: there is no other implementation to fall back to."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise RuntimeError(f"{path} is missing: run `python cv-cuda_b200/build.py` (or __graft_entry__.build()). "
                               "This package has no CPU or PyTorch fallback.")
        L = C.CDLL(path)
        L.b200ppResizeCropConvertReformat.restype = C.c_int
        L.b200ppResizeCropConvertReformat.argtypes = [C.POINTER(_Source), C.POINTER(_Dest), C.POINTER(_ResizeOp),
                                                      C.c_void_p]
        L.b200ppCropFlipNormalizeReformat.restype = C.c_int
        L.b200ppCropFlipNormalizeReformat.argtypes = [C.POINTER(_Source), C.POINTER(_Dest), C.POINTER(_SliceOp),
                                                      C.c_void_p]
        L.b200ppGetLastErrorMessage.restype = C.c_char_p
        L.b200ppSetKernelPath.restype = C.c_int
        L.b200ppResize.restype = C.c_int
        L.b200ppResize.argtypes = [C.POINTER(_ImageSet), C.POINTER(_ImageSet), C.c_int32, C.c_void_p]
        L.b200ppNormalize.restype = C.c_int
        L.b200ppNormalize.argtypes = [C.POINTER(_ImageSet), C.POINTER(_ImageSet), C.POINTER(_NormalizeOp), C.c_void_p]
        L.b200ppReformat.restype = C.c_int
        L.b200ppReformat.argtypes = [C.POINTER(_Dest), C.POINTER(_Dest), C.c_int32, C.c_void_p]
        L.b200ppRandomCropCreate.restype = C.c_int
        L.b200ppRandomCropCreate.argtypes = [C.POINTER(C.c_void_p), C.c_double, C.c_double, C.c_double, C.c_double, C.c_uint32]
        L.b200ppRandomCropDestroy.restype = None
        L.b200ppRandomCropDestroy.argtypes = [C.c_void_p]
        L.b200ppRandomCropNext.restype = C.c_int
        L.b200ppRandomCropNext.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.POINTER(C.c_int32)]
        L.b200ppResizedCrop.restype = C.c_int
        L.b200ppResizedCrop.argtypes = [C.POINTER(_ImageSet), C.POINTER(_ImageSet), C.c_void_p, C.c_int32, C.c_void_p]
        L.b200ppCopyMakeBorder.restype = C.c_int
        L.b200ppCopyMakeBorder.argtypes = [C.POINTER(_ImageSet), C.POINTER(_ImageSet), C.c_int32, C.c_int32, C.c_void_p,
                                           C.c_void_p, C.c_int32, C.POINTER(C.c_float), C.c_void_p]
        L.b200ppConvertTo.restype = C.c_int
        L.b200ppConvertTo.argtypes = [C.POINTER(_ImageSet), C.POINTER(_ImageSet), C.c_double, C.c_double, C.c_void_p]
        L.b200ppSetKernelPath.argtypes = [C.c_int]
        L.b200ppGetLaunchCount.restype = C.c_uint64
        L.b200ppReadDeviceError.restype = C.c_int
        L.b200ppReadDeviceError.argtypes = [C.POINTER(C.c_uint32)]
        L.b200ppSelfTestWaitTimeout.restype = C.c_int
        L.b200ppSelfTestWaitTimeout.argtypes = [C.c_uint32, C.c_void_p]
        _lib = L
    return _lib


def last_error() -> str:
    return lib().b200ppGetLastErrorMessage().decode()


def set_kernel_path(path: int) -> int:
    """0 automatic, 1 per-pixel gather kernels, 2 staged kernels where they apply. Returns the previous setting."""
    return lib().b200ppSetKernelPath(int(path))


def launch_count() -> int:
    return int(lib().b200ppGetLaunchCount())


def read_device_error() -> int:
    v = C.c_uint32(0)
    _check(lib().b200ppReadDeviceError(C.byref(v)))
    return int(v.value)


def self_test_wait_timeout(limit_ms: int = 20, stream=None) -> None:
    """Launches the bounded-wait self-test (a wait that must give up after `limit_ms`)."""
    _check(lib().b200ppSelfTestWaitTimeout(int(limit_ms), _stream_handle(stream)))


def _check(status: int) -> None:
    if status != 0:
        raise Error(status, last_error())


def _stream_handle(stream) -> int:
    if stream is None:
        return torch.cuda.current_stream().cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


# ------------------------------------------------------------------------------------------------ tensor views

class ImageBatchVarShape:
    """A batch of images of different sizes, the counterpart of nvcv.ImageBatchVarShape.

    Images are CUDA tensors: ``[H, W, C]`` (interleaved) or ``[C, H, W]`` (planar, ``planar=True``), innermost dimension
    contiguous, rows possibly padded. The device-side descriptor table has the memory layout of
    ``NVCVImageBufferStrided[]`` (src/nvcv/src/include/nvcv/ImageData.h:52-66) and is uploaded when first needed after
    a change, like ``ImageBatchVarShape::exportData`` does (src/nvcv/src/priv/ImageBatchVarShape.cpp:215-254).
    """

    def __init__(self, images: Sequence[torch.Tensor] = (), planar: bool = False):
        self.planar = planar
        self._images = []
        self._table = None
        self._max_size = None
        self.pushback(images)

    def pushback(self, images: Union[torch.Tensor, Sequence[torch.Tensor]]) -> None:
        if isinstance(images, torch.Tensor):
            images = [images]
        for im in images:
            if im.dim() != 3 or not (im.is_cuda or im.is_pinned()):
                raise Error(Status.ERROR_INVALID_ARGUMENT, "Images must be 3-D CUDA (or page-locked host) tensors")
            if im.stride(2) != 1 or (not self.planar and im.stride(1) != im.shape[2]):
                raise Error(Status.ERROR_INVALID_ARGUMENT, "Image pixels must be contiguous within a row")
            if self._images and (im.dtype != self._images[0].dtype or self._channels(im) != self.channels):
                raise Error(Status.ERROR_INVALID_ARGUMENT,
                            "All input images in a batch must have the same format (including number of channels)")
            self._images.append(im)
        self._table = None
        self._max_size = None

    def popback(self, count: int = 1) -> None:
        """Removes the last `count` images (nvcv.ImageBatchVarShape.popback)."""
        if count < 0 or count > len(self._images):
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Cannot remove more images than the batch holds")
        if count:
            del self._images[-count:]
            self._table = None
            self._max_size = None

    def clear(self) -> None:
        self._images = []
        self._table = None
        self._max_size = None

    def _channels(self, im: torch.Tensor) -> int:
        return im.shape[0] if self.planar else im.shape[2]

    def __len__(self) -> int:
        return len(self._images)

    def __getitem__(self, i: int) -> torch.Tensor:
        return self._images[i]

    @property
    def channels(self) -> int:
        return self._channels(self._images[0])

    @property
    def dtype(self) -> torch.dtype:
        return self._images[0].dtype

    @property
    def device(self) -> torch.device:
        d = self._images[0].device
        return d if d.type == "cuda" else torch.device("cuda", torch.cuda.current_device())

    def size(self, i: int) -> Tuple[int, int]:
        im = self._images[i]
        return (im.shape[2], im.shape[1]) if self.planar else (im.shape[1], im.shape[0])

    @property
    def max_size(self) -> Tuple[int, int]:
        # kept with the batch like the reference keeps its maxSize (src/nvcv/src/priv/ImageBatchVarShape.cpp:215-254): an
        # operator call must not walk the images
        if self._max_size is None:
            sizes = [self.size(i) for i in range(len(self))]
            self._max_size = (max(s[0] for s in sizes), max(s[1] for s in sizes))
        return self._max_size

    def descriptor_table(self) -> torch.Tensor:
        """uint8 CUDA tensor holding ``NVCVImageBufferStrided[len(self)]``."""
        if self._table is None:
            arr = (_ImageBuffer * len(self._images))()
            for i, im in enumerate(self._images):
                es = im.element_size()
                if self.planar:
                    c, h, w = im.shape
                    arr[i].numPlanes = c
                    for k in range(c):
                        arr[i].planes[k] = _ImagePlane(w, h, im.stride(1) * es, im.data_ptr() + k * im.stride(0) * es)
                else:
                    h, w, c = im.shape
                    arr[i].numPlanes = 1
                    arr[i].planes[0] = _ImagePlane(w, h, im.stride(0) * es, im.data_ptr())
            host = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).pin_memory()
            # a blocking copy: the table is complete before this returns, so a kernel launched on any stream sees it
            # (the launch stream is the caller's choice and need not be torch's current stream)
            self._table = host.to(self.device, non_blocking=False)
        return self._table


def _device_accessible(t: torch.Tensor) -> bool:
    """CUDA memory, or page-locked host memory (which the GPU addresses directly under unified addressing)."""
    return t.is_cuda or t.is_pinned()


def _source_of(src: Union[torch.Tensor, ImageBatchVarShape]):
    """Returns (struct, keepalive)."""
    s = _Source()
    if isinstance(src, ImageBatchVarShape):
        if len(src) == 0:
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Input image batch is empty")
        table = src.descriptor_table()
        s.dtype = _DTYPE_CODE[src.dtype]
        s.channels, s.planar, s.numSamples = src.channels, int(src.planar), len(src)
        s.imageList = table.data_ptr()
        s.maxWidth, s.maxHeight = src.max_size
        return s, table
    if not _device_accessible(src):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input must be a cuda-accessible, pitch-linear tensor")
    t = src if src.dim() == 4 else src.unsqueeze(0)
    if t.dim() != 4:
        raise Error(Status.ERROR_NOT_COMPATIBLE, "Input tensor must have 'NHWC' or 'HWC' layout")
    n, h, w, c = t.shape
    es = t.element_size()
    if t.stride(3) != 1 or t.stride(2) != c:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input pixels must be contiguous within a row")
    s.dtype = _DTYPE_CODE[t.dtype]
    s.channels, s.planar, s.numSamples = c, 0, n
    s.base = t.data_ptr()
    s.sampleStride, s.rowStride, s.planeStride = t.stride(0) * es, t.stride(1) * es, 0
    s.width, s.height = w, h
    return s, t


def _dest_of(dst: torch.Tensor, layout: str):
    """layout: 'NHWC', 'HWC', 'NCHW' or 'CHW'. Returns (struct, samples)."""
    if not _device_accessible(dst):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Output must be a cuda-accessible, pitch-linear tensor")
    if layout not in ("NHWC", "HWC", "NCHW", "CHW"):
        raise Error(Status.ERROR_NOT_COMPATIBLE,
                    f"Output tensor must have 'NHWC', 'NCHW', 'HWC', or 'CHW' layout: Layout provided {layout}")
    if dst.dim() != len(layout):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Output tensor rank does not match its layout")
    t = dst if dst.dim() == 4 else dst.unsqueeze(0)
    es = t.element_size()
    d = _Dest()
    d.base, d.dtype = t.data_ptr(), _DTYPE_CODE[t.dtype]
    if layout.endswith("HWC"):
        n, h, w, c = t.shape
        d.sampleStride, d.rowStride, d.pixStride, d.chanStride = (t.stride(i) * es for i in range(4))
    else:
        n, c, h, w = t.shape
        d.sampleStride, d.chanStride, d.rowStride, d.pixStride = (t.stride(i) * es for i in range(4))
    d.channels, d.width, d.height = c, w, h
    return d, n


def _default_layout(t: torch.Tensor, layout: str) -> str:
    if layout:
        return layout
    return "NHWC" if t.dim() == 4 else "HWC"


# ------------------------------------------------------------------------------------------------ operators

def fused_preprocess_into(dst: torch.Tensor, src: Union[torch.Tensor, ImageBatchVarShape], *, resize_dim, interp,
                          crop_pos=(0, 0), layout: str = "", manip=ChannelManip.NO_OP, scale: float = 1.0,
                          offset: float = 0.0, base: Optional[Sequence[float]] = None,
                          mul: Optional[Sequence[float]] = None, gscale: float = 1.0, shift: float = 0.0,
                          srcCast: bool = True, roi: Optional[torch.Tensor] = None,
                          flip_code: Optional[torch.Tensor] = None, dst_pos=(0, 0), region_size=None,
                          pad_value: float = 0.0, stream=None) -> torch.Tensor:
    """The whole fused pass in one call: resize (of the optional per-sample ``roi``) -> crop -> optional flip ->
    affine -> channel map -> cast -> layout, optionally placed inside a padded canvas.

    A superset of :func:`resize_crop_convert_reformat_into`: ``base``/``mul`` select the per-channel form
    ``(v - base[c]) * mul[c] * gscale + shift``; ``roi`` is an int32 CUDA tensor ``[N, 4]`` of ``(x, y, w, h)``;
    ``flip_code`` an int32 CUDA tensor ``[N]``; ``dst_pos``/``region_size``/``pad_value`` describe a letterbox.
    float16 destinations are accepted here.
    """
    layout = _default_layout(dst, layout)
    s, keep_src = _source_of(src)
    d, n_out = _dest_of(dst, layout)
    if n_out != s.numSamples:
        raise Error(Status.ERROR_INVALID_ARGUMENT,
                    "Input and output must have the same batch size (i.e., same number of images): Provided "
                    f"{s.numSamples} input and {n_out} output images / samples")
    op = _ResizeOp()
    op.resizeW, op.resizeH = int(resize_dim[0]), int(resize_dim[1])
    op.cropX, op.cropY = int(crop_pos[0]), int(crop_pos[1])
    op.interp, op.srcCast, op.manip = int(interp), int(bool(srcCast)), int(manip)
    op.perChannel = int(base is not None or mul is not None)
    op.scale, op.offset, op.gscale, op.shift = float(scale), float(offset), float(gscale), float(shift)
    for i in range(4):
        op.base[i] = float(base[i]) if base is not None and i < len(base) else 0.0
        op.mul[i] = float(mul[i]) if mul is not None and i < len(mul) else 1.0
    if region_size is not None:
        op.dstX, op.dstY = int(dst_pos[0]), int(dst_pos[1])
        op.regionW, op.regionH = int(region_size[0]), int(region_size[1])
    op.padValue = float(pad_value)
    if roi is not None:
        if roi.dtype != torch.int32 or not roi.is_cuda or roi.shape[-1] != 4 or roi.stride(-1) != 1:
            raise Error(Status.ERROR_INVALID_ARGUMENT, "roi must be an int32 CUDA tensor [N, 4]")
        op.roi = roi.data_ptr()
        op.roiStride = roi.stride(0) * 4 if roi.dim() > 1 else 16
    if flip_code is not None:
        if flip_code.dtype != torch.int32 or not flip_code.is_cuda or not flip_code.is_contiguous():
            raise Error(Status.ERROR_INVALID_ARGUMENT, "flip_code must be a packed int32 CUDA tensor [N]")
        op.flipCode = flip_code.data_ptr()
    _check(lib().b200ppResizeCropConvertReformat(C.byref(s), C.byref(d), C.byref(op), _stream_handle(stream)))
    return dst


def resize_crop_convert_reformat_into(dst: torch.Tensor, src: Union[torch.Tensor, ImageBatchVarShape],
                                      resize_dim: Tuple[int, int], interp: Interp, cropPos: Tuple[int, int], *,
                                      layout: str = "", manip: ChannelManip = ChannelManip.NO_OP, scale: float = 1.0,
                                      offset: float = 0.0, srcCast: bool = True, stream=None) -> torch.Tensor:
    """cvcuda.resize_crop_convert_reformat_into (python/mod_cvcuda/OpResizeCropConvertReformat.cpp:263-316,374-420).

    ``layout`` names the layout of ``dst`` (a torch tensor carries none); default NHWC / HWC by rank. The crop size
    is the width and height of ``dst``. Like the reference operator, float16 output is refused here
    (src/cvcuda/priv/OpResizeCropConvertReformat.cu:476-479); use :func:`fused_preprocess_into` for it.
    """
    if dst.dtype not in (torch.uint8, torch.float32):
        raise Error(Status.ERROR_NOT_COMPATIBLE, "Output must be of data type uchar or float.")
    return fused_preprocess_into(dst, src, resize_dim=resize_dim, interp=interp, crop_pos=cropPos, layout=layout,
                                 manip=manip, scale=scale, offset=offset, srcCast=srcCast, stream=stream)


def resize_crop_convert_reformat(src: Union[torch.Tensor, ImageBatchVarShape], resize_dim: Tuple[int, int],
                                 interp: Interp, crop_rect: Union[RectI, Tuple[int, int, int, int]], *,
                                 layout: str = "", data_type: Optional[torch.dtype] = None,
                                 manip: ChannelManip = ChannelManip.NO_OP, scale: float = 1.0, offset: float = 0.0,
                                 srcCast: bool = True, stream=None) -> torch.Tensor:
    """cvcuda.resize_crop_convert_reformat (python/mod_cvcuda/OpResizeCropConvertReformat.cpp:58-104,145-196).

    Allocates the output: shape from ``crop_rect`` (x, y, width, height), layout from ``layout`` (default: the
    input's), element type from ``data_type`` (default: the input's).
    """
    rect = RectI(*crop_rect)
    if isinstance(src, ImageBatchVarShape):
        n, c, rank4, dev, in_dtype = len(src), src.channels, True, src.device, src.dtype
        if c != 3:
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Input must have 3 channels.")
        out_layout = layout or "NHWC"
        if out_layout in ("HWC", "NHW", "HW"):
            out_layout = "NHWC"
        elif out_layout == "CHW":
            out_layout = "NCHW"
    else:
        if src.dim() not in (3, 4):
            raise Error(Status.ERROR_INVALID_IMAGE_FORMAT, "Input tensor must have layout 'HWC' or 'NHWC'.")
        rank4 = src.dim() == 4
        n = src.shape[0] if rank4 else 1
        c, in_dtype = src.shape[-1], src.dtype
        dev = src.device if src.is_cuda else torch.device("cuda", torch.cuda.current_device())
        out_layout = layout or ("NHWC" if rank4 else "HWC")
        if len(out_layout) != src.dim():
            raise Error(Status.ERROR_INVALID_IMAGE_FORMAT, "Output tensor rank must match input tensor rank.")
    if out_layout not in ("HWC", "NHWC", "CHW", "NCHW"):
        raise Error(Status.ERROR_INVALID_IMAGE_FORMAT, "Output tensor must have layout 'HWC', 'NHWC', 'CHW', or 'NCHW'.")
    shape = (rect.height, rect.width, c) if out_layout.endswith("HWC") else (c, rect.height, rect.width)
    if rank4:
        shape = (n,) + shape
    dst = torch.empty(shape, dtype=data_type or in_dtype, device=dev)
    return resize_crop_convert_reformat_into(dst, src, resize_dim, interp, (rect.x, rect.y), layout=out_layout,
                                             manip=manip, scale=scale, offset=offset, srcCast=srcCast, stream=stream)


def _param_tensor(t: torch.Tensor, what: str):
    if not t.is_cuda or t.dtype != torch.float32:
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"Input {what} must be cuda-accessible, pitch-linear tensor")
    return t.data_ptr(), t.shape[-1], t.stride(-1) * 4


def crop_flip_normalize_reformat_into(dst: torch.Tensor, src: ImageBatchVarShape, rect: torch.Tensor,
                                      flip_code: torch.Tensor, base: torch.Tensor, scale: torch.Tensor,
                                      globalscale: float = 1.0, globalshift: float = 0.0, epsilon: float = 0.0,
                                      flags: Optional[int] = None, border: Border = Border.CONSTANT,
                                      bvalue: float = 0.0, *, layout: str = "", stream=None) -> torch.Tensor:
    """cvcuda.crop_flip_normalize_reformat_into (python/mod_cvcuda/OpCropFlipNormalizeReformat.cpp:37-63,128-165).

    ``rect``: int32 CUDA tensor ``[N, 1, 1, 4]`` of (x, y, w, h); ``flip_code``: int32 ``[N]``; ``base``/``scale``:
    float32 ``[1, 1, 1, C]`` (or one value). ``layout`` names the layout of ``dst`` ('NHWC' default, or 'NCHW').
    """
    layout = layout or "NHWC"
    if layout not in ("NHWC", "NCHW"):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Invalid tensor layout in output")
    if not isinstance(src, ImageBatchVarShape):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input must be a var-shape image batch")
    s, keep = _source_of(src)
    d, n_out = _dest_of(dst, layout)
    if n_out < s.numSamples:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Output has fewer samples than the input batch")
    if rect.dtype != torch.int32 or not rect.is_cuda or rect.shape[-1] != 4 or rect.stride(-1) != 1:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input cropRect must be cuda-accessible, pitch-linear tensor")
    if flip_code.dtype != torch.int32 or not flip_code.is_cuda or not flip_code.is_contiguous():
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input flipCode must be cuda-accessible, pitch-linear tensor")
    op = _SliceOp()
    op.cropRect, op.cropRectStride = rect.data_ptr(), rect.stride(0) * 4
    op.flipCode = flip_code.data_ptr()
    op.border, op.borderValue = int(border), float(bvalue)
    op.base, op.baseChannels, op.baseChanStride = _param_tensor(base, "base")
    op.scale, op.scaleChannels, op.scaleChanStride = _param_tensor(scale, "scale")
    op.gscale, op.shift, op.epsilon = float(globalscale), float(globalshift), float(epsilon)
    op.flags = int(flags or 0)
    _check(lib().b200ppCropFlipNormalizeReformat(C.byref(s), C.byref(d), C.byref(op), _stream_handle(stream)))
    return dst


def crop_flip_normalize_reformat(src: ImageBatchVarShape, out_shape: Sequence[int], out_dtype: torch.dtype,
                                 out_layout: str, rect: torch.Tensor, flip_code: torch.Tensor, base: torch.Tensor,
                                 scale: torch.Tensor, globalscale: float = 1.0, globalshift: float = 0.0,
                                 epsilon: float = 0.0, flags: Optional[int] = None, border: Border = Border.CONSTANT,
                                 bvalue: float = 0.0, *, stream=None) -> torch.Tensor:
    """cvcuda.crop_flip_normalize_reformat (python/mod_cvcuda/OpCropFlipNormalizeReformat.cpp:65-74,86-126)."""
    dst = torch.empty(tuple(out_shape), dtype=out_dtype, device=src.device)
    return crop_flip_normalize_reformat_into(dst, src, rect, flip_code, base, scale, globalscale, globalshift, epsilon,
                                             flags, border, bvalue, layout=out_layout, stream=stream)


# ------------------------------------------------------------------------------------------------ stand-alone Resize

def _image_set(x: Union[torch.Tensor, ImageBatchVarShape], what: str):
    """_ImageSet of a dense (N)HWC tensor or an image batch, plus the objects that must stay alive."""
    s = _ImageSet()
    if isinstance(x, ImageBatchVarShape):
        if x.planar:
            raise Error(Status.ERROR_INVALID_ARGUMENT, f"{what} images must be interleaved")
        if len(x) == 0:
            s.numSamples = 0
            return s, None
        table = x.descriptor_table()
        s.imageList = table.data_ptr()
        s.dtype, s.channels, s.numSamples = _DTYPE_CODE.get(x.dtype, -1), x.channels, len(x)
        s.maxWidth, s.maxHeight = x.max_size
        return s, table
    if x.dim() not in (3, 4):
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"{what} must have (N)HWC layout")
    if not _device_accessible(x) or x.stride(-1) != 1 or x.stride(-2) != x.shape[-1]:
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"{what} must be a cuda-accessible, pitch-linear tensor")
    es = x.element_size()
    s.base, s.dtype, s.channels = x.data_ptr(), _DTYPE_CODE.get(x.dtype, -1), x.shape[-1]
    s.numSamples = x.shape[0] if x.dim() == 4 else 1
    s.height, s.width = x.shape[-3], x.shape[-2]
    s.rowStride = x.stride(-3) * es
    s.sampleStride = x.stride(0) * es if x.dim() == 4 else 0
    return s, x


def resized_crop_into(dst: Union[torch.Tensor, ImageBatchVarShape], src: Union[torch.Tensor, ImageBatchVarShape],
                      rects: torch.Tensor, interp: Interp = Interp.LINEAR, *, stream=None):
    """Every image of ``src`` cropped to its rectangle and resized to the size of the corresponding image of ``dst``:
    ``rects`` is an int32 CUDA tensor [N, 4] of (left, top, width, height). The resampling step of
    cvcuda.random_resized_crop with caller-chosen rectangles (the reference draws them inside the operator,
    src/cvcuda/priv/legacy/random_resized_crop.cu:459-467)."""
    if isinstance(src, ImageBatchVarShape) != isinstance(dst, ImageBatchVarShape):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input and output must both be tensors or both be image batches")
    if not isinstance(src, ImageBatchVarShape) and src.dim() != dst.dim():
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input and output data layout are different")
    s, keep_s = _image_set(src, "Input")
    d, keep_d = _image_set(dst, "Output")
    if not isinstance(rects, torch.Tensor) or not rects.is_cuda or rects.dtype != torch.int32 or not rects.is_contiguous() \
            or rects.numel() != 4 * s.numSamples:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "rects must be a contiguous int32 CUDA tensor [N, 4]")
    if s.numSamples == 0:
        return dst
    _check(lib().b200ppResizedCrop(C.byref(s), C.byref(d), rects.data_ptr(), int(interp), _stream_handle(stream)))
    return dst


def random_crop_rects(sizes: Sequence[Tuple[int, int]], min_scale: float = 0.08, max_scale: float = 1.0,
                      min_ratio: float = 0.75, max_ratio: float = 1.3333333333333333, seed: int = 0) -> List[Tuple[int, int, int, int]]:
    """The crop rectangles (left, top, width, height) the reference's RandomResizedCrop operator draws for images of the
    given (width, height) sizes, in order, from a fresh generator (src/cvcuda/priv/legacy/random_resized_crop.cu:336-390;
    seed 0 = a random seed, as there)."""
    gen = C.c_void_p()
    status = lib().b200ppRandomCropCreate(C.byref(gen), float(min_scale), float(max_scale), float(min_ratio),
                                          float(max_ratio), int(seed) & 0xFFFFFFFF)
    if status != 0:
        raise Error(Status(status), "Invalid Parameter: scale and ratio should be of kind (min, max)")
    try:
        out, rect = [], (C.c_int32 * 4)()
        for (w, h) in sizes:
            if lib().b200ppRandomCropNext(gen, int(h), int(w), rect) != 0:
                raise Error(Status.ERROR_INVALID_ARGUMENT, f"Invalid image size {w}x{h}")
            out.append(tuple(rect))
        return out
    finally:
        lib().b200ppRandomCropDestroy(gen)


def random_resized_crop_into(dst, src, min_scale: float = 0.08, max_scale: float = 1.0, min_ratio: float = 0.75,
                             max_ratio: float = 1.3333333333333333, interp: Interp = Interp.LINEAR, seed: int = 0, *,
                             stream=None):
    """cvcuda.random_resized_crop_into for tensors and image batches (python/mod_cvcuda/OpRandomResizedCrop.cpp:29-52,
    :65-88): like the reference, every call builds a fresh generator from ``seed`` and draws one rectangle per image."""
    if int(interp) == 2:
        raise Error(Status.ERROR_NOT_IMPLEMENTED, "Interpolation not implemented: NVCV_INTERP_CUBIC")
    if int(interp) not in (0, 1):
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"Invalid interpolation {int(interp)}")
    if isinstance(src, ImageBatchVarShape):
        sizes = [(im.shape[1], im.shape[0]) for im in src._images]
    else:
        if src.dim() not in (3, 4):
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Input must have (N)HWC layout")
        sizes = [(src.shape[-2], src.shape[-3])] * (src.shape[0] if src.dim() == 4 else 1)
    rects = random_crop_rects(sizes, min_scale, max_scale, min_ratio, max_ratio, seed)
    dev = src.device if isinstance(src, ImageBatchVarShape) or src.is_cuda else torch.device("cuda", torch.cuda.current_device())
    # a blocking upload from pageable memory: complete before the launch, whatever stream that is on
    table = torch.tensor(rects, dtype=torch.int32).reshape(-1, 4).to(dev)
    if stream is not None:
        # the table goes back to torch's caching allocator when this function returns; tell it which stream still reads it
        table.record_stream(stream if isinstance(stream, torch.cuda.Stream) else torch.cuda.ExternalStream(int(stream)))
    return resized_crop_into(dst, src, table, interp, stream=stream)


def random_resized_crop(src, shape_or_sizes, min_scale: float = 0.08, max_scale: float = 1.0, min_ratio: float = 0.75,
                        max_ratio: float = 1.3333333333333333, interp: Interp = Interp.LINEAR, seed: int = 0, *, stream=None):
    """cvcuda.random_resized_crop: allocates the output ((N)HWC shape for a tensor, (width, height) per image for a batch)."""
    if isinstance(src, ImageBatchVarShape):
        sizes = list(shape_or_sizes)
        if len(sizes) != len(src):
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Invalid outputs sizes, must be equal to input batch size")
        out = ImageBatchVarShape([torch.empty((int(h), int(w), src.channels), dtype=src.dtype, device=src.device)
                                  for (w, h) in sizes])
    else:
        dev = src.device if src.is_cuda else torch.device("cuda", torch.cuda.current_device())
        out = torch.empty(tuple(int(v) for v in shape_or_sizes), dtype=src.dtype, device=dev)
    return random_resized_crop_into(out, src, min_scale, max_scale, min_ratio, max_ratio, interp, seed, stream=stream)


def resize_into(dst: Union[torch.Tensor, ImageBatchVarShape], src: Union[torch.Tensor, ImageBatchVarShape],
                interp: Interp = Interp.LINEAR, *, stream=None):
    """cvcuda.resize_into for tensors and image batches (python/mod_cvcuda/OpResize.cpp:32-49,58-76): every image of
    ``src`` is resized to the size of the corresponding image of ``dst``. Nearest and linear interpolation."""
    if isinstance(src, ImageBatchVarShape) != isinstance(dst, ImageBatchVarShape):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input and output must both be tensors or both be image batches")
    if not isinstance(src, ImageBatchVarShape) and src.dim() != dst.dim():
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input and output data layout are different")
    s, keep_s = _image_set(src, "Input")
    d, keep_d = _image_set(dst, "Output")
    _check(lib().b200ppResize(C.byref(s), C.byref(d), int(interp), _stream_handle(stream)))
    return dst


def resize(src: Union[torch.Tensor, ImageBatchVarShape], shape_or_sizes, interp: Interp = Interp.LINEAR, *, stream=None):
    """cvcuda.resize (python/mod_cvcuda/OpResize.cpp:51-56,78-97). For a tensor, ``shape_or_sizes`` is the output shape
    ((N)HWC); for an image batch, a list of (width, height) per image. Allocates the output."""
    if isinstance(src, ImageBatchVarShape):
        sizes = list(shape_or_sizes)
        if len(sizes) != len(src):
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Invalid outputs sizes, must be equal to input batch size")
        out = ImageBatchVarShape([torch.empty((int(h), int(w), src.channels), dtype=src.dtype, device=src.device)
                                  for (w, h) in sizes])
        return resize_into(out, src, interp, stream=stream)
    dev = src.device if src.is_cuda else torch.device("cuda", torch.cuda.current_device())
    out = torch.empty(tuple(int(v) for v in shape_or_sizes), dtype=src.dtype, device=dev)
    return resize_into(out, src, interp, stream=stream)


# ------------------------------------------------------------------------------------------------ stand-alone Normalize

def _broadcast_param(t: torch.Tensor, what: str, extents):
    """Pointer and the four byte strides (sample, row, column, channel; 0 where the extent is 1) of a float32 CUDA
    parameter tensor of rank 1 to 4, aligned to the right ((N)HWC). ``extents`` = the input's (N, H, W, C), H and W being
    None for an image batch: every extent of the parameter must be 1 or the input's
    (src/cvcuda/priv/legacy/normalize.cu:300-306)."""
    if not t.is_cuda or t.dtype != torch.float32 or t.dim() < 1 or t.dim() > 4:
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"Input {what} must be cuda-accessible, pitch-linear tensor")
    shape = (1,) * (4 - t.dim()) + tuple(t.shape)
    stride = (0,) * (4 - t.dim()) + tuple(t.stride())
    if any(shape[k] != 1 and shape[k] != extents[k] for k in range(4)):
        raise Error(Status.ERROR_INVALID_ARGUMENT,
                    f"Input {what} has shape {shape}: every extent must be 1 or equal to the input's")
    return t.data_ptr(), (C.c_int64 * 4)(*[0 if shape[k] == 1 else stride[k] * 4 for k in range(4)])


def normalize_into(dst, src, base: torch.Tensor, scale: torch.Tensor, flags: Optional[int] = None,
                   globalscale: float = 1.0, globalshift: float = 0.0, epsilon: float = 0.0, *, stream=None):
    """cvcuda.normalize_into for tensors and image batches (python/mod_cvcuda/OpNormalize.cpp): dst = (src - base) * mul *
    globalscale + globalshift, mul = scale, or 1 / sqrt(scale^2 + epsilon) with NORMALIZE_SCALE_IS_STDDEV."""
    if isinstance(src, ImageBatchVarShape) != isinstance(dst, ImageBatchVarShape):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input and output must both be tensors or both be image batches")
    if not isinstance(src, ImageBatchVarShape) and src.dim() != dst.dim():
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Invalid DataFormat between input and output")
    s, keep_s = _image_set(src, "Input")
    d, keep_d = _image_set(dst, "Output")
    op = _NormalizeOp()
    extents = (s.numSamples, None, None, s.channels) if isinstance(src, ImageBatchVarShape) \
        else (s.numSamples, s.height, s.width, s.channels)
    op.base, op.baseStride = _broadcast_param(base, "base", extents)
    op.scale, op.scaleStride = _broadcast_param(scale, "scale", extents)
    op.gscale, op.shift, op.epsilon, op.flags = float(globalscale), float(globalshift), float(epsilon), int(flags or 0)
    _check(lib().b200ppNormalize(C.byref(s), C.byref(d), C.byref(op), _stream_handle(stream)))
    return dst


def normalize(src, base: torch.Tensor, scale: torch.Tensor, flags: Optional[int] = None, globalscale: float = 1.0,
              globalshift: float = 0.0, epsilon: float = 0.0, *, stream=None):
    """cvcuda.normalize: allocates an output like the input (same sizes, element type and layout)."""
    if isinstance(src, ImageBatchVarShape):
        out = ImageBatchVarShape([torch.empty(tuple(im.shape), dtype=im.dtype, device=src.device) for im in src._images])
    else:
        dev = src.device if src.is_cuda else torch.device("cuda", torch.cuda.current_device())
        out = torch.empty(tuple(src.shape), dtype=src.dtype, device=dev)
    return normalize_into(out, src, base, scale, flags, globalscale, globalshift, epsilon, stream=stream)


# ------------------------------------------------------------------------------------------------ stand-alone Reformat

def reformat_into(dst: torch.Tensor, src: torch.Tensor, *, src_layout: str = "", dst_layout: str = "", stream=None):
    """cvcuda.reformat_into (python/mod_cvcuda/OpReformat.cpp): copies ``src`` into ``dst`` changing between the NHWC / HWC
    and NCHW / CHW layouts (a torch tensor carries no layout, so both are named; default (N)HWC by rank)."""
    src_layout, dst_layout = _default_layout(src, src_layout), _default_layout(dst, dst_layout)
    if len(src_layout) != len(dst_layout) or src_layout not in ("NHWC", "HWC", "NCHW", "CHW") \
            or dst_layout not in ("NHWC", "HWC", "NCHW", "CHW"):
        raise Error(Status.ERROR_INVALID_ARGUMENT,
                    f"Invalid combination of input format {src_layout} and output format {dst_layout}")
    if not _device_accessible(src):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input must be cuda-accessible, pitch-linear tensor")
    s, n_in = _dest_of(src, src_layout)
    d, n_out = _dest_of(dst, dst_layout)
    if n_in != n_out:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input and output samples are different")
    _check(lib().b200ppReformat(C.byref(s), C.byref(d), n_in, _stream_handle(stream)))
    return dst


def reformat(src: torch.Tensor, dst_layout: str, *, src_layout: str = "", stream=None) -> torch.Tensor:
    """cvcuda.reformat: allocates the output in ``dst_layout``."""
    src_layout = _default_layout(src, src_layout)
    if len(src_layout) != len(dst_layout):
        raise Error(Status.ERROR_INVALID_ARGUMENT,
                    f"Invalid combination of input format {src_layout} and output format {dst_layout}")
    dims = dict(zip(src_layout, src.shape))
    dev = src.device if src.is_cuda else torch.device("cuda", torch.cuda.current_device())
    out = torch.empty(tuple(dims[k] for k in dst_layout), dtype=src.dtype, device=dev)
    return reformat_into(out, src, src_layout=src_layout, dst_layout=dst_layout, stream=stream)


# ------------------------------------------------------------------------------------------------ stand-alone ConvertTo

def convertto_into(dst: torch.Tensor, src: torch.Tensor, scale: float = 1.0, offset: float = 0.0, *, stream=None):
    """cvcuda.convertto_into (python/mod_cvcuda/OpConvertTo.cpp): dst = SaturateCast(scale * src + offset), (N)HWC tensors of
    equal shape, the element type of ``dst`` decides the conversion."""
    if isinstance(src, ImageBatchVarShape) or isinstance(dst, ImageBatchVarShape):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "ConvertTo works on tensors")
    if src.dim() != dst.dim():
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Invalid DataFormat between input and output")
    s, keep_s = _image_set(src, "Input")
    d, keep_d = _image_set(dst, "Output")
    _check(lib().b200ppConvertTo(C.byref(s), C.byref(d), float(scale), float(offset), _stream_handle(stream)))
    return dst


def convertto(src: torch.Tensor, dtype: torch.dtype, scale: float = 1.0, offset: float = 0.0, *, stream=None):
    """cvcuda.convertto: allocates an output of the input's shape with element type ``dtype``."""
    dev = src.device if src.is_cuda else torch.device("cuda", torch.cuda.current_device())
    out = torch.empty(tuple(src.shape), dtype=dtype, device=dev)
    return convertto_into(out, src, scale, offset, stream=stream)


# ------------------------------------------------------------------------------------------------ stand-alone CopyMakeBorder

def _border_value(border_value) -> "C.Array":
    vals = [float(v) for v in (border_value or [])]
    if len(vals) > 4:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Channels of borderValue should <= 4.")
    return (C.c_float * 4)(*(vals + [0.0] * (4 - len(vals))))


def _offset_list(t: torch.Tensor, what: str, count: int):
    """top / left of the variable-shape forms: an int32 CUDA tensor with one packed value per image."""
    if not isinstance(t, torch.Tensor) or not t.is_cuda or t.dtype != torch.int32:
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"Invalid {what} DataType")
    if t.numel() < count or not t.is_contiguous():
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"{what} must hold one packed int32 per image")
    return t


def copymakeborder_into(dst, src, border_mode: Border = Border.CONSTANT, border_value: Sequence[float] = (), *, top, left,
                        stream=None):
    """cvcuda.copymakeborder_into (python/mod_cvcuda/OpCopyMakeBorder.cpp:234-262 for tensors, :358-386 for image
    batches) and cvcuda.copymakeborderstack_into (:295-325: image batch -> tensor). ``top`` / ``left`` are ints for
    tensors, int32 CUDA tensors with one value per image for image batches."""
    value = _border_value(border_value)
    s, keep_s = _image_set(src, "Input")
    d, keep_d = _image_set(dst, "Output")
    if isinstance(src, ImageBatchVarShape):
        tl, ll = _offset_list(top, "Top", len(src)), _offset_list(left, "Left", len(src))
        _check(lib().b200ppCopyMakeBorder(C.byref(s), C.byref(d), 0, 0, tl.data_ptr(), ll.data_ptr(), int(border_mode), value,
                                          _stream_handle(stream)))
        return dst
    if isinstance(dst, ImageBatchVarShape):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input must be varshape image batch")
    if src.dim() != dst.dim():
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Invalid DataFormat between input and output")
    _check(lib().b200ppCopyMakeBorder(C.byref(s), C.byref(d), int(top), int(left), None, None, int(border_mode), value,
                                      _stream_handle(stream)))
    return dst


def copymakeborder(src, border_mode: Border = Border.CONSTANT, border_value: Sequence[float] = (), *, top, left, bottom=None,
                   right=None, out_heights=None, out_widths=None, stream=None):
    """cvcuda.copymakeborder: allocates the output. Tensors take top / bottom / left / right
    (python/mod_cvcuda/OpCopyMakeBorder.cpp:81-99); image batches take top / left tensors and out_heights / out_widths
    lists (:161-192)."""
    if isinstance(src, ImageBatchVarShape):
        if out_heights is None or out_widths is None or len(out_heights) != len(src) or len(out_widths) != len(src):
            raise Error(Status.ERROR_INVALID_ARGUMENT, "out_heights / out_widths must have one entry per input image")
        out = ImageBatchVarShape([torch.empty((int(h), int(w), src.channels), dtype=src.dtype, device=src.device)
                                  for h, w in zip(out_heights, out_widths)])
        return copymakeborder_into(out, src, border_mode, border_value, top=top, left=left, stream=stream)
    if bottom is None or right is None:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Tensor inputs need top, bottom, left and right")
    shape = list(src.shape)
    shape[-3] += int(top) + int(bottom)
    shape[-2] += int(left) + int(right)
    dev = src.device if src.is_cuda else torch.device("cuda", torch.cuda.current_device())
    out = torch.empty(tuple(shape), dtype=src.dtype, device=dev)
    return copymakeborder_into(out, src, border_mode, border_value, top=top, left=left, stream=stream)


def copymakeborderstack_into(dst: torch.Tensor, src: ImageBatchVarShape, border_mode: Border = Border.CONSTANT,
                             border_value: Sequence[float] = (), *, top, left, stream=None):
    """cvcuda.copymakeborderstack_into (python/mod_cvcuda/OpCopyMakeBorder.cpp:101-127): every image of the batch lands in
    one sample of the (N)HWC tensor ``dst``."""
    if not isinstance(src, ImageBatchVarShape) or isinstance(dst, ImageBatchVarShape):
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Input must be varshape image batch, output a tensor")
    return copymakeborder_into(dst, src, border_mode, border_value, top=top, left=left, stream=stream)


def copymakeborderstack(src: ImageBatchVarShape, border_mode: Border = Border.CONSTANT, border_value: Sequence[float] = (), *,
                        top, left, out_height: int, out_width: int, stream=None):
    """cvcuda.copymakeborderstack (python/mod_cvcuda/OpCopyMakeBorder.cpp:129-141): allocates the NHWC output."""
    out = torch.empty((len(src), int(out_height), int(out_width), src.channels), dtype=src.dtype, device=src.device)
    return copymakeborderstack_into(out, src, border_mode, border_value, top=top, left=left, stream=stream)
