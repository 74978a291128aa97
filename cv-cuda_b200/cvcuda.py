"""The reference's Python surface for the operators of this library: code written for ``import cvcuda, nvcv`` runs with

    cvcuda = nvcv = cvcuda_b200.cvcuda

Objects carry their layout, as the reference's do: :class:`Tensor` (``cvcuda.Tensor(shape, dtype, layout)``,
``.shape / .dtype / .layout / .cuda()``), :class:`Image`, :class:`ImageBatchVarShape` (``pushback`` / ``popback``),
:class:`Stream`, ``as_tensor`` / ``as_image`` for anything that exports ``__cuda_array_interface__`` or DLPack (torch, cupy,
numba, ... -- no copy), and the enums ``Interp``, ``ChannelManip``, ``Border``, ``NormalizeFlags``, ``Type``, ``Format``,
``RectI``. The operator functions have the reference's names, argument names, order and defaults
(python/mod_cvcuda/Op*.cpp); they unwrap the objects and call :mod:`cvcuda_b200.ops`, which works on torch tensors.
Memory comes from torch's CUDA allocator; every value is computed by ``libcvcuda_b200.so``.
"""
from __future__ import annotations

import enum
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch

from . import ops
from .ops import Border, ChannelManip, Error, Interp, RectI, Status  # noqa: F401  (re-exported)


class NormalizeFlags(enum.IntEnum):
    """cvcuda.NormalizeFlags (python/mod_cvcuda/OpNormalize.cpp)."""
    SCALE_IS_STDDEV = 1


class Type:
    """nvcv.Type: element types. The members are numpy dtypes, so ``tensor.dtype == nvcv.Type.F32`` and
    ``tensor.dtype == np.float32`` both hold, as with the reference's objects."""
    U8 = np.dtype(np.uint8)
    S8 = np.dtype(np.int8)
    U16 = np.dtype(np.uint16)
    S16 = np.dtype(np.int16)
    S32 = np.dtype(np.int32)
    F32 = np.dtype(np.float32)
    F16 = np.dtype(np.float16)


class Format(enum.Enum):
    """nvcv.Format, the members the operators of this library can take: (element type, channels, planar)."""
    U8 = (np.uint8, 1, False)
    S16 = (np.int16, 1, False)
    S32 = (np.int32, 1, False)
    F32 = (np.float32, 1, False)
    RGB8 = (np.uint8, 3, False)
    BGR8 = (np.uint8, 3, False, "bgr")
    RGBA8 = (np.uint8, 4, False)
    BGRA8 = (np.uint8, 4, False, "bgra")
    RGB8p = (np.uint8, 3, True)
    RGBA8p = (np.uint8, 4, True)
    RGBf32 = (np.float32, 3, False)
    RGBAf32 = (np.float32, 4, False)
    RGBf32p = (np.float32, 3, True)
    RGBAf32p = (np.float32, 4, True)

    @property
    def dtype(self):
        return np.dtype(self.value[0])

    @property
    def channels(self) -> int:
        return self.value[1]

    @property
    def planar(self) -> bool:
        return self.value[2]


_TORCH = {np.dtype(np.uint8): torch.uint8, np.dtype(np.int8): torch.int8, np.dtype(np.int16): torch.int16,
          np.dtype(np.int32): torch.int32, np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16}
if hasattr(torch, "uint16"):
    _TORCH[np.dtype(np.uint16)] = torch.uint16
_NUMPY = {v: k for k, v in _TORCH.items()}


def _torch_dtype(dt) -> torch.dtype:
    if isinstance(dt, torch.dtype):
        return dt
    try:
        return _TORCH[np.dtype(dt)]
    except (KeyError, TypeError):
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"Unsupported element type {dt!r}") from None


def _device() -> torch.device:
    return torch.device("cuda", torch.cuda.current_device())


class Stream:
    """cvcuda.Stream: a CUDA stream (``Stream.current`` is torch's current stream)."""

    def __init__(self, stream: Optional[torch.cuda.Stream] = None):
        self._stream = stream if stream is not None else torch.cuda.Stream()

    @property
    def handle(self) -> int:
        return self._stream.cuda_stream

    cuda_stream = handle

    def sync(self) -> None:
        self._stream.synchronize()

    @classmethod
    def current(cls) -> "Stream":
        return cls(torch.cuda.current_stream())


def _stream_of(stream):
    if stream is None or isinstance(stream, (int, torch.cuda.Stream)):
        return stream
    if isinstance(stream, Stream):
        return stream._stream
    raise Error(Status.ERROR_INVALID_ARGUMENT, "stream must be a cvcuda.Stream, a torch.cuda.Stream or a raw handle")


class Tensor:
    """cvcuda.Tensor / nvcv.Tensor: a CUDA tensor that knows its layout.

    ``Tensor(shape, dtype, layout)`` allocates (zero-filled); ``Tensor(nimages, (width, height), format)`` allocates an
    image batch tensor (NHWC, or NCHW for planar formats), as nvcv.Tensor does."""

    def __init__(self, *args, layout: Optional[str] = None, _data: Optional[torch.Tensor] = None):
        if _data is not None:
            self._t, self._layout = _data, layout or ""
            return
        if len(args) == 3 and isinstance(args[0], int) and isinstance(args[2], Format):
            n, (w, h), fmt = args
            shape = (n, fmt.channels, h, w) if fmt.planar else (n, h, w, fmt.channels)
            self._t = torch.zeros(shape, dtype=_torch_dtype(fmt.dtype), device=_device())
            self._layout = "NCHW" if fmt.planar else "NHWC"
            return
        if len(args) == 2 and layout is not None:
            args = (*args, layout)
        if len(args) != 3:
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Tensor(shape, dtype, layout) or Tensor(nimages, (w, h), format)")
        shape, dtype, lay = args
        lay = str(lay or "")
        if lay and len(lay) != len(tuple(shape)):
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Layout rank must match the shape's")
        self._t = torch.zeros(tuple(int(v) for v in shape), dtype=_torch_dtype(dtype), device=_device())
        self._layout = lay

    @property
    def shape(self) -> Tuple[int, ...]:
        return tuple(self._t.shape)

    @property
    def dtype(self):
        return _NUMPY[self._t.dtype]

    @property
    def layout(self) -> str:
        return self._layout

    @property
    def ndim(self) -> int:
        return self._t.dim()

    def cuda(self) -> torch.Tensor:
        """The device buffer as an object that exports ``__cuda_array_interface__`` (a torch tensor: no copy)."""
        return self._t

    @property
    def __cuda_array_interface__(self):
        return self._t.__cuda_array_interface__

    def __dlpack__(self, stream=None):
        return self._t.__dlpack__(stream=stream) if stream is not None else self._t.__dlpack__()

    def __dlpack_device__(self):
        return self._t.__dlpack_device__()

    def reshape(self, shape, layout: str) -> "Tensor":
        return Tensor(_data=self._t.reshape(tuple(shape)), layout=layout)

    def __repr__(self) -> str:
        return f"<cvcuda_b200 Tensor layout={self._layout} shape={self.shape} dtype={self.dtype}>"


def _ingest(obj) -> torch.Tensor:
    """A torch CUDA tensor sharing memory with `obj`: torch tensors as they are, ``__cuda_array_interface__`` exporters
    (cupy, numba, the objects of this module) and DLPack exporters without a copy."""
    if isinstance(obj, Tensor):
        return obj._t
    if isinstance(obj, torch.Tensor):
        if not (obj.is_cuda or obj.is_pinned()):
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Buffer must be CUDA (or page-locked host) memory")
        return obj
    if hasattr(obj, "__cuda_array_interface__"):
        return torch.as_tensor(obj, device=_device())
    if hasattr(obj, "__dlpack__"):
        return torch.from_dlpack(obj)
    raise Error(Status.ERROR_INVALID_ARGUMENT, "Object exports neither __cuda_array_interface__ nor DLPack")


def as_tensor(obj, layout: Optional[str] = None) -> Tensor:
    """cvcuda.as_tensor(buffer, layout): wraps existing device memory (no copy). Without a layout, rank 3 is taken as HWC
    and rank 4 as NHWC, as the reference does for image-like buffers."""
    if isinstance(obj, Tensor) and layout is None:
        return obj
    if isinstance(obj, Image):
        t = obj._t
        return Tensor(_data=t, layout=layout or ("CHW" if obj.format.planar else "HWC"))
    t = _ingest(obj)
    lay = layout if layout is not None else {3: "HWC", 4: "NHWC"}.get(t.dim(), "")
    if lay and len(lay) != t.dim():
        raise Error(Status.ERROR_INVALID_ARGUMENT, "Layout rank must match the buffer's")
    return Tensor(_data=t, layout=str(lay))


class Image:
    """cvcuda.Image / nvcv.Image: one image, ``Image((width, height), format)``; rows are padded to a multiple of 32 bytes
    like the reference's allocator does (src/nvcv/src/priv/Image.cpp:47-116)."""

    def __init__(self, size: Tuple[int, int], format: Format, *, _data: Optional[torch.Tensor] = None):
        self.format = format
        if _data is not None:
            self._t = _data
            return
        w, h = int(size[0]), int(size[1])
        es = format.dtype.itemsize
        row_elems = w if format.planar else w * format.channels
        pitch = (row_elems * es + 31) // 32 * 32 // es
        rows = h * format.channels if format.planar else h
        store = torch.zeros((rows, pitch), dtype=_torch_dtype(format.dtype), device=_device())
        if format.planar:
            self._t = torch.as_strided(store, (format.channels, h, w), (h * pitch, pitch, 1))
        else:
            self._t = torch.as_strided(store, (h, w, format.channels), (pitch, format.channels, 1))

    @property
    def size(self) -> Tuple[int, int]:
        return (self._t.shape[2], self._t.shape[1]) if self.format.planar else (self._t.shape[1], self._t.shape[0])

    @property
    def width(self) -> int:
        return self.size[0]

    @property
    def height(self) -> int:
        return self.size[1]

    def cuda(self) -> torch.Tensor:
        return self._t


def as_image(obj, format: Optional[Format] = None) -> Image:
    """cvcuda.as_image(buffer, format): wraps an HWC (or CHW, for a planar format) device buffer as an image, no copy."""
    t = _ingest(obj)
    if t.dim() != 3:
        raise Error(Status.ERROR_INVALID_ARGUMENT, "An image buffer has three dimensions")
    if format is None:
        c = t.shape[2]
        by = {(np.dtype(np.uint8), 1): Format.U8, (np.dtype(np.uint8), 3): Format.RGB8, (np.dtype(np.uint8), 4): Format.RGBA8,
              (np.dtype(np.float32), 1): Format.F32, (np.dtype(np.float32), 3): Format.RGBf32,
              (np.dtype(np.float32), 4): Format.RGBAf32}
        format = by.get((_NUMPY[t.dtype], c))
        if format is None:
            raise Error(Status.ERROR_INVALID_ARGUMENT, "Cannot infer an image format; pass one")
    return Image((0, 0), format, _data=t)


class ImageBatchVarShape(ops.ImageBatchVarShape):
    """cvcuda.ImageBatchVarShape(capacity): images of one format and any sizes. ``pushback`` takes :class:`Image` objects
    (or device buffers); the device-side descriptor table is uploaded again after every change, when next needed."""

    def __init__(self, capacity: int = 0):
        super().__init__((), planar=False)
        self.capacity = int(capacity)
        self.uniqueformat: Optional[Format] = None

    def pushback(self, images) -> None:
        if isinstance(images, (Image, torch.Tensor)) or not isinstance(images, (list, tuple)):
            images = [images]
        for im in images:
            img = im if isinstance(im, Image) else as_image(im)
            if self.capacity and len(self) >= self.capacity:
                raise Error(Status.ERROR_OVERFLOW, "Image batch capacity exceeded")
            if len(self) == 0:
                self.planar, self.uniqueformat = img.format.planar, img.format
            elif img.format.planar != self.planar:
                raise Error(Status.ERROR_INVALID_ARGUMENT,
                            "All input images in a batch must have the same format (including number of channels)")
            super().pushback(img._t)

    def popback(self, count: int = 1) -> None:
        super().popback(count)
        if len(self) == 0:
            self.uniqueformat = None


# ------------------------------------------------------------------------------------------------ operators

def _wrap(t: torch.Tensor, layout: str) -> Tensor:
    return Tensor(_data=t, layout=layout)


def _src_of(src, what="Input"):
    """(torch tensor or batch, layout or None)."""
    if isinstance(src, ops.ImageBatchVarShape):
        return src, None
    t = as_tensor(src)
    return t._t, t.layout


def resize_crop_convert_reformat(src, resize_dim: Tuple[int, int], interp: Interp, crop_rect, *, layout: str = "",
                                 data_type=0, manip: ChannelManip = ChannelManip.NO_OP, scale: float = 1.0, offset: float = 0.0,
                                 srcCast: bool = True, stream=None) -> Tensor:
    """cvcuda.resize_crop_convert_reformat (python/mod_cvcuda/OpResizeCropConvertReformat.cpp:58-104,145-196,207-262)."""
    s, lay = _src_of(src)
    if lay is not None and lay not in ("HWC", "NHWC"):
        raise Error(Status.ERROR_INVALID_IMAGE_FORMAT, "Input tensor must have layout 'HWC' or 'NHWC'.")
    out_layout = str(layout) if layout else (lay or "NHWC")
    dt = _torch_dtype(data_type) if data_type not in (0, None) else None
    out = ops.resize_crop_convert_reformat(s, tuple(resize_dim), interp, RectI(*crop_rect), layout=out_layout, data_type=dt,
                                           manip=manip, scale=scale, offset=offset, srcCast=srcCast, stream=_stream_of(stream))
    if isinstance(s, ops.ImageBatchVarShape) and out_layout in ("HWC", "CHW"):
        out_layout = "N" + out_layout
    return _wrap(out, out_layout)


def resize_crop_convert_reformat_into(dst: Tensor, src, resize_dim: Tuple[int, int], interp: Interp, cropPos, *,
                                      manip: ChannelManip = ChannelManip.NO_OP, scale: float = 1.0, offset: float = 0.0,
                                      srcCast: bool = True, stream=None) -> Tensor:
    """cvcuda.resize_crop_convert_reformat_into (python/mod_cvcuda/OpResizeCropConvertReformat.cpp:33-56,106-130,263-316):
    ``cropPos`` = (x, y) of the crop window's top-left corner in the resized image; the window's size is ``dst``'s."""
    s, lay = _src_of(src)
    if lay is not None and lay not in ("HWC", "NHWC"):
        raise Error(Status.ERROR_NOT_COMPATIBLE, f"Input tensor must have 'NHWC' or 'HWC' layout: Layout provided {lay}")
    d = as_tensor(dst)
    ops.resize_crop_convert_reformat_into(d._t, s, tuple(resize_dim), interp, (int(cropPos[0]), int(cropPos[1])), layout=d.layout,
                                          manip=manip, scale=scale, offset=offset, srcCast=srcCast, stream=_stream_of(stream))
    return dst


def _flat_int32(t, what):
    x = as_tensor(t)._t
    if x.dtype != torch.int32 or not x.is_contiguous():
        raise Error(Status.ERROR_INVALID_ARGUMENT, f"Input {what} must be cuda-accessible, pitch-linear tensor")
    return x.reshape(-1)


def crop_flip_normalize_reformat_into(dst: Tensor, src: ImageBatchVarShape, rect, flip_code, base, scale, globalscale: float = 1.0,
                                      globalshift: float = 0.0, epsilon: float = 0.0, flags: Optional[int] = None,
                                      border: Border = Border.CONSTANT, bvalue: float = 0.0, *, stream=None) -> Tensor:
    """cvcuda.crop_flip_normalize_reformat_into (python/mod_cvcuda/OpCropFlipNormalizeReformat.cpp:37-63,128-165)."""
    d = as_tensor(dst)
    ops.crop_flip_normalize_reformat_into(d._t, src, as_tensor(rect)._t, _flat_int32(flip_code, "flipCode"), as_tensor(base)._t,
                                          as_tensor(scale)._t, globalscale, globalshift, epsilon, int(flags or 0), border, bvalue,
                                          layout=d.layout or "NHWC", stream=_stream_of(stream))
    return dst


def crop_flip_normalize_reformat(src: ImageBatchVarShape, out_shape: Sequence[int], out_dtype, out_layout: str, rect, flip_code,
                                 base, scale, globalscale: float = 1.0, globalshift: float = 0.0, epsilon: float = 0.0,
                                 flags: Optional[int] = None, border: Border = Border.CONSTANT, bvalue: float = 0.0, *,
                                 stream=None) -> Tensor:
    """cvcuda.crop_flip_normalize_reformat (python/mod_cvcuda/OpCropFlipNormalizeReformat.cpp:65-74,86-126)."""
    out = Tensor(tuple(out_shape), out_dtype, str(out_layout))
    return crop_flip_normalize_reformat_into(out, src, rect, flip_code, base, scale, globalscale, globalshift, epsilon, flags,
                                             border, bvalue, stream=stream)


def _like(src):
    if isinstance(src, ops.ImageBatchVarShape):
        return None
    return as_tensor(src).layout


def resize(src, shape_or_sizes, interp: Interp = Interp.LINEAR, *, stream=None):
    """cvcuda.resize (python/mod_cvcuda/OpResize.cpp): tensors keep their layout; image batches come back as batches."""
    s, lay = _src_of(src)
    out = ops.resize(s, shape_or_sizes, interp, stream=_stream_of(stream))
    return out if lay is None else _wrap(out, lay)


def resize_into(dst, src, interp: Interp = Interp.LINEAR, *, stream=None):
    s, _ = _src_of(src)
    d, _ = _src_of(dst)
    ops.resize_into(d, s, interp, stream=_stream_of(stream))
    return dst


def normalize(src, base, scale, flags: Optional[int] = None, globalscale: float = 1.0, globalshift: float = 0.0,
              epsilon: float = 0.0, *, stream=None):
    """cvcuda.normalize (python/mod_cvcuda/OpNormalize.cpp)."""
    s, lay = _src_of(src)
    out = ops.normalize(s, as_tensor(base)._t, as_tensor(scale)._t, flags, globalscale, globalshift, epsilon,
                        stream=_stream_of(stream))
    return out if lay is None else _wrap(out, lay)


def normalize_into(dst, src, base, scale, flags: Optional[int] = None, globalscale: float = 1.0, globalshift: float = 0.0,
                   epsilon: float = 0.0, *, stream=None):
    s, _ = _src_of(src)
    d, _ = _src_of(dst)
    ops.normalize_into(d, s, as_tensor(base)._t, as_tensor(scale)._t, flags, globalscale, globalshift, epsilon,
                       stream=_stream_of(stream))
    return dst


def reformat(src, layout: str, *, stream=None) -> Tensor:
    """cvcuda.reformat (python/mod_cvcuda/OpReformat.cpp): the tensor in another of the NHWC / NCHW / HWC / CHW layouts."""
    t = as_tensor(src)
    return _wrap(ops.reformat(t._t, str(layout), src_layout=t.layout, stream=_stream_of(stream)), str(layout))


def reformat_into(dst: Tensor, src, *, stream=None) -> Tensor:
    t, d = as_tensor(src), as_tensor(dst)
    ops.reformat_into(d._t, t._t, src_layout=t.layout, dst_layout=d.layout, stream=_stream_of(stream))
    return dst


def convertto(src, dtype, scale: float = 1.0, offset: float = 0.0, *, stream=None) -> Tensor:
    """cvcuda.convertto (python/mod_cvcuda/OpConvertTo.cpp)."""
    t = as_tensor(src)
    return _wrap(ops.convertto(t._t, _torch_dtype(dtype), scale, offset, stream=_stream_of(stream)), t.layout)


def convertto_into(dst: Tensor, src, scale: float = 1.0, offset: float = 0.0, *, stream=None) -> Tensor:
    ops.convertto_into(as_tensor(dst)._t, as_tensor(src)._t, scale, offset, stream=_stream_of(stream))
    return dst


def copymakeborder(src, border_mode: Border = Border.CONSTANT, border_value=(), *, top, bottom, left, right, stream=None):
    """cvcuda.copymakeborder (python/mod_cvcuda/OpCopyMakeBorder.cpp)."""
    s, lay = _src_of(src)
    if lay is None:
        tops = _flat_int32(top, "top") if not isinstance(top, (list, tuple)) else top
        lefts = _flat_int32(left, "left") if not isinstance(left, (list, tuple)) else left
        return ops.copymakeborder(s, border_mode, border_value, top=tops, left=lefts, bottom=bottom, right=right,
                                  stream=_stream_of(stream))
    out = ops.copymakeborder(s, border_mode, border_value, top=top, left=left, bottom=bottom, right=right, stream=_stream_of(stream))
    return _wrap(out, lay)


def random_resized_crop(src, shape_or_sizes, min_scale: float = 0.08, max_scale: float = 1.0, min_ratio: float = 0.75,
                        max_ratio: float = 1.3333333333333333, interp: Interp = Interp.LINEAR, seed: int = 0, *, stream=None):
    """cvcuda.random_resized_crop (python/mod_cvcuda/OpRandomResizedCrop.cpp)."""
    s, lay = _src_of(src)
    out = ops.random_resized_crop(s, shape_or_sizes, min_scale, max_scale, min_ratio, max_ratio, interp, seed, stream=_stream_of(stream))
    return out if lay is None else _wrap(out, lay)
