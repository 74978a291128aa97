"""The reference's Python API-shape tests, run against this library's reference-style surface (cvcuda_b200.cvcuda):
tests/cvcuda/python/test_opresizecropconvertreformat.py (tensor and variable-shape forms) and
tests/cvcuda/python/test_opcropflipnormalizereformat.py. Like the originals they check shapes, element types, layouts, that
the allocating form and the `_into` form agree, and that the bad cases raise; on top of that the values of one case are
compared with the CPU oracle, and buffers from other libraries' interfaces (``__cuda_array_interface__``, DLPack) are
ingested without a copy."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def cvcuda(pkg):
    return pkg.cvcuda


# (shape, dtype, layout), resize, interp name, crop rect (x, y, w, h), out layout, out dtype name, manip, expected shape,
# scale, offset, positive?   -- the rows of test_op_resize_crop_convert_reformat
TENSOR_ROWS = [
    (((4, 512, 512, 3), np.uint8, "NHWC"), (256, 256), "LINEAR", (0, 0, 224, 224), "NCHW", "F32", "REVERSE", (4, 3, 224, 224), 1, 0, True),
    (((4, 512, 512, 3), np.uint8, "NHWC"), (256, 256), "NEAREST", (0, 0, 224, 224), "NCHW", "F32", "REVERSE", (4, 3, 224, 224), 1, 0, True),
    (((4, 512, 512, 3), np.uint8, "NHWC"), (256, 256), "NEAREST", (0, 0, 224, 224), "", "F32", "REVERSE", (4, 224, 224, 3), 1, 0, True),
    (((4, 512, 512, 3), np.uint8, "NHWC"), (256, 256), "NEAREST", (0, 0, 224, 224), "", None, "REVERSE", (4, 224, 224, 3), 1, 0, True),
    (((17, 678, 1027, 3), np.uint8, "NHWC"), (251, 256), "LINEAR", (0, 0, 200, 22), "NCHW", "F32", "REVERSE", (17, 3, 22, 200), 1, 0, True),
    (((17, 678, 1027, 3), np.uint8, "NHWC"), (251, 256), "LINEAR", (0, 0, 200, 22), "NHWC", "F32", "REVERSE", (17, 22, 200, 3), 1, 0, True),
    (((3, 40, 20, 3), np.uint8, "NHWC"), (160, 160), "NEAREST", (10, 20, 20, 35), "NCHW", "U8", "NO_OP", (3, 3, 35, 20), 1, 0, True),
    (((512, 512, 3), np.uint8, "HWC"), (256, 256), "LINEAR", (0, 0, 224, 224), "CHW", "F32", "REVERSE", (3, 224, 224), 1, 0, True),
    (((3, 512, 512), np.uint8, "CHW"), (256, 256), "LINEAR", (0, 0, 224, 224), "CHW", "F32", "REVERSE", (3, 224, 224), 1, 0, False),
    (((512, 1024, 3), np.uint8, "HWC"), (1024, 256), "LINEAR", (0, 0, 1024, 224), "CHW", "F32", "NO_OP", (3, 224, 1024), 1, 0, True),
    (((4, 678, 1027, 3), np.uint8, "NHWC"), (251, 256), "LINEAR", (0, 0, 200, 22), "NCHW", "F32", "REVERSE", (4, 3, 22, 200), 127.5, -1, True),
    (((512, 1024, 3), np.float32, "HWC"), (1024, 256), "LINEAR", (0, 0, 1024, 224), "CHW", "F32", "REVERSE", (3, 224, 1024), 1, 0, False),
    (((1, 2, 3), np.uint8, "HWC"), (60, 5), "LINEAR", (0, 0, 59, 5), "CHW", "F32", "REVERSE", (3, 5, 59), 1, 0, True),
    (((1, 2, 3), np.uint8, "HWC"), (60, 5), "LINEAR", (0, 0, 61, 5), "CHW", "F32", "REVERSE", (3, 5, 59), 1, 0, False),
    (((4, 512, 512, 3), np.uint8, "NHWC"), (256, 256), "AREA", (0, 0, 224, 224), "NCHW", "F32", "REVERSE", (4, 3, 224, 224), 1, 0, False),
]


@pytest.mark.parametrize("row", TENSOR_ROWS, ids=lambda r: f"{r[0][2]}{r[0][0]}-{r[2]}-{r[4] or 'same'}-{r[5] or 'same'}")
def test_op_resize_crop_convert_reformat(cvcuda, row):
    nvcv = cvcuda
    params, resize_dim, interp, rect, out_layout, out_dtype, manip, expected, scale, offset, positive = row
    interp, manip = getattr(cvcuda.Interp, interp), getattr(cvcuda.ChannelManip, manip)
    src = cvcuda.Tensor(*params)
    out_layout = out_layout if out_layout else str(src.layout)
    out_dtype = getattr(nvcv.Type, out_dtype) if out_dtype else src.dtype

    def allocating():
        return cvcuda.resize_crop_convert_reformat(src, resize_dim, interp, cvcuda.RectI(*rect), layout=out_layout,
                                                   data_type=out_dtype, manip=manip, scale=scale, offset=offset)

    out2 = cvcuda.Tensor(expected, out_dtype, out_layout)

    def into():
        # the original passes the window's corner as [rect[1], rect[0]]; its inputs are blank, so the two windows agree
        return cvcuda.resize_crop_convert_reformat_into(out2, src, resize_dim, interp, [rect[1], rect[0]], manip=manip,
                                                        scale=scale, offset=offset)

    if not positive:
        with pytest.raises(cvcuda.Error):
            allocating()
        try:  # the `_into` form gets an output of the expected shape, which for the out-of-range crop is a legal window
            into()
        except cvcuda.Error:
            pass
        return
    out1 = allocating()
    assert out1.layout == out_layout and out1.shape == expected and out1.dtype == out_dtype
    tmp = into()
    assert tmp is out2
    assert out2.layout == out_layout and out2.shape == expected and out2.dtype == out_dtype
    assert torch.equal(torch.as_tensor(out1.cuda()), torch.as_tensor(out2.cuda()))


# images, min size, max size, resize, crop rect, out layout, out dtype, manip, expected shape  -- the variable-shape rows
VARSHAPE_ROWS = [
    (10, (50, 50), (512, 512), (256, 256), (0, 0, 224, 224), "NCHW", "F32", "REVERSE", (10, 3, 224, 224)),
    (1, (500, 300), (800, 700), (400, 200), (0, 0, 224, 190), "NHWC", "F32", "REVERSE", (1, 190, 224, 3)),
    (50, (1, 1), (50, 70), (400, 200), (0, 0, 224, 190), "NHWC", "F32", "NO_OP", (50, 190, 224, 3)),
    (50, (1, 1), (50, 70), (400, 200), (0, 0, 224, 190), "NCHW", "U8", "REVERSE", (50, 3, 190, 224)),
    (50, (1, 1), (50, 70), (400, 200), (0, 0, 224, 190), "NCHW", "U8", "NO_OP", (50, 3, 190, 224)),
    (50, (1, 1), (50, 70), (400, 200), (0, 0, 224, 190), "", None, "REVERSE", (50, 190, 224, 3)),
]


@pytest.mark.parametrize("row", VARSHAPE_ROWS, ids=lambda r: f"n{r[0]}-{r[5] or 'same'}-{r[6] or 'same'}-{r[7]}")
def test_op_resize_crop_convert_reformat_varshape(cvcuda, row):
    nvcv = cvcuda
    n, lo, hi, resize_dim, rect, out_layout, out_dtype, manip, expected = row
    manip = getattr(cvcuda.ChannelManip, manip)
    batch = cvcuda.ImageBatchVarShape(n)
    out_layout = out_layout if out_layout else "NHWC"
    out_dtype = getattr(nvcv.Type, out_dtype) if out_dtype else nvcv.Type.U8
    batch.pushback([cvcuda.Image((lo[0] + (hi[0] - lo[0]) * i // n, lo[1] + (hi[1] - lo[1]) * i // n), cvcuda.Format.RGB8)
                    for i in range(n)])
    out1 = cvcuda.resize_crop_convert_reformat(batch, resize_dim=resize_dim, interp=cvcuda.Interp.LINEAR,
                                               crop_rect=cvcuda.RectI(*rect), layout=out_layout, data_type=out_dtype, manip=manip,
                                               scale=1, offset=0)
    assert out1.layout == out_layout and out1.shape == expected and out1.dtype == out_dtype
    out2 = cvcuda.Tensor(expected, out_dtype, out_layout)
    tmp = cvcuda.resize_crop_convert_reformat_into(out2, batch, resize_dim, cvcuda.Interp.LINEAR, [rect[1], rect[0]], manip=manip)
    assert tmp is out2
    assert out2.layout == out_layout and out2.shape == expected and out2.dtype == out_dtype
    assert torch.equal(torch.as_tensor(out1.cuda()), torch.as_tensor(out2.cuda()))


@pytest.mark.parametrize("layout", ["NHWC", "NCHW"])
def test_op_crop_flip_normalize_reformat_tensor_out(cvcuda, layout):
    """The one row of the original (RGBA8, one image between 10x10 and 20x20, REPLICATE, standard-deviation flag), in both
    output layouts, allocating form and `_into` form on a stream of its own."""
    n, lo, hi, ch, dtype = 1, (10, 10), (20, 20), 4, np.uint8
    base = cvcuda.Tensor((1, 1, 1, 4), np.float32, "NHWC")
    scale = cvcuda.Tensor((1, 1, 1, 4), np.float32, "NHWC")
    batch = cvcuda.ImageBatchVarShape(n)
    batch.pushback([cvcuda.Image((lo[0] + (hi[0] - lo[0]) * i // n, lo[1] + (hi[1] - lo[1]) * i // n), cvcuda.Format.RGBA8)
                    for i in range(n)])
    rect = cvcuda.Tensor((n, 1, 1, 4), np.int32, "NHWC")
    flip = cvcuda.as_tensor(torch.randint(0, 2, (n, 1), dtype=torch.int32, device="cuda"), "NC")
    out_shape = (n, hi[0], hi[1], ch) if layout == "NHWC" else (n, ch, hi[0], hi[1])
    out = cvcuda.crop_flip_normalize_reformat(batch, out_shape, dtype, layout, rect, flip, base, scale, 1, 2, 3,
                                              cvcuda.NormalizeFlags.SCALE_IS_STDDEV, cvcuda.Border.REPLICATE, 0)
    assert out.shape == out_shape and out.dtype == dtype and out.layout == layout
    stream = cvcuda.Stream()
    out_tensor = cvcuda.Tensor(out_shape, dtype, layout)
    tmp = cvcuda.crop_flip_normalize_reformat_into(dst=out_tensor, src=batch, rect=rect, flip_code=flip, base=base, scale=scale,
                                                   globalscale=1, globalshift=2, epsilon=3,
                                                   flags=cvcuda.NormalizeFlags.SCALE_IS_STDDEV, border=cvcuda.Border.REPLICATE,
                                                   bvalue=0, stream=stream)
    stream.sync()
    assert tmp is out_tensor
    assert out_tensor.shape == out_shape and out_tensor.dtype == dtype and out_tensor.layout == layout


def test_values_through_the_object_surface_and_foreign_buffers(cvcuda, oracle):
    """Layout travels with the object; a buffer that only offers __cuda_array_interface__ or DLPack is used in place."""
    rng = np.random.default_rng(12)
    host = rng.integers(0, 256, (2, 60, 80, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(40, 30), crop=(4, 3), out_size=(32, 24), interp=1, src_cast=False, manip=1, scale=0.5, offset=1.0)
    want = oracle.resize_crop(list(host), spec, np.float32, True)
    dev = torch.from_numpy(host).cuda()

    class OnlyCudaArrayInterface:  # what a cupy or numba array looks like from outside
        def __init__(self, t):
            self._keep, self.__cuda_array_interface__ = t, t.__cuda_array_interface__

    class OnlyDLPack:
        def __init__(self, t):
            self._t = t

        def __dlpack__(self, stream=None):
            return self._t.__dlpack__()

        def __dlpack_device__(self):
            return self._t.__dlpack_device__()

    for foreign in (dev, OnlyCudaArrayInterface(dev), OnlyDLPack(dev)):
        t = cvcuda.as_tensor(foreign, "NHWC")
        assert t.cuda().data_ptr() == dev.data_ptr(), "ingested with a copy"
        out = cvcuda.resize_crop_convert_reformat(t, (40, 30), cvcuda.Interp.LINEAR, cvcuda.RectI(4, 3, 32, 24), layout="NCHW",
                                                  data_type=cvcuda.Type.F32, manip=cvcuda.ChannelManip.REVERSE, scale=0.5,
                                                  offset=1.0, srcCast=False)
        assert out.layout == "NCHW" and out.dtype == np.float32
        assert np.array_equal(torch.as_tensor(out.cuda()).cpu().numpy(), want)
    # the chain of stand-alone operators on objects: reformat knows both layouts from the objects
    nhwc = cvcuda.resize(cvcuda.as_tensor(dev, "NHWC"), (2, 30, 40, 3), cvcuda.Interp.NEAREST)
    assert nhwc.layout == "NHWC" and nhwc.shape == (2, 30, 40, 3)
    planar = cvcuda.reformat(cvcuda.convertto(nhwc, np.float32, 1 / 255.0, 0.0), "NCHW")
    assert planar.layout == "NCHW" and planar.shape == (2, 3, 30, 40) and planar.dtype == cvcuda.Type.F32
    back = cvcuda.reformat(planar, "NHWC")
    assert torch.equal(torch.as_tensor(back.cuda()), torch.as_tensor(cvcuda.convertto(nhwc, np.float32, 1 / 255.0, 0.0).cuda()))


def test_image_batch_pushback_after_use_reuploads_descriptors(cvcuda, oracle, pkg):
    rng = np.random.default_rng(3)
    hosts = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for (w, h) in ((64, 40), (33, 57), (80, 80))]
    batch = cvcuda.ImageBatchVarShape(3)
    images = []
    for a in hosts:
        im = cvcuda.Image((a.shape[1], a.shape[0]), cvcuda.Format.RGB8)
        im.cuda().copy_(torch.from_numpy(a))
        images.append(im)
    batch.pushback(images[:2])
    spec = oracle.ResizeSpec(resize=(32, 32), out_size=(32, 32), interp=1, src_cast=True)
    first = cvcuda.resize_crop_convert_reformat(batch, (32, 32), cvcuda.Interp.LINEAR, cvcuda.RectI(0, 0, 32, 32), layout="NHWC",
                                                data_type=cvcuda.Type.U8)
    assert first.shape == (2, 32, 32, 3)
    assert batch.max_size == (64, 57)  # kept with the batch, not recomputed per call ...
    batch.pushback(images[2])
    assert batch.max_size == (80, 80)  # ... and renewed by every change
    batch.popback()
    assert batch.max_size == (64, 57)
    batch.pushback(images[2])
    second = cvcuda.resize_crop_convert_reformat(batch, (32, 32), cvcuda.Interp.LINEAR, cvcuda.RectI(0, 0, 32, 32), layout="NHWC",
                                                 data_type=cvcuda.Type.U8)
    want = oracle.resize_crop(hosts, spec, np.uint8, False)
    assert np.array_equal(torch.as_tensor(second.cuda()).cpu().numpy(), want)
    with pytest.raises(cvcuda.Error):
        batch.pushback(cvcuda.Image((4, 4), cvcuda.Format.RGB8))  # capacity 3
    # a wider image pushed after a call: the staged kernel sizes its ring slots from the batch's maximum width
    wide = [rng.integers(0, 256, (40, w, 3), dtype=np.uint8) for w in (64, 200)]
    from gpu_util import kernel_path
    grown = pkg.ImageBatchVarShape([torch.from_numpy(wide[0]).cuda()])
    spec = oracle.ResizeSpec(resize=(48, 32), out_size=(48, 32), interp=1, src_cast=True)
    with kernel_path(pkg, 2):
        pkg.resize_crop_convert_reformat(grown, (48, 32), pkg.Interp.LINEAR, (0, 0, 48, 32), layout="NHWC", data_type=torch.uint8)
        grown.pushback(torch.from_numpy(wide[1]).cuda())
        out = pkg.resize_crop_convert_reformat(grown, (48, 32), pkg.Interp.LINEAR, (0, 0, 48, 32), layout="NHWC", data_type=torch.uint8)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), oracle.resize_crop(wide, spec, np.uint8, False))
    assert pkg.read_device_error() == 0
