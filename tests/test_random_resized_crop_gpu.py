"""GPU parity of RandomResizedCrop and of the resized-crop kernel under it, against the CPU restatement of the
reference's golden (test::ResizedCrop, tests/cvcuda/system/ResizeUtils.cpp:189-241 with crop arguments) and the
rectangle sequences of the reference test's GetCropParams (tests/golden/random_crop_golden.npz, generated from the
reference function): the reference's table rows (nearest / linear), tensors and variable-shape batches, every element
type, the operator symbols with their generator state, and the reference's negative cases. Bit-exact for the integer
types (the reference's own test allows +-1 because its kernel blends in float32)."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import nvcv_fake as NF
from gpu_util import _TORCH_DTYPE, padded_images, to_dev

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
PARAMS = (0.08, 1.0, 3.0 / 4.0, 4.0 / 3.0)  # TestOpRandomResizedCrop.cpp:128-131
# srcWidth, srcHeight, dstWidth, dstHeight, interpolation, images (TestOpRandomResizedCrop.cpp:97-106; cubic rows left out)
REF_ROWS = [(42, 48, 23, 24, 0, 1), (113, 12, 12, 36, 0, 1), (421, 148, 223, 124, 0, 2), (313, 212, 412, 336, 0, 3),
            (42, 40, 21, 20, 1, 1), (21, 21, 42, 42, 1, 1), (420, 420, 210, 210, 1, 4), (210, 210, 420, 420, 1, 5)]


def _image(rng, w, h, ch, dt):
    if dt == np.float32:
        return rng.uniform(0.0, 300.0, (h, w, ch)).astype(np.float32)
    info = np.iinfo(dt)
    return rng.integers(info.min, int(info.max) + 1, (h, w, ch)).astype(dt)


def _same(a, b, what):
    assert a.shape == b.shape and a.dtype == b.dtype, what
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{what}: {int((a != b).sum())} differing elements"


def test_generator_matches_the_committed_reference_sequences(pkg):
    g = np.load(os.path.join(HERE, "golden", "random_crop_golden.npz"))
    for k in range(int(g["count"])):
        seed = int(g[f"seq{k}_seed"])
        par = [float(v) for v in g[f"seq{k}_par"]]
        sizes = [tuple(int(v) for v in s) for s in g[f"seq{k}_sizes"]]
        got = np.array(pkg.random_crop_rects(sizes, *par, seed=seed), np.int32)
        assert np.array_equal(got, g[f"seq{k}_rects"]), f"sequence {k}"


@pytest.mark.parametrize("row", REF_ROWS, ids=lambda r: "x".join(str(v) for v in r))
def test_reference_table_tensor_and_varshape(pkg, oracle, row):
    sw, sh, dw, dh, interp, n = row
    rng = np.random.default_rng(sw + dh)
    images = [_image(rng, sw, sh, 4, np.uint8) for _ in range(n)]  # RGBA8, as the reference test
    seed = 1
    rects = pkg.random_crop_rects([(sw, sh)] * n, *PARAMS, seed=seed)
    want = oracle.resize_plain(images, [(dw, dh)] * n, interp, rects=rects)
    got = pkg.random_resized_crop(to_dev(np.stack(images)), (n, dh, dw, 4), *PARAMS, interp, seed)
    torch.cuda.synchronize()
    _same(got.cpu().numpy(), np.stack(want), "tensor")
    # variable-shape: image sizes drawn around the row's size (TestOpRandomResizedCrop.cpp:240-262), own rectangles
    var = [_image(rng, int(rng.integers(max(2, sw * 8 // 10), sw * 11 // 10 + 1)),
                  int(rng.integers(max(2, sh * 8 // 10), sh * 11 // 10 + 1)), 4, np.uint8) for _ in range(n)]
    sizes = [(int(rng.integers(max(2, dw * 8 // 10), dw * 11 // 10 + 1)), int(rng.integers(max(2, dh * 8 // 10), dh * 11 // 10 + 1)))
             for _ in range(n)]
    rects = pkg.random_crop_rects([(im.shape[1], im.shape[0]) for im in var], *PARAMS, seed=seed)
    want = oracle.resize_plain(var, sizes, interp, rects=rects)
    got = pkg.random_resized_crop(pkg.ImageBatchVarShape(padded_images(var, pad_to=32)), sizes, *PARAMS, interp, seed)
    torch.cuda.synchronize()
    for i in range(n):
        _same(got[i].cpu().numpy(), want[i], f"var-shape image {i}")


@pytest.mark.parametrize("dt", [np.uint8, np.uint16, np.int16, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("ch", [1, 3, 4])
@pytest.mark.parametrize("interp", [0, 1])
def test_resized_crop_types_channels_rectangles(pkg, oracle, dt, ch, interp):
    """Caller-chosen rectangles: whole image, a 1 x 1 corner, up- and down-scaled interiors, rectangles reaching past the
    image (taps clamp at the image's edges, as in the golden); odd pitches and bases."""
    rng = np.random.default_rng(7 * ch + interp)
    images = [_image(rng, 37, 29, ch, dt), _image(rng, 64, 5, ch, dt), _image(rng, 3, 50, ch, dt), _image(rng, 40, 40, ch, dt),
              _image(rng, 20, 30, ch, dt)]
    rects = [(0, 0, 37, 29), (63, 4, 1, 1), (1, 10, 2, 30), (5, 6, 30, 31), (10, 20, 25, 25)]
    sizes = [(50, 41), (9, 40), (31, 7), (17, 13), (33, 19)]
    want = oracle.resize_plain(images, sizes, interp, golden_float=False, rects=rects)
    es = np.dtype(dt).itemsize
    src = pkg.ImageBatchVarShape(padded_images(images, pad_to=es, offset=es))
    dst = pkg.ImageBatchVarShape([torch.zeros((h, w, ch), dtype=_TORCH_DTYPE[np.dtype(dt)], device="cuda") for (w, h) in sizes])
    pkg.resized_crop_into(dst, src, to_dev(np.array(rects, np.int32)), interp)
    torch.cuda.synchronize()
    for i in range(len(images)):
        _same(dst[i].cpu().numpy(), want[i], f"image {i}")  # float32: the golden's double-precision sum, un-rounded


def test_through_operator_symbols(pkg, oracle):
    """cvcudaRandomResizedCropCreate / Submit / VarShapeSubmit: the handle's generator advances from call to call exactly
    like one std::mt19937 walking through all the images (the way the reference test replays it)."""
    ops = NF.bind_operators(pkg.lib_path())
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(33)
    h_op = C.c_void_p()
    assert ops.cvcudaRandomResizedCropCreate(None, 0.2, 1.0, 0.8, 1.3, 2, 0) == 2     # TestOpRandomResizedCrop.cpp:356-359
    assert ops.cvcudaRandomResizedCropCreate(C.byref(h_op), 1.0, 0.2, 0.8, 1.3, 2, 0) == 2  # :361-365
    assert ops.cvcudaRandomResizedCropCreate(C.byref(h_op), 0.2, 1.0, 1.3, 0.8, 2, 0) == 2  # :367-371
    seed = 77
    assert ops.cvcudaRandomResizedCropCreate(C.byref(h_op), *PARAMS, 4, seed) == 0
    images = [_image(rng, 60, 44, 3, np.uint8) for _ in range(3)]
    var = [_image(rng, 50, 70, 3, np.uint8), _image(rng, 90, 30, 3, np.uint8)]
    all_sizes = [(60, 44)] * 3 + [(50, 70), (90, 30)] + [(60, 44)] * 3
    rects = pkg.random_crop_rects(all_sizes, *PARAMS, seed=seed)  # one generator over the three calls below

    tsrc, tdst = to_dev(np.stack(images)), torch.empty((3, 32, 40, 3), dtype=torch.uint8, device="cuda")
    st = ops.cvcudaRandomResizedCropSubmit(h_op, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), 1)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    _same(tdst.cpu().numpy(), np.stack(oracle.resize_plain(images, [(40, 32)] * 3, 1, rects=rects[:3])), "first call")

    bin_ = pkg.ImageBatchVarShape(padded_images(var, pad_to=32))
    out_sizes = [(31, 45), (64, 20)]
    bout = pkg.ImageBatchVarShape([torch.empty((h, w, 3), dtype=torch.uint8, device="cuda") for (w, h) in out_sizes])
    st = ops.cvcudaRandomResizedCropVarShapeSubmit(h_op, stream, NF.image_batch_handle(bin_), NF.image_batch_handle(bout), 0)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    want = oracle.resize_plain(var, out_sizes, 0, rects=rects[3:5])
    for i in range(2):
        _same(bout[i].cpu().numpy(), want[i], f"var-shape call, image {i}")

    st = ops.cvcudaRandomResizedCropSubmit(h_op, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), 0)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    _same(tdst.cpu().numpy(), np.stack(oracle.resize_plain(images, [(40, 32)] * 3, 0, rects=rects[5:])), "third call")

    # negative rows (TestOpRandomResizedCrop.cpp:375-384): layouts, element types, interpolation; cubic is refused
    chw = torch.empty((3, 24, 24), dtype=torch.uint8, device="cuda")
    hwc = torch.empty((24, 24, 2), dtype=torch.uint8, device="cuda")
    u32 = torch.empty((24, 24, 2), dtype=torch.int32, device="cuda")
    H = NF.tensor_handle
    assert ops.cvcudaRandomResizedCropSubmit(h_op, stream, H(chw, "CHW"), H(hwc, "HWC"), 0) == 2
    assert ops.cvcudaRandomResizedCropSubmit(h_op, stream, H(hwc, "HWC"), H(chw, "CHW"), 0) == 2
    assert ops.cvcudaRandomResizedCropSubmit(h_op, stream, H(u32, "HWC"), H(hwc, "HWC"), 0) == 2
    assert ops.cvcudaRandomResizedCropSubmit(h_op, stream, H(hwc, "HWC"), H(u32, "HWC"), 0) == 2
    assert ops.cvcudaRandomResizedCropSubmit(h_op, stream, H(hwc, "HWC"), H(hwc, "HWC"), 3) == 2   # NVCV_INTERP_AREA
    assert ops.cvcudaRandomResizedCropSubmit(h_op, stream, H(hwc, "HWC"), H(hwc, "HWC"), 2) == 1   # cubic: not implemented
    big = torch.empty((5, 8, 8, 3), dtype=torch.uint8, device="cuda")
    assert ops.cvcudaRandomResizedCropSubmit(h_op, stream, H(big, "NHWC"), H(big, "NHWC"), 0) == 2  # beyond maxBatchSize
    other = C.c_void_p()
    assert ops.cvcudaResizeCreate(C.byref(other)) == 0
    assert ops.cvcudaRandomResizedCropSubmit(other, stream, H(tsrc, "NHWC"), H(tdst, "NHWC"), 0) == 9
    ops.nvcvOperatorDestroy(other)
    ops.nvcvOperatorDestroy(h_op)


def test_python_negative_cases(pkg):
    u8 = torch.zeros((2, 16, 16, 3), dtype=torch.uint8, device="cuda")
    def status(fn):
        with pytest.raises(pkg.ops.Error) as e:
            fn()
        return e.value.status
    INVALID = pkg.ops.Status.ERROR_INVALID_ARGUMENT
    assert status(lambda: pkg.random_resized_crop(u8, (2, 8, 8, 3), 1.0, 0.2)) == INVALID
    assert status(lambda: pkg.random_resized_crop(u8, (2, 8, 8, 3), 0.2, 1.0, 1.3, 0.8)) == INVALID
    assert status(lambda: pkg.random_resized_crop(u8, (2, 8, 8, 3), interp=3)) == INVALID
    assert status(lambda: pkg.random_resized_crop(u8, (2, 8, 8, 3), interp=2)) == pkg.ops.Status.ERROR_NOT_IMPLEMENTED
    assert status(lambda: pkg.random_resized_crop(u8, (3, 8, 8, 3))) == INVALID
    assert status(lambda: pkg.resized_crop_into(torch.zeros((2, 8, 8, 3), dtype=torch.uint8, device="cuda"), u8,
                                                torch.zeros((1, 4), dtype=torch.int32, device="cuda"))) == INVALID
    # seed 0: a random seed; the result is still a valid crop of the right shape
    assert pkg.random_resized_crop(u8, (2, 8, 8, 3)).shape == (2, 8, 8, 3)
