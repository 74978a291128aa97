"""GPU parity of the stand-alone Normalize against the CPU oracle (bit-exact), through the plain-C entry point, the
Python mirror and the reference's own operator symbols: the reference's test table in tensor and variable-shape form,
other element types and channel counts, broadcast forms of base / scale, odd strides, and argument errors."""
import ctypes as C

import numpy as np
import pytest
import torch

import nvcv_fake as NF
import ref_tables as T
from gpu_util import kernel_path, _TORCH_DTYPE, padded_images, to_dev

pytestmark = pytest.mark.gpu


def _same(a, b, what):
    assert a.shape == b.shape and a.dtype == b.dtype, what
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{what}: {int((a != b).sum())} differing elements"


@pytest.mark.parametrize("idx", range(len(T.NORMALIZE_ROWS)))
def test_normalize_tensor_rows(pkg, oracle, idx):
    row = T.NORMALIZE_ROWS[idx]
    images, base, scale = T.normalize_case(row, 300 + idx)
    want = np.stack(oracle.normalize(images, base, scale, None, row.gscale, row.gshift, row.eps, row.flags))
    got = pkg.normalize(to_dev(np.stack(images)), to_dev(base), to_dev(scale), row.flags, row.gscale, row.gshift, row.eps)
    torch.cuda.synchronize()
    _same(got.cpu().numpy(), want, "tensor")


@pytest.mark.parametrize("idx", range(len(T.NORMALIZE_ROWS)))
def test_normalize_varshape_rows(pkg, oracle, idx):
    """Variable-shape form: per-image sizes, base / scale scalar or per channel (the reference's var-shape test uses
    [1,1,1,C] parameters, tests/cvcuda/system/TestOpNormalize.cpp:262-290)."""
    row = T.NORMALIZE_ROWS[idx]
    rng = np.random.default_rng(500 + idx)
    n = max(row.images, 2)
    images = [rng.integers(0, 256, (int(rng.integers(max(1, row.height * 8 // 10), row.height * 11 // 10 + 1)),
                                    int(rng.integers(max(1, row.width * 8 // 10), row.width * 11 // 10 + 1)), 4), dtype=np.uint8)
              for _ in range(n)]
    base = rng.uniform(0, 255, (1, 1, 1, 1 if row.scalar_base else 4)).astype(np.float32)
    scale = rng.uniform(0, 1, (1, 1, 1, 1 if row.scalar_scale else 4)).astype(np.float32)
    want = oracle.normalize(images, base, scale, None, row.gscale, row.gshift, row.eps, row.flags)
    src = pkg.ImageBatchVarShape(padded_images(images, pad_to=32))
    got = pkg.normalize(src, to_dev(base), to_dev(scale), row.flags, row.gscale, row.gshift, row.eps)
    torch.cuda.synchronize()
    for i in range(n):
        _same(got[i].cpu().numpy(), want[i], f"image {i}")


@pytest.mark.parametrize("src_dt,dst_dt", [(np.uint8, np.float32), (np.int8, np.int8), (np.uint16, np.uint16),
                                           (np.int16, np.float32), (np.int32, np.int32), (np.float32, np.uint8),
                                           (np.float32, np.float32)], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("ch", [1, 3, 4])
def test_normalize_types_channels_broadcast(pkg, oracle, src_dt, dst_dt, ch):
    rng = np.random.default_rng(ch)
    n, h, w = 3, 19, 23
    if src_dt == np.float32:
        images = [rng.uniform(-300, 300, (h, w, ch)).astype(np.float32) for _ in range(n)]
    else:
        info = np.iinfo(src_dt)
        lo, hi = max(info.min, -70000), min(info.max, 70000)
        images = [rng.integers(lo, hi + 1, (h, w, ch)).astype(src_dt) for _ in range(n)]
    for bshape, sshape in [((1, 1, 1, ch), (1, 1, 1, 1)), ((n, 1, 1, 1), (1, h, 1, ch)), ((1, 1, w, 1), (n, h, w, ch))]:
        base = rng.uniform(-50, 50, bshape).astype(np.float32)
        scale = rng.uniform(0.1, 2.0, sshape).astype(np.float32)
        for flags, eps in ((0, 0.0), (1, 0.5)):
            want = np.stack(oracle.normalize(images, base, scale, dst_dt, 1.5, -2.0, eps, flags))
            dst = torch.empty((n, h, w, ch), dtype=_TORCH_DTYPE[np.dtype(dst_dt)], device="cuda")
            pkg.normalize_into(dst, to_dev(np.stack(images)), to_dev(base), to_dev(scale), flags, 1.5, -2.0, eps)
            torch.cuda.synchronize()
            _same(dst.cpu().numpy(), want, f"base {bshape} scale {sshape} flags {flags}")


@pytest.mark.parametrize("ch", [1, 3, 4])
def test_normalize_float32_per_channel_both_kernels(pkg, oracle, ch):
    """float32 -> float32 with per-channel constants takes the vector kernel (rows on 16-byte boundaries) or its element
    path (any other row); both, and the arithmetic kernel (path 1), must equal the golden bit for bit at every width."""
    rng = np.random.default_rng(40 + ch)
    base = rng.uniform(-50, 50, (1, 1, 1, ch)).astype(np.float32)
    scale = rng.uniform(0.1, 2.0, (1, 1, 1, ch)).astype(np.float32)
    for w in list(range(1, 41)) + [224]:
        images = [rng.uniform(-300, 300, (7, w, ch)).astype(np.float32) for _ in range(2)]
        for flags, eps in ((0, 0.0), (1, 0.5)):
            want = np.stack(oracle.normalize(images, base, scale, np.float32, 1.5, -2.0, eps, flags))
            for path in (0, 1):
                dst = torch.empty((2, 7, w, ch), dtype=torch.float32, device="cuda")
                with kernel_path(pkg, path):
                    pkg.normalize_into(dst, to_dev(np.stack(images)), to_dev(base), to_dev(scale), flags, 1.5, -2.0, eps)
                torch.cuda.synchronize()
                _same(dst.cpu().numpy(), want, f"width {w} flags {flags} path {path}")


@pytest.mark.parametrize("dst_dt", [np.uint8, np.int8, np.uint16, np.int16, np.int32, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("ch", [1, 2, 3, 4])
def test_normalize_uint8_per_channel_both_kernels(pkg, oracle, dst_dt, ch):
    """uint8 sources with per-channel base / scale take the table kernel; kernel path 1 keeps the arithmetic kernel on the
    same inputs. Row lengths that are no multiple of four elements, aligned and unaligned rows, every destination type."""
    rng = np.random.default_rng(40 + ch)
    images = [rng.integers(0, 256, (9, 21, ch), dtype=np.uint8), rng.integers(0, 256, (14, 5, ch), dtype=np.uint8),
              rng.integers(0, 256, (3, 1, ch), dtype=np.uint8)]
    base = rng.uniform(0, 255, (1, 1, 1, ch)).astype(np.float32)
    scale = rng.uniform(0.2, 3.0, (1, 1, 1, ch)).astype(np.float32)
    for flags, eps, gs, sh in ((0, 0.0, 1.0, 0.0), (1, 0.25, 40.0, 100.0)):
        want = oracle.normalize(images, base, scale, dst_dt, gs, sh, eps, flags)
        for pad, off in ((32, 0), (1, 1)):
            for path in (0, 1):
                src = pkg.ImageBatchVarShape(padded_images(images, pad_to=pad, offset=off))
                dst = pkg.ImageBatchVarShape([torch.zeros(im.shape, dtype=_TORCH_DTYPE[np.dtype(dst_dt)], device="cuda")
                                              for im in images])
                with kernel_path(pkg, path):
                    pkg.normalize_into(dst, src, to_dev(base), to_dev(scale), flags, gs, sh, eps)
                torch.cuda.synchronize()
                for i in range(len(images)):
                    _same(dst[i].cpu().numpy(), want[i], f"image {i}, pad {pad}, path {path}, flags {flags}")


def test_normalize_strided_views_and_errors(pkg, oracle):
    rng = np.random.default_rng(9)
    images = [rng.integers(0, 256, (11, 13, 3), dtype=np.uint8) for _ in range(2)]
    base = rng.uniform(0, 255, (1, 1, 1, 3)).astype(np.float32)
    scale = rng.uniform(0, 1, (1, 1, 1, 3)).astype(np.float32)
    want = oracle.normalize(images, base, scale, np.float32)
    src = pkg.ImageBatchVarShape(padded_images(images, pad_to=1, offset=1))
    store = [torch.zeros((13, 16, 3), dtype=torch.float32, device="cuda") for _ in range(2)]
    dst = pkg.ImageBatchVarShape([t[1:12, 2:15] for t in store])
    pkg.normalize_into(dst, src, to_dev(base), to_dev(scale))
    torch.cuda.synchronize()
    for i in range(2):
        _same(dst[i].cpu().numpy(), want[i], f"image {i}")
        frame = store[i].cpu().numpy().copy()
        frame[1:12, 2:15] = 0
        assert not frame.any(), "wrote outside the destination view"
    INVALID = pkg.ops.Status.ERROR_INVALID_ARGUMENT
    t8 = torch.zeros((2, 4, 4, 3), dtype=torch.uint8, device="cuda")
    b, s = to_dev(base), to_dev(scale)
    for bad in (lambda: pkg.normalize_into(torch.zeros((1, 4, 4, 3), dtype=torch.uint8, device="cuda"), t8, b, s),
                lambda: pkg.normalize_into(torch.zeros((2, 4, 4, 4), dtype=torch.uint8, device="cuda"), t8, b, s),
                lambda: pkg.normalize_into(torch.zeros((2, 4, 5, 3), dtype=torch.uint8, device="cuda"), t8, b, s),
                lambda: pkg.normalize_into(torch.zeros((2, 4, 4, 3), dtype=torch.float16, device="cuda"), t8, b, s),
                lambda: pkg.normalize_into(torch.zeros((2, 4, 4, 3), dtype=torch.uint8, device="cuda"), t8, b.double(), s)):
        with pytest.raises(pkg.ops.Error) as e:
            bad()
        assert e.value.status == INVALID
    assert pkg.normalize(torch.empty((0, 4, 4, 3), dtype=torch.uint8, device="cuda"), b, s).shape == (0, 4, 4, 3)


def test_normalize_refuses_base_and_scale_shapes_that_do_not_broadcast(pkg):
    """Every extent of base / scale must be 1 or the input's (src/cvcuda/priv/legacy/normalize.cu:300-306); for an image
    batch, whose images have no common size, rows and columns must be 1. Checked through the Python mirror and through
    the operator symbols."""
    INVALID = pkg.ops.Status.ERROR_INVALID_ARGUMENT
    src = torch.zeros((2, 8, 6, 3), dtype=torch.uint8, device="cuda")
    dst = torch.zeros_like(src)
    one = torch.ones((1, 1, 1, 3), dtype=torch.float32, device="cuda")
    shapes = [(1, 2, 1, 3), (1, 1, 5, 3), (3, 1, 1, 3), (1, 1, 1, 4), (1, 1, 1, 2), (1, 16, 1, 3)]
    batch = pkg.ImageBatchVarShape([torch.zeros((8, 6, 3), dtype=torch.uint8, device="cuda") for _ in range(2)])
    bout = pkg.ImageBatchVarShape([torch.zeros((8, 6, 3), dtype=torch.uint8, device="cuda") for _ in range(2)])
    ops = NF.bind_operators(pkg.lib_path())
    stream = torch.cuda.current_stream().cuda_stream
    h_op = C.c_void_p()
    assert ops.cvcudaNormalizeCreate(C.byref(h_op)) == 0
    for shape in shapes + [(1, 8, 6, 3)]:
        p = torch.ones(shape, dtype=torch.float32, device="cuda")
        full = shape == (1, 8, 6, 3)  # fits the tensor, not the image batch
        for args in ((dst, src, p, one), (dst, src, one, p), (bout, batch, p, one)):
            if full and args[0] is dst:
                pkg.normalize_into(*args)
                continue
            with pytest.raises(pkg.ops.Error) as e:
                pkg.normalize_into(*args)
            assert e.value.status == INVALID
        st = ops.cvcudaNormalizeSubmit(h_op, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(p, "NHWC"),
                                       NF.tensor_handle(one, "NHWC"), NF.tensor_handle(dst, "NHWC"), 1.0, 0.0, 0.0, 0)
        assert st == (0 if full else 2), shape
        st = ops.cvcudaNormalizeVarShapeSubmit(h_op, stream, NF.image_batch_handle(batch), NF.tensor_handle(one, "NHWC"),
                                               NF.tensor_handle(p, "NHWC"), NF.image_batch_handle(bout), 1.0, 0.0, 0.0, 0)
        assert st == 2, shape
    torch.cuda.synchronize()
    ops.nvcvOperatorDestroy(h_op)


def test_normalize_through_operator_symbols(pkg, oracle):
    ops = NF.bind_operators(pkg.lib_path())
    stream = torch.cuda.current_stream().cuda_stream
    row = T.NORMALIZE_ROWS[3]  # full-size base and scale
    images, base, scale = T.normalize_case(row, 77)
    want = np.stack(oracle.normalize(images, base, scale, None, row.gscale, row.gshift, row.eps, row.flags))
    src, dst = to_dev(np.stack(images)), torch.empty((row.images, row.height, row.width, 4), dtype=torch.uint8, device="cuda")
    tb, ts = to_dev(base), to_dev(scale)
    h_op = C.c_void_p()
    assert ops.cvcudaNormalizeCreate(C.byref(h_op)) == 0
    st = ops.cvcudaNormalizeSubmit(h_op, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(tb, "NHWC"),
                                   NF.tensor_handle(ts, "NHWC"), NF.tensor_handle(dst, "NHWC"), row.gscale, row.gshift,
                                   row.eps, row.flags)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    _same(dst.cpu().numpy(), want, "tensor handles")
    # layouts differ -> INVALID_ARGUMENT; another operator's handle -> NOT_COMPATIBLE
    chw = torch.empty((row.images, 4, row.height, row.width), dtype=torch.uint8, device="cuda")
    assert ops.cvcudaNormalizeSubmit(h_op, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(tb, "NHWC"),
                                     NF.tensor_handle(ts, "NHWC"), NF.tensor_handle(chw, "NCHW"), 1.0, 0.0, 0.0, 0) == 2
    other = C.c_void_p()
    assert ops.cvcudaResizeCreate(C.byref(other)) == 0
    assert ops.cvcudaNormalizeSubmit(other, stream, NF.tensor_handle(src, "NHWC"), NF.tensor_handle(tb, "NHWC"),
                                     NF.tensor_handle(ts, "NHWC"), NF.tensor_handle(dst, "NHWC"), 1.0, 0.0, 0.0, 0) == 9
    ops.nvcvOperatorDestroy(other)

    rng = np.random.default_rng(5)
    vimages = [rng.integers(0, 256, (h, w, 4), dtype=np.uint8) for (w, h) in ((30, 17), (8, 40))]
    pb = rng.uniform(0, 255, (1, 1, 1, 4)).astype(np.float32)
    ps = rng.uniform(0, 1, (1, 1, 1, 4)).astype(np.float32)
    vwant = oracle.normalize(vimages, pb, ps, None, 1.25, 3.0, 0.1, 1)
    bin_ = pkg.ImageBatchVarShape(padded_images(vimages))
    bout = pkg.ImageBatchVarShape([torch.empty(im.shape, dtype=torch.uint8, device="cuda") for im in vimages])
    tpb, tps = to_dev(pb), to_dev(ps)
    st = ops.cvcudaNormalizeVarShapeSubmit(h_op, stream, NF.image_batch_handle(bin_), NF.tensor_handle(tpb, "NHWC"),
                                           NF.tensor_handle(tps, "NHWC"), NF.image_batch_handle(bout), 1.25, 3.0, 0.1, 1)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    for i in range(2):
        _same(bout[i].cpu().numpy(), vwant[i], f"batch handles, image {i}")
    ops.nvcvOperatorDestroy(h_op)
