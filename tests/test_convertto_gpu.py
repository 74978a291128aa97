"""GPU parity of the stand-alone ConvertTo against the reference test's expectation
SaturateCast<DstT>(alpha * val + beta) in double precision (tests/cvcuda/system/TestOpConvertTo.cpp:118-133, restated in
oracle.convert_to): the reference's own cases (constant images of value 0x10, its alpha / beta table, its six type
pairs), random data over every type pair, odd strides, the reference's negative table, and its operator symbols."""
import ctypes as C

import numpy as np
import pytest
import torch

import nvcv_fake as NF
from gpu_util import _TORCH_DTYPE, to_dev

pytestmark = pytest.mark.gpu

TYPES = [np.uint8, np.int8, np.uint16, np.int16, np.int32, np.float32]
# width, height, alpha, beta, batch (TestOpConvertTo.cpp:109-115); (from, to, channels) of its six tests (:118-237)
REF_PARAMS = [(5, 5, 1.0, 1.0, 1), (5, 5, 2.1, 2.0, 5), (1, 1, 2.1, -1.0, 1)]
REF_PAIRS = [(np.uint8, np.uint8, 4), (np.uint8, np.float32, 4), (np.float32, np.uint8, 4), (np.float32, np.float32, 4),
             (np.uint8, np.uint16, 1), (np.uint16, np.float32, 2), (np.uint8, np.float32, 3)]


def _same(a, b, what):
    assert a.shape == b.shape and a.dtype == b.dtype, what
    assert np.array_equal(a.view(np.uint8), b.view(np.uint8)), f"{what}: {int((a != b).sum())} differing elements"


@pytest.mark.parametrize("params", REF_PARAMS, ids=str)
@pytest.mark.parametrize("pair", REF_PAIRS, ids=lambda p: f"{np.dtype(p[0]).name}-{np.dtype(p[1]).name}x{p[2]}")
def test_reference_cases(pkg, oracle, params, pair):
    w, h, alpha, beta, n = params
    st, dt, ch = pair
    src = np.full((n, h, w, ch), 0x10, dtype=st)
    got = pkg.convertto(to_dev(src), _TORCH_DTYPE[np.dtype(dt)], alpha, beta)
    torch.cuda.synchronize()
    _same(got.cpu().numpy(), oracle.convert_to(src, dt, alpha, beta), "constant image")


@pytest.mark.parametrize("st", TYPES, ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("dt", TYPES, ids=lambda d: np.dtype(d).name)
def test_random_all_pairs(pkg, oracle, st, dt):
    rng = np.random.default_rng(17)
    shape = (2, 13, 37, 3)
    if st == np.float32:
        src = rng.uniform(-70000, 70000, shape).astype(np.float32)
        src.flat[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, 254.5, 255.5, 1e10]  # ties and saturation
    else:
        info = np.iinfo(st)
        src = rng.integers(info.min, int(info.max) + 1, shape).astype(st)
    for alpha, beta in ((1.0, 0.0), (0.5, 0.0), (2.1, -1.0), (-1.0 / 3.0, 127.5), (1e-3, 2.5)):
        got = pkg.convertto(to_dev(src), _TORCH_DTYPE[np.dtype(dt)], alpha, beta)
        torch.cuda.synchronize()
        _same(got.cpu().numpy(), oracle.convert_to(src, dt, alpha, beta), f"alpha {alpha} beta {beta}")


def test_strided_views_rank3_and_errors(pkg, oracle):
    rng = np.random.default_rng(4)
    big = rng.integers(0, 256, (2, 9, 40, 3), dtype=np.uint8)
    store = torch.zeros((2, 9, 40, 3), dtype=torch.float32, device="cuda")
    pkg.convertto_into(store[:, 1:8, 2:36], to_dev(big)[:, 1:8, 3:37], 1 / 255.0, -0.5)
    torch.cuda.synchronize()
    out = store.cpu().numpy()
    _same(np.ascontiguousarray(out[:, 1:8, 2:36]), oracle.convert_to(big[:, 1:8, 3:37], np.float32, 1 / 255.0, -0.5), "views")
    out[:, 1:8, 2:36] = 0
    assert not out.any(), "wrote outside the destination view"
    hwc = rng.integers(-32768, 32768, (11, 7, 4)).astype(np.int16)
    got = pkg.convertto(to_dev(hwc), torch.uint8, 0.01, 100.0)
    _same(got.cpu().numpy(), oracle.convert_to(hwc, np.uint8, 0.01, 100.0), "rank 3")
    # the reference's negative table (TestOpConvertTo.cpp:240-249): all NVCV_ERROR_INVALID_ARGUMENT
    INVALID = pkg.ops.Status.ERROR_INVALID_ARGUMENT
    f32 = torch.zeros((3, 24, 24, 1), dtype=torch.float32, device="cuda")
    for bad in (lambda: pkg.convertto(torch.zeros((3, 24, 24, 1), dtype=torch.float16, device="cuda"), torch.float32),
                lambda: pkg.convertto(f32, torch.float16),
                lambda: pkg.convertto_into(torch.zeros((3, 24, 25, 1), dtype=torch.float32, device="cuda"), f32),
                lambda: pkg.convertto_into(torch.zeros((3, 25, 24, 1), dtype=torch.float32, device="cuda"), f32),
                lambda: pkg.convertto_into(torch.zeros((4, 24, 24, 1), dtype=torch.float32, device="cuda"), f32)):
        with pytest.raises((pkg.ops.Error, KeyError)) as e:
            bad()
        if isinstance(e.value, pkg.ops.Error):
            assert e.value.status == INVALID
    assert pkg.convertto(torch.empty((0, 4, 4, 3), dtype=torch.uint8, device="cuda"), torch.float32).shape == (0, 4, 4, 3)


@pytest.mark.parametrize("st", [np.uint8, np.int8, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("dt", TYPES, ids=lambda d: np.dtype(d).name)
def test_vector_and_table_kernels_against_the_plain_one(pkg, oracle, st, dt):
    """8-bit sources take the table kernel and float32 sources the vector kernel when rows sit on word / vector
    boundaries; kernel path 1 keeps the element-by-element kernel. Views of wider storage give aligned rows with ragged
    ends (1, 2, 3 elements past the last full group)."""
    from gpu_util import kernel_path
    rng = np.random.default_rng(23)
    for w in (37, 38, 39, 40, 1):
        if st == np.float32:
            full = rng.uniform(-400, 400, (2, 13, 48, 3)).astype(np.float32)
            full.flat[:8] = [0.5, 1.5, 2.5, -0.5, -1.5, 254.5, 255.5, 1e10]
        else:
            info = np.iinfo(st)
            full = rng.integers(info.min, int(info.max) + 1, (2, 13, 48, 3)).astype(st)
        src = to_dev(full)[:, :, :w]
        for alpha, beta in ((1.0, 0.0), (0.7, 3.5), (-2.1, 100.25)):
            want = oracle.convert_to(full[:, :, :w], dt, alpha, beta)
            for path in (0, 1):
                store = torch.zeros((2, 13, 48, 3), dtype=_TORCH_DTYPE[np.dtype(dt)], device="cuda")
                with kernel_path(pkg, path):
                    pkg.convertto_into(store[:, :, :w], src, alpha, beta)
                torch.cuda.synchronize()
                out = store.cpu().numpy()
                _same(np.ascontiguousarray(out[:, :, :w]), want, f"w {w} alpha {alpha} path {path}")
                out[:, :, :w] = 0
                assert not out.view(np.uint8).any(), "wrote outside the destination view"


def test_convertto_through_operator_symbols(pkg, oracle):
    ops = NF.bind_operators(pkg.lib_path())
    stream = torch.cuda.current_stream().cuda_stream
    rng = np.random.default_rng(2)
    src = rng.integers(0, 256, (2, 24, 24, 4), dtype=np.uint8)
    tsrc, tdst = to_dev(src), torch.empty((2, 24, 24, 4), dtype=torch.float32, device="cuda")
    h_op = C.c_void_p()
    assert ops.cvcudaConvertToCreate(None) == 2  # TestOpConvertTo.cpp:281
    assert ops.cvcudaConvertToCreate(C.byref(h_op)) == 0
    st = ops.cvcudaConvertToSubmit(h_op, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), 2.1, -1.0)
    assert st == 0, NF.fake().fakeLastMessage()
    torch.cuda.synchronize()
    _same(tdst.cpu().numpy(), oracle.convert_to(src, np.float32, 2.1, -1.0), "tensor handles")
    # planar input -> INVALID_ARGUMENT (first row of the reference's negative table); another operator's handle
    chw = torch.empty((2, 4, 24, 24), dtype=torch.uint8, device="cuda")
    u8o = torch.empty((2, 24, 24, 4), dtype=torch.uint8, device="cuda")
    assert ops.cvcudaConvertToSubmit(h_op, stream, NF.tensor_handle(chw, "NCHW"), NF.tensor_handle(u8o, "NHWC"), 1.0, 0.0) == 2
    other = C.c_void_p()
    assert ops.cvcudaReformatCreate(C.byref(other)) == 0
    assert ops.cvcudaConvertToSubmit(other, stream, NF.tensor_handle(tsrc, "NHWC"), NF.tensor_handle(tdst, "NHWC"), 1.0, 0.0) == 9
    ops.nvcvOperatorDestroy(other)
    ops.nvcvOperatorDestroy(h_op)


@pytest.mark.parametrize("dt", [np.uint8, np.int8, np.uint16, np.int16], ids=lambda d: np.dtype(d).name)
def test_float32_fast_path_agrees_at_rounding_boundaries(pkg, oracle, dt):
    """float32 sources to small integers run a float32 multiply-add first and redo in double precision whatever lies near a
    rounding boundary: exact ties, values a few float32 steps either side of one, products that cancel against beta, factors
    float32 cannot hold, values far outside the type's range, NaN and infinities must all come out as the double-precision rule
    gives them."""
    info = np.iinfo(dt)
    k = np.arange(int(info.min) - 3, int(info.max) + 4, dtype=np.float64)
    ties = (k + 0.5).astype(np.float32)
    near = np.concatenate([np.nextafter(ties, np.float32(np.inf)), np.nextafter(ties, np.float32(-np.inf)),
                           np.nextafter(np.nextafter(ties, np.float32(np.inf)), np.float32(np.inf))])
    rng = np.random.default_rng(5)
    vals = np.concatenate([ties, near, rng.uniform(float(info.min) - 2, float(info.max) + 2, 4096).astype(np.float32),
                           np.array([1e10, -1e10, 3e38, -3e38, np.inf, -np.inf, 0.0, -0.0], np.float32)])
    vals = np.resize(vals, (1, (vals.size + 767) // 768, 256, 3)).astype(np.float32)  # rows of 768 elements: vector kernel
    src = to_dev(vals)
    cases = [(1.0, 0.0), (0.5, 0.25), (255.0, 0.0), (1.0 / 3.0, 0.5), (-1.0, 0.5), (1e6, -1e6 * 0.001), (1.0000000001, 0.0),
             (1e-3, 100.5), (3.0, -0.5)]
    for alpha, beta in cases:
        want = oracle.convert_to(vals, dt, alpha, beta)
        out = torch.zeros(vals.shape, dtype=_TORCH_DTYPE[np.dtype(dt)], device="cuda")
        pkg.convertto_into(out, src, alpha, beta)
        torch.cuda.synchronize()
        _same(out.cpu().numpy(), want, f"alpha {alpha} beta {beta}")
    # NaN: the reference's saturate cast is not defined for it; both kernels of this library must agree with each other
    from gpu_util import kernel_path
    nan = to_dev(np.full((1, 2, 256, 3), np.nan, np.float32))
    got = []
    for path in (0, 1):
        out = torch.zeros((1, 2, 256, 3), dtype=_TORCH_DTYPE[np.dtype(dt)], device="cuda")
        with kernel_path(pkg, path):
            pkg.convertto_into(out, nan, 2.0, 1.0)
        torch.cuda.synchronize()
        got.append(out.cpu().numpy())
    assert np.array_equal(got[0], got[1])
