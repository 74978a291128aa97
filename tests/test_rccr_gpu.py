"""GPU parity: ResizeCropConvertReformat (dense and var-shape) and its fused extensions, against the CPU oracle,
through the library's C entry points, on both kernel paths (1 = per-pixel gather, 2 = staged bulk-copy pipeline)."""
import numpy as np
import pytest
import torch

import ref_tables as T
from gpu_util import assert_parity, kernel_path, padded_images, to_dev

pytestmark = pytest.mark.gpu

PATHS = (1, 2, 3)  # per-pixel gather, staged pipeline, row walk
MEAN = (123.675, 116.28, 103.53)
STD = (58.395, 57.12, 57.375)
INV_STD = tuple(float(np.float32(1.0) / np.float32(s)) for s in STD)


def _torch_dtype(dt):
    return {np.uint8: torch.uint8, np.float32: torch.float32, np.float16: torch.float16}[dt]


def _run_dense(pkg, src, r, path):
    with kernel_path(pkg, path):
        out = pkg.resize_crop_convert_reformat(
            to_dev(src), r.resize, r.interp, (*r.crop, *r.out), layout="NCHW" if r.planar else "NHWC",
            data_type=_torch_dtype(r.dtype), manip=r.manip, scale=r.scale, offset=r.offset, srcCast=r.src_cast)
        torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("idx", range(len(T.RCCR_ROWS)))
def test_reference_table_tensor(pkg, oracle, idx):
    """The reference's 63 tensor test rows, on its ramp input and on seeded uniform bytes."""
    r = T.RCCR_ROWS[idx]
    w, h, n = r.src
    n = min(n, 3)
    rng = np.random.default_rng(1234 + idx)
    spec = oracle.ResizeSpec(resize=r.resize, crop=r.crop, out_size=r.out, interp=r.interp, src_cast=r.src_cast,
                             manip=r.manip, scale=r.scale, offset=r.offset)
    for name, src in (("ramp", T.ramp_batch(n, h, w)), ("uniform", rng.integers(0, 256, (n, h, w, 3), dtype=np.uint8))):
        want = oracle.resize_crop(list(src), spec, r.dtype, r.planar, nthreads=8)
        for path in PATHS:
            got = _run_dense(pkg, src, r, path)
            assert_parity(got, want, exact=(r.interp == T.NEAREST), what=f"row {idx} {name} path {path}")
    assert pkg.read_device_error() == 0


@pytest.mark.parametrize("idx", range(0, len(T.RCCR_ROWS), 3))
def test_reference_table_varshape(pkg, oracle, idx):
    """Var-shape variant of the reference test: image sizes drawn in [0.8, 1.2] x nominal when interpolating."""
    r = T.RCCR_ROWS[idx]
    w, h, n = r.src
    n = min(n, 4)
    rng = np.random.default_rng(4321 + idx)
    images = []
    for _ in range(n):
        iw = int(rng.integers(int(w * 0.8), int(w * 1.2) + 1)) if r.interp else w
        ih = int(rng.integers(int(h * 0.8), int(h * 1.2) + 1)) if r.interp else h
        images.append(rng.integers(0, 256, (max(ih, 1), max(iw, 1), 3), dtype=np.uint8))
    spec = oracle.ResizeSpec(resize=r.resize, crop=r.crop, out_size=r.out, interp=r.interp, src_cast=r.src_cast,
                             manip=r.manip, scale=r.scale, offset=r.offset)
    want = oracle.resize_crop(images, spec, r.dtype, r.planar, nthreads=8)
    batch = pkg.ImageBatchVarShape(padded_images(images))
    for path in PATHS:
        with kernel_path(pkg, path):
            out = pkg.resize_crop_convert_reformat(batch, r.resize, r.interp, (*r.crop, *r.out),
                                                   layout="NCHW" if r.planar else "NHWC",
                                                   data_type=_torch_dtype(r.dtype), manip=r.manip, scale=r.scale,
                                                   offset=r.offset, srcCast=r.src_cast)
            torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, exact=(r.interp == T.NEAREST), what=f"row {idx} path {path}")
    assert pkg.read_device_error() == 0


@pytest.mark.parametrize("src_cast", [False, True])
def test_config1_small_dense_batch(pkg, oracle, src_cast):
    """N=4, 480x640 RGB -> bilinear 256x256 -> centre 224x224 -> BGR -> float32 NCHW, value*(1/255)+0."""
    rng = np.random.default_rng(1234)
    src = rng.integers(0, 256, (4, 480, 640, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=1, src_cast=src_cast,
                             manip=1, scale=1.0 / 255.0, offset=0.0)
    want = oracle.resize_crop(list(src), spec, np.float32, True, nthreads=8)
    for path in PATHS:
        with kernel_path(pkg, path):
            out = pkg.resize_crop_convert_reformat(to_dev(src), (256, 256), pkg.Interp.LINEAR, (16, 16, 224, 224),
                                                   layout="NCHW", data_type=torch.float32,
                                                   manip=pkg.ChannelManip.REVERSE, scale=1.0 / 255.0, srcCast=src_cast)
            torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert got.shape == (4, 3, 224, 224)
        assert_parity(got, want, what=f"config 1 path {path}")
        assert np.array_equal(got, want), "expected bit-equality with the golden arithmetic"


def test_config2_classification_reduced_batch(pkg, oracle):
    """1080p -> 256x256 -> 224x224, per-channel mean/std, float32 NCHW (4 images instead of 256)."""
    rng = np.random.default_rng(1234)
    src = rng.integers(0, 256, (4, 1080, 1920, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=1, src_cast=False,
                             base=MEAN, mul=INV_STD)
    want = oracle.resize_crop(list(src), spec, np.float32, True, nthreads=8)
    tsrc = to_dev(src)
    for path in PATHS:
        out = torch.empty((4, 3, 224, 224), dtype=torch.float32, device="cuda")
        with kernel_path(pkg, path):
            pkg.fused_preprocess_into(out, tsrc, resize_dim=(256, 256), interp=1, crop_pos=(16, 16), layout="NCHW",
                                      base=MEAN, mul=INV_STD, srcCast=False)
            torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, what=f"config 2 path {path}")


def _random_resized_crop_rects(rng, sizes):
    """One rectangle per image: 8-100 % of the area, aspect in [3/4, 4/3], ten tries then a centre fallback."""
    rects = []
    for w, h in sizes:
        for _ in range(10):
            area = rng.uniform(0.08, 1.0) * w * h
            logr = rng.uniform(np.log(3 / 4), np.log(4 / 3))
            ar = np.exp(logr)
            cw, ch = int(round(np.sqrt(area * ar))), int(round(np.sqrt(area / ar)))
            if 0 < cw <= w and 0 < ch <= h:
                rects.append((int(rng.integers(0, w - cw + 1)), int(rng.integers(0, h - ch + 1)), cw, ch))
                break
        else:
            s = min(w, h)
            rects.append(((w - s) // 2, (h - s) // 2, s, s))
    return np.array(rects, np.int32)


def test_config3_varshape_crop_resize_flip_normalize_fp16(pkg, oracle):
    """Random rectangle -> bilinear 224x224 -> horizontal flip p=0.5 -> mean/std -> float16 NCHW (8 images)."""
    rng = np.random.default_rng(1234)
    n = 8
    sizes = [(int(rng.integers(480, 3841)), int(rng.integers(360, 2161))) for _ in range(n)]
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for w, h in sizes]
    rects = _random_resized_crop_rects(rng, sizes)
    flips = np.where(rng.random(n) < 0.5, 1, 2).astype(np.int32)
    flips[0], flips[1] = 1, 2
    spec = oracle.ResizeSpec(resize=(224, 224), out_size=(224, 224), interp=1, src_cast=True, base=MEAN, mul=INV_STD)
    want = oracle.resize_crop(images, spec, np.float16, True, roi=rects, flip=flips, nthreads=8)
    batch = pkg.ImageBatchVarShape(padded_images(images))
    for path in PATHS:
        out = torch.empty((n, 3, 224, 224), dtype=torch.float16, device="cuda")
        with kernel_path(pkg, path):
            pkg.fused_preprocess_into(out, batch, resize_dim=(224, 224), interp=1, layout="NCHW", base=MEAN,
                                      mul=INV_STD, srcCast=True, roi=to_dev(rects), flip_code=to_dev(flips))
            torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, what=f"config 3 path {path}")
    assert pkg.read_device_error() == 0


def test_config4_letterbox(pkg, oracle):
    """1080p -> 640x360 placed at rows 140..499 of a 640x640 canvas padded with 114, BGR, x/255, float32 NCHW."""
    rng = np.random.default_rng(1234)
    src = rng.integers(0, 256, (2, 1080, 1920, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(640, 360), out_size=(640, 360), interp=1, src_cast=True, manip=1,
                             scale=1.0 / 255.0, canvas=(640, 640), dst_pos=(0, 140), pad_value=114.0)
    want = oracle.resize_crop(list(src), spec, np.float32, True, nthreads=8)
    tsrc = to_dev(src)
    for path in PATHS:
        out = torch.full((2, 3, 640, 640), -1.0, dtype=torch.float32, device="cuda")
        with kernel_path(pkg, path):
            pkg.fused_preprocess_into(out, tsrc, resize_dim=(640, 360), interp=1, layout="NCHW", manip=1,
                                      scale=1.0 / 255.0, srcCast=True, dst_pos=(0, 140), region_size=(640, 360),
                                      pad_value=114.0)
            torch.cuda.synchronize()
        got = out.cpu().numpy()
        assert_parity(got, want, what=f"config 4 path {path}")
        assert np.all(got[:, :, :140, :] == np.float32(114.0) * np.float32(1.0 / 255.0))


@pytest.mark.parametrize("interp", [0, 1])
def test_config5_4k_to_448_fp16(pkg, oracle, interp):
    """4K -> 512x512 -> centre 448x448, mean/std, float16 NCHW, nearest and linear (2 images per GPU here)."""
    rng = np.random.default_rng(1234)
    src = rng.integers(0, 256, (2, 2160, 3840, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(512, 512), crop=(32, 32), out_size=(448, 448), interp=interp, src_cast=False,
                             base=MEAN, mul=INV_STD)
    want = oracle.resize_crop(list(src), spec, np.float16, True, nthreads=8)
    tsrc = to_dev(src)
    for path in PATHS:
        out = torch.empty((2, 3, 448, 448), dtype=torch.float16, device="cuda")
        with kernel_path(pkg, path):
            pkg.fused_preprocess_into(out, tsrc, resize_dim=(512, 512), interp=interp, crop_pos=(32, 32), layout="NCHW",
                                      base=MEAN, mul=INV_STD, srcCast=False)
            torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, exact=(interp == 0), what=f"config 5 interp {interp} path {path}")


@pytest.mark.parametrize("offset,pad", [(0, 32), (1, 32), (16, 16), (0, 1), (3, 1)])
@pytest.mark.parametrize("interp", [0, 1])
def test_alignment_and_pitch_variants(pkg, oracle, offset, pad, interp):
    """Unaligned base pointers and unpadded odd pitches make the staged kernel read straight from global memory."""
    rng = np.random.default_rng(99 + offset + pad)
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for w, h in ((101, 77), (333, 45), (64, 64))]
    spec = oracle.ResizeSpec(resize=(80, 60), crop=(3, 2), out_size=(70, 50), interp=interp, src_cast=False, manip=1,
                             scale=0.25, offset=-3.0)
    want = oracle.resize_crop(images, spec, np.float32, True)
    batch = pkg.ImageBatchVarShape(padded_images(images, pad_to=pad, offset=offset))
    for path in PATHS:
        with kernel_path(pkg, path):
            out = pkg.resize_crop_convert_reformat(batch, (80, 60), interp, (3, 2, 70, 50), layout="NCHW",
                                                   data_type=torch.float32, manip=1, scale=0.25, offset=-3.0,
                                                   srcCast=False)
            torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, exact=(interp == 0), what=f"offset {offset} pad {pad} path {path}")
    assert pkg.read_device_error() == 0


@pytest.mark.parametrize("case", [
    # (src w, h), resize, crop, out
    ((1, 1), (2, 2), (0, 0), (2, 2)),
    ((2, 1), (5, 3), (1, 0), (4, 3)),
    ((1, 7), (3, 9), (0, 2), (3, 5)),
    ((500, 3), (40, 2), (0, 0), (40, 2)),
    ((4000, 16), (33, 8), (0, 0), (33, 8)),   # 121x horizontal reduction: taps skip whole sectors
    ((16, 4000), (8, 35), (1, 1), (7, 33)),
    ((70, 50), (700, 500), (100, 100), (517, 311)),  # 10x enlargement: consecutive rows share source rows
    ((9000, 8), (3000, 8), (0, 0), (3000, 8)),  # wide rows: the destination row is split into chunks
])
@pytest.mark.parametrize("interp", [0, 1])
def test_shape_edge_cases(pkg, oracle, case, interp):
    (w, h), rs, crop, osz = case
    rng = np.random.default_rng(w * 31 + h)
    src = rng.integers(0, 256, (2, h, w, 3), dtype=np.uint8)
    for dt, planar in ((np.float32, True), (np.uint8, False), (np.uint8, True), (np.float32, False)):
        spec = oracle.ResizeSpec(resize=rs, crop=crop, out_size=osz, interp=interp, src_cast=False, scale=0.5, offset=1.0)
        want = oracle.resize_crop(list(src), spec, dt, planar)
        for path in PATHS:
            with kernel_path(pkg, path):
                out = pkg.resize_crop_convert_reformat(to_dev(src), rs, interp, (*crop, *osz),
                                                       layout="NCHW" if planar else "NHWC", data_type=_torch_dtype(dt),
                                                       scale=0.5, offset=1.0, srcCast=False)
                torch.cuda.synchronize()
            assert_parity(out.cpu().numpy(), want, exact=(interp == 0), what=f"{case} {dt.__name__} path {path}")
    assert pkg.read_device_error() == 0


def test_hwc_rank3_tensors_and_strided_output(pkg, oracle):
    """A single HWC image in, CHW out; and writing into a sub-view of a larger output tensor (true strides)."""
    rng = np.random.default_rng(11)
    src = rng.integers(0, 256, (1, 90, 120, 3), dtype=np.uint8)
    spec = oracle.ResizeSpec(resize=(60, 45), crop=(5, 5), out_size=(48, 36), interp=1, src_cast=True, scale=2.0)
    want = oracle.resize_crop(list(src), spec, np.float32, True)
    out = pkg.resize_crop_convert_reformat(to_dev(src[0]), (60, 45), 1, (5, 5, 48, 36), layout="CHW",
                                           data_type=torch.float32, scale=2.0)
    assert out.shape == (3, 36, 48)
    assert_parity(out.cpu().numpy()[None], want, what="rank-3")
    big = torch.zeros((1, 3, 50, 64), dtype=torch.float32, device="cuda")
    view = big[:, :, 7:43, 8:56]
    pkg.resize_crop_convert_reformat_into(view, to_dev(src), (60, 45), 1, (5, 5), layout="NCHW", scale=2.0)
    torch.cuda.synchronize()
    assert_parity(view.cpu().numpy(), want, what="strided output")
    assert float(big.sum()) == pytest.approx(float(view.sum()))  # nothing written outside the view


def test_empty_batch_is_a_noop(pkg):
    src = torch.empty((0, 32, 32, 3), dtype=torch.uint8, device="cuda")
    before = pkg.launch_count()
    out = pkg.resize_crop_convert_reformat(src, (16, 16), 1, (0, 0, 16, 16), layout="NCHW", data_type=torch.float32)
    assert out.shape == (0, 3, 16, 16) and pkg.launch_count() == before


@pytest.mark.parametrize("idx", range(len(T.RCCR_NEGATIVE_ROWS)))
@pytest.mark.parametrize("varshape", [False, True])
def test_negative_rows_return_the_reference_status(pkg, idx, varshape):
    """The reference's negative tests: same NVCVStatus code for the same bad argument, and nothing is launched."""
    r = T.RCCR_NEGATIVE_ROWS[idx]
    tdt = {"u8": torch.uint8, "f32": torch.float32, "f16": torch.float16}
    if varshape:
        if r.src_planar:
            src = pkg.ImageBatchVarShape([torch.zeros((r.src_channels, 32, 32), dtype=tdt[r.src_dtype], device="cuda")
                                          for _ in range(r.n_in)], planar=True)
        else:
            src = pkg.ImageBatchVarShape([torch.zeros((32, 32, r.src_channels), dtype=tdt[r.src_dtype], device="cuda")
                                          for _ in range(r.n_in)])
    else:
        if r.src_planar:
            pytest.skip("a planar source tensor is expressed by its layout string, which torch tensors do not carry")
        src = torch.zeros((r.n_in, 32, 32, r.src_channels), dtype=tdt[r.src_dtype], device="cuda")
    dst = torch.zeros((r.n_out, r.out[1], r.out[0], r.dst_channels), dtype=tdt[r.dst_dtype], device="cuda")
    before = pkg.launch_count()
    with pytest.raises(pkg.ops.Error) as e:
        pkg.resize_crop_convert_reformat_into(dst, src, r.resize, r.interp, r.crop, layout="NHWC")
    assert pkg.ops.Status(e.value.status).name == r.status, e.value.message
    assert pkg.launch_count() == before


def test_bounded_wait_gives_up_and_reports(pkg, oracle):
    """Failure detection without a fault: a wait nothing satisfies runs out after 20 ms, the kernel returns, the host
    reads the give-up bit, and the context keeps working."""
    import time
    assert pkg.read_device_error() == 0
    t0 = time.perf_counter()
    pkg.self_test_wait_timeout(20)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert 0.015 < elapsed < 1.0
    # the word reaches the host by itself: the next call on this device is refused as an internal error, unasked and
    # without a synchronisation of its own, until the word has been read
    src = np.random.default_rng(1).integers(0, 256, (1, 40, 60, 3), dtype=np.uint8)
    before = pkg.launch_count()
    for _ in range(2):
        with pytest.raises(pkg.ops.Error) as e:
            pkg.resize_crop_convert_reformat(to_dev(src), (48, 32), 1, (0, 0, 48, 32), layout="NCHW", data_type=torch.float32)
        assert e.value.status == pkg.ops.Status.ERROR_INTERNAL and "bounded internal wait" in e.value.message
    assert pkg.launch_count() == before
    assert pkg.read_device_error() == 8
    assert pkg.read_device_error() == 0  # reading clears the word
    spec = oracle.ResizeSpec(resize=(48, 32), out_size=(48, 32), interp=1, src_cast=False)
    out = pkg.resize_crop_convert_reformat(to_dev(src), (48, 32), 1, (0, 0, 48, 32), layout="NCHW", data_type=torch.float32,
                                           srcCast=False)
    assert_parity(out.cpu().numpy(), oracle.resize_crop(list(src), spec, np.float32, True), what="after the self-test")


def test_offsets_beyond_two_gib(pkg, oracle):
    """400 x 1080p is 2.49 GB: the reference refuses it (sample offsets are 32-bit there); here the last sample of the
    batch must come out right."""
    n = 400
    src = torch.zeros((n, 1080, 1920, 3), dtype=torch.uint8, device="cuda")
    rng = np.random.default_rng(9)
    last = rng.integers(0, 256, (1080, 1920, 3), dtype=np.uint8)
    first = rng.integers(0, 256, (1080, 1920, 3), dtype=np.uint8)
    src[n - 1].copy_(to_dev(last))
    src[0].copy_(to_dev(first))
    spec = oracle.ResizeSpec(resize=(256, 256), crop=(16, 16), out_size=(224, 224), interp=1, src_cast=False, manip=1,
                             scale=1.0 / 255.0)
    want = oracle.resize_crop([first, last], spec, np.float32, True, nthreads=2)
    for path in PATHS:
        with kernel_path(pkg, path):
            out = pkg.resize_crop_convert_reformat(src, (256, 256), 1, (16, 16, 224, 224), layout="NCHW",
                                                   data_type=torch.float32, manip=1, scale=1.0 / 255.0, srcCast=False)
            torch.cuda.synchronize()
        got = out[[0, n - 1]].cpu().numpy()
        assert_parity(got, want, what=f"path {path}")
        assert float(out[1:n - 1].abs().max()) == 0.0
    del src


def test_one_handle_many_threads_and_streams(pkg, oracle):
    """Operators hold no mutable state: several host threads, each on its own stream, run different shapes at once."""
    import threading
    rng = np.random.default_rng(21)
    cases = []
    for k in range(4):
        w, h = 200 + 37 * k, 150 + 21 * k
        src = rng.integers(0, 256, (3, h, w, 3), dtype=np.uint8)
        spec = oracle.ResizeSpec(resize=(96 + 8 * k, 80), crop=(k, 2 * k), out_size=(64, 48), interp=k % 2, src_cast=False,
                                 manip=k % 2, scale=0.5, offset=float(k))
        cases.append((src, spec, oracle.resize_crop(list(src), spec, np.float32, True)))
    results, errors = [None] * 4, []

    def work(k):
        try:
            src, spec, _ = cases[k]
            stream = torch.cuda.Stream()
            tsrc = to_dev(src)
            torch.cuda.synchronize()
            with torch.cuda.stream(stream):
                for _ in range(20):
                    out = pkg.resize_crop_convert_reformat(tsrc, spec.resize, spec.interp, (*spec.crop, 64, 48),
                                                           layout="NCHW", data_type=torch.float32, manip=spec.manip,
                                                           scale=0.5, offset=float(k), srcCast=False, stream=stream)
            stream.synchronize()
            results[k] = out.cpu().numpy()
        except Exception as e:  # noqa: BLE001
            errors.append(e)

    threads = [threading.Thread(target=work, args=(k,)) for k in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    for k in range(4):
        assert_parity(results[k], cases[k][2], exact=(cases[k][1].interp == 0), what=f"thread {k}")
    assert pkg.read_device_error() == 0


@pytest.mark.parametrize("interp", [0, 1])
@pytest.mark.parametrize("dtype,planar", [(np.uint8, False), (np.float16, True), (np.float32, False)])
def test_region_placement_roi_and_all_flip_codes(pkg, oracle, interp, dtype, planar):
    """A region placed off both edges of a larger canvas, per-sample regions of interest and every flip code,
    on a variable-shape batch with odd pitches."""
    rng = np.random.default_rng(77 + interp)
    sizes = [(151, 93), (64, 200), (333, 47), (90, 90), (1203, 77)]
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for w, h in sizes]
    rois = np.array([(3, 5, 120, 80), (0, 0, 64, 200), (100, 7, 233, 40), (17, 29, 50, 33), (2, 1, 1200, 70)], np.int32)
    flips = np.array([1, 0, -1, 2, 1], np.int32)
    spec = oracle.ResizeSpec(resize=(66, 44), crop=(4, 3), out_size=(60, 40), interp=interp, src_cast=True, manip=1,
                             base=(1.0, 2.0, 3.0), mul=(0.5, 0.25, 2.0), gscale=1.5, shift=-4.0, canvas=(100, 80),
                             dst_pos=(13, 7), pad_value=114.0)
    want = oracle.resize_crop(images, spec, dtype, planar, roi=rois, flip=flips)
    for pad_to, offset in ((32, 0), (1, 3)):
        batch = pkg.ImageBatchVarShape(padded_images(images, pad_to=pad_to, offset=offset))
        for path in PATHS:
            shape = (5, 3, 80, 100) if planar else (5, 80, 100, 3)
            out = torch.zeros(shape, dtype=_torch_dtype(dtype), device="cuda")
            with kernel_path(pkg, path):
                pkg.fused_preprocess_into(out, batch, resize_dim=(66, 44), interp=interp, crop_pos=(4, 3),
                                          layout="NCHW" if planar else "NHWC", manip=1, base=(1.0, 2.0, 3.0),
                                          mul=(0.5, 0.25, 2.0), gscale=1.5, shift=-4.0, srcCast=True, roi=to_dev(rois),
                                          flip_code=to_dev(flips), dst_pos=(13, 7), region_size=(60, 40), pad_value=114.0)
                torch.cuda.synchronize()
            assert_parity(out.cpu().numpy(), want, exact=(interp == 0), what=f"pad {pad_to} path {path}")
    assert pkg.read_device_error() == 0


def test_wide_rows_in_chunks_with_horizontal_flip(pkg, oracle):
    """Rows whose source span exceeds a shared-memory slot are processed in column chunks; mirrored columns walk the
    chunks from the other end."""
    rng = np.random.default_rng(5)
    src = rng.integers(0, 256, (2, 6, 20000, 3), dtype=np.uint8)
    flips = np.array([1, -1], np.int32)
    spec = oracle.ResizeSpec(resize=(5000, 6), crop=(10, 0), out_size=(4980, 6), interp=1, src_cast=False, scale=0.5)
    want = oracle.resize_crop(list(src), spec, np.float32, True, flip=flips, nthreads=4)
    for path in PATHS:
        out = torch.empty((2, 3, 6, 4980), dtype=torch.float32, device="cuda")
        with kernel_path(pkg, path):
            pkg.fused_preprocess_into(out, to_dev(src), resize_dim=(5000, 6), interp=1, crop_pos=(10, 0), layout="NCHW",
                                      scale=0.5, srcCast=False, flip_code=to_dev(flips))
            torch.cuda.synchronize()
        assert_parity(out.cpu().numpy(), want, what=f"path {path}")


@pytest.mark.parametrize("factor", [(1, 1), (2, 2), (3, 1), (1, 4), (5, 3)])
def test_integer_reduction_factors(pkg, oracle, factor):
    """Whole-number scale factors put every sample point on a pixel centre or exactly between two (weights 0 or 0.5);
    taps of weight zero are skipped by the kernels and must not change a bit."""
    fx, fy = factor
    ow, oh = 96, 40
    rng = np.random.default_rng(fx * 10 + fy)
    src = rng.integers(0, 256, (2, oh * fy, ow * fx, 3), dtype=np.uint8)
    for dtype, planar, cast in ((np.float32, True, False), (np.uint8, False, True), (np.float16, True, True)):
        spec = oracle.ResizeSpec(resize=(ow, oh), crop=(3, 2), out_size=(ow - 5, oh - 4), interp=1, src_cast=cast,
                                 manip=1, scale=0.75, offset=-1.5)
        want = oracle.resize_crop(list(src), spec, dtype, planar)
        for path in PATHS:
            shape = (2, 3, oh - 4, ow - 5) if planar else (2, oh - 4, ow - 5, 3)
            out = torch.empty(shape, dtype=_torch_dtype(dtype), device="cuda")
            with kernel_path(pkg, path):
                pkg.fused_preprocess_into(out, to_dev(src), resize_dim=(ow, oh), interp=1, crop_pos=(3, 2),
                                          layout="NCHW" if planar else "NHWC", manip=1, scale=0.75, offset=-1.5,
                                          srcCast=cast)
                torch.cuda.synchronize()
            got = out.cpu().numpy()
            assert_parity(got, want, what=f"factor {factor} {np.dtype(dtype).name} path {path}")
            assert np.array_equal(got.view(np.uint8), want.view(np.uint8))
