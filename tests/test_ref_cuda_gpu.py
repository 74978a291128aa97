"""GPU cross-check against the reference project's OWN CUDA kernels (compiled for sm_100a into oracle/_ref by
oracle/build_oracle.py), at the reference tests' own tolerances: +-1 for ResizeCropConvertReformat
(TestOpResizeCropConvertReformat.cpp:437,564), 1e-4 for CropFlipNormalizeReformat (TestOpCropFlipNormalizeReformat.cpp:405).
The reference kernels contract a*b+c into FMAs and blend in a different order than their CPU golden, so they are close
to, not equal to, the golden; the new kernels equal the golden."""
import numpy as np
import pytest
import torch

import ref_tables as T
from gpu_util import padded_images, to_dev

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def refcuda(built):
    from oracle import ref_cuda
    if ref_cuda.lib() is None:
        pytest.skip("reference CUDA kernels were not built (reference tree absent at build time)")
    return ref_cuda


TORCH = {np.uint8: torch.uint8, np.float32: torch.float32}


@pytest.mark.parametrize("idx", [0, 5, 7, 9, 11, 24, 31, 41, 45, 52, 54, 55, 57, 58, 60, 61])
def test_rccr_tensor_against_reference_kernels(pkg, refcuda, idx):
    r = T.RCCR_ROWS[idx]
    w, h, n = r.src
    n = min(n, 3)
    src = to_dev(np.random.default_rng(idx).integers(0, 256, (n, h, w, 3), dtype=np.uint8))
    shape = (n, 3, r.out[1], r.out[0]) if r.planar else (n, r.out[1], r.out[0], 3)
    ref = torch.empty(shape, dtype=TORCH[r.dtype], device="cuda")
    refcuda.rccr_tensor(src, ref, r.planar, r.resize, r.interp, r.crop, r.manip, float(np.float32(r.scale)),
                        float(np.float32(r.offset)), r.src_cast)
    out = pkg.resize_crop_convert_reformat(src, r.resize, r.interp, (*r.crop, *r.out),
                                           layout="NCHW" if r.planar else "NHWC", data_type=TORCH[r.dtype],
                                           manip=r.manip, scale=r.scale, offset=r.offset, srcCast=r.src_cast)
    torch.cuda.synchronize()
    diff = (out.double() - ref.double()).abs().max().item()
    assert diff <= 1.0, f"row {idx}: max |new - reference kernel| = {diff}"


@pytest.mark.parametrize("idx", [3, 9, 31, 44, 57])
def test_rccr_varshape_against_reference_kernels(pkg, refcuda, idx):
    r = T.RCCR_ROWS[idx]
    w, h, _ = r.src
    rng = np.random.default_rng(100 + idx)
    images = [rng.integers(0, 256, (int(h * s), int(w * s), 3), dtype=np.uint8) for s in (0.8, 1.0, 1.2)]
    batch = pkg.ImageBatchVarShape(padded_images(images))
    shape = (3, 3, r.out[1], r.out[0]) if r.planar else (3, r.out[1], r.out[0], 3)
    ref = torch.empty(shape, dtype=TORCH[r.dtype], device="cuda")
    refcuda.rccr_varshape(batch.descriptor_table(), 3, ref, r.planar, r.resize, r.interp, r.crop, r.manip,
                          float(np.float32(r.scale)), float(np.float32(r.offset)), r.src_cast)
    out = pkg.resize_crop_convert_reformat(batch, r.resize, r.interp, (*r.crop, *r.out),
                                           layout="NCHW" if r.planar else "NHWC", data_type=TORCH[r.dtype],
                                           manip=r.manip, scale=r.scale, offset=r.offset, srcCast=r.src_cast)
    torch.cuda.synchronize()
    diff = (out.double() - ref.double()).abs().max().item()
    assert diff <= 1.0, f"row {idx}: max |new - reference kernel| = {diff}"


@pytest.mark.parametrize("border", range(5))
@pytest.mark.parametrize("planar,dtype", [(True, np.float32), (False, np.uint8)])
def test_cfnr_against_reference_kernel(pkg, refcuda, border, planar, dtype):
    rng = np.random.default_rng(border)
    images = [rng.integers(0, 256, (h, w, 3), dtype=np.uint8) for w, h in ((51, 53), (40, 61), (77, 35))]
    rects = np.array([(-3, 2, 45, 50), (4, -2, 36, 58), (0, 0, 77, 35)], np.int32)
    flips = np.array([1, -1, 0], np.int32)
    base = rng.uniform(0, 255, 3).astype(np.float32)
    scale = rng.uniform(0.1, 1, 3).astype(np.float32)
    batch = pkg.ImageBatchVarShape(padded_images(images))
    ow, oh = 80, 64
    shape = (3, 3, oh, ow) if planar else (3, oh, ow, 3)
    ref = torch.zeros(shape, dtype=TORCH[dtype], device="cuda")
    trect, tflip = to_dev(rects.reshape(3, 1, 1, 4)), to_dev(flips)
    tbase, tscale = to_dev(base.reshape(1, 1, 1, 3)), to_dev(scale.reshape(1, 1, 1, 3))
    refcuda.cfnr_u8(batch.descriptor_table(), 3, 3, ref, planar, trect, tflip, tbase, tscale, border, 1.0, 1.1, 0.3, 0.0, 0)
    out = pkg.crop_flip_normalize_reformat(batch, shape, TORCH[dtype], "NCHW" if planar else "NHWC", trect, tflip, tbase,
                                           tscale, 1.1, 0.3, 0.0, 0, border, 1.0)
    torch.cuda.synchronize()
    diff = (out.double() - ref.double()).abs().max().item()
    assert diff <= (1e-4 if dtype == np.float32 else 1.0), f"max |new - reference kernel| = {diff}"
