"""Calls of the library can be captured into a CUDA graph and replayed: they only enqueue work on the caller's stream.

One un-captured call per device comes first (it sets function attributes and makes the page-locked error word). The replayed
results must equal the eager ones bit for bit, for a dense batch (staged kernel), an image list with rectangles and flips
(row-walk kernel) and CropFlipNormalizeReformat.
"""
import numpy as np
import pytest
import torch

from gpu_util import to_dev

pytestmark = pytest.mark.gpu

MEAN, MUL = (123.675, 116.28, 103.53), (0.017, 0.0175, 0.0174)


def test_calls_replay_from_a_cuda_graph(pkg):
    rng = np.random.default_rng(11)
    dense = to_dev(rng.integers(0, 256, (3, 90, 160, 3), dtype=np.uint8))
    images = [to_dev(rng.integers(0, 256, (h, w, 3), dtype=np.uint8)) for (w, h) in ((120, 80), (64, 96), (200, 50))]
    batch = pkg.ImageBatchVarShape(images)
    roi = to_dev(np.array([[4, 4, 100, 60], [0, 0, 64, 96], [10, 5, 150, 40]], np.int32))
    flips = to_dev(np.array([1, 2, 1], np.int32))
    rects = to_dev(np.array([[0, 0, 48, 40]] * 3, np.int32).reshape(3, 1, 1, 4))
    base = to_dev(np.array(MEAN, np.float32).reshape(1, 1, 1, 3))
    scale = to_dev(np.array(MUL, np.float32).reshape(1, 1, 1, 3))

    outs = [torch.zeros((3, 3, 48, 64), dtype=torch.float32, device="cuda"),
            torch.zeros((3, 3, 48, 64), dtype=torch.float16, device="cuda"),
            torch.zeros((3, 3, 40, 48), dtype=torch.float32, device="cuda")]

    def calls():
        pkg.fused_preprocess_into(outs[0], dense, resize_dim=(72, 56), interp=1, crop_pos=(4, 4), layout="NCHW", base=MEAN, mul=MUL,
                                  srcCast=False)
        pkg.fused_preprocess_into(outs[1], batch, resize_dim=(64, 48), interp=1, layout="NCHW", base=MEAN, mul=MUL, srcCast=True,
                                  roi=roi, flip_code=flips)
        pkg.crop_flip_normalize_reformat_into(outs[2], batch, rects, flips, base, scale, 1.0, 0.0, 0.0, 0, pkg.Border.REFLECT101, 0.0,
                                              layout="NCHW")

    calls()  # the first call on a device is not capturable
    torch.cuda.synchronize()
    want = [o.clone() for o in outs]
    for o in outs:
        o.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        calls()
    torch.cuda.synchronize()
    assert all(float(o.abs().max()) == 0.0 for o in outs), "capture must not run the kernels"
    graph.replay()
    torch.cuda.synchronize()
    for got, exp in zip(outs, want):
        assert torch.equal(got, exp)
    assert pkg.read_device_error() == 0
