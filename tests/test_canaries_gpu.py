"""Guard bands around every destination: no kernel may write a byte that is not an element of its output.

Each destination is a strided view inside a buffer filled with a pattern: 256 bytes before and after, padding between the
rows (odd pitches), between the planes and between the samples, and a base address off every vector alignment. After the
call the bytes of the view are blanked with the pattern on the host and the whole buffer must equal the pattern again. The
kernels that write with vectors (quads of the resize kernels, 16-byte groups of CopyMakeBorder and Reformat, the table
kernels of Normalize and ConvertTo, the four-pixel threads of CropFlipNormalizeReformat) are run at every width from 1 to
40, where the ragged end of a row is where an overrun would hide. This is the stand-in for a memory checker.
"""
import numpy as np
import pytest
import torch

from gpu_util import _TORCH_DTYPE, kernel_path, to_dev

pytestmark = pytest.mark.gpu

PATTERN = 0xA5
BAND = 256
WIDTHS = list(range(1, 41))


class Guarded:
    """A destination tensor of `shape` (elements of `dtype`) whose dimension i is `pads[i]` ELEMENTS further apart than
    packed, inside a pattern-filled buffer, starting `offset` elements after the leading band."""

    def __init__(self, shape, dtype, pads, offset=1):
        self.np_dtype = np.dtype(dtype)
        es = self.np_dtype.itemsize
        # innermost stride 1; the stride of dimension i = extent * stride of dimension i + 1, plus pads[i]
        strides = [1] * len(shape)
        for i in range(len(shape) - 2, -1, -1):
            strides[i] = shape[i + 1] * strides[i + 1] + pads[i]
        s = shape[0] * strides[0]
        self.shape, self.strides, self.offset_bytes = tuple(shape), tuple(strides), BAND + offset * es
        total = self.offset_bytes + s * es + BAND
        self.buf = torch.full((total,), PATTERN, dtype=torch.uint8, device="cuda")
        typed = self.buf[self.offset_bytes:self.offset_bytes + (s * es)].view(_TORCH_DTYPE[self.np_dtype])
        self.view = torch.as_strided(typed, self.shape, self.strides)

    def check(self, what):
        host = self.buf.cpu().numpy().copy()
        es = self.np_dtype.itemsize
        inside = np.lib.stride_tricks.as_strided(host[self.offset_bytes:], shape=self.shape + (es,),
                                                 strides=tuple(st * es for st in self.strides) + (1,), writeable=True)
        inside[...] = PATTERN
        bad = np.flatnonzero(host != PATTERN)
        assert bad.size == 0, f"{what}: {bad.size} bytes written outside the destination, first at {int(bad[0]) - self.offset_bytes}"


def _nhwc(n, h, w, c, dtype, offset=1):
    return Guarded((n, h, w, c), dtype, pads=(7, 5, 0, 0), offset=offset)  # row pitch + 5 elements, sample + 7


def _nchw(n, c, h, w, dtype, offset=1):
    return Guarded((n, c, h, w), dtype, pads=(11, 9, 3, 0), offset=offset)  # row + 3, plane + 9, sample + 11


MEAN, MUL = (123.675, 116.28, 103.53), (0.017, 0.0175, 0.0174)


@pytest.mark.parametrize("dtype", [np.uint8, np.float32, np.float16], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("planar", [False, True], ids=["nhwc", "nchw"])
def test_fused_resize_writes_only_its_output(pkg, dtype, planar):
    rng = np.random.default_rng(1)
    src = to_dev(rng.integers(0, 256, (2, 23, 97, 3), dtype=np.uint8))
    for w in WIDTHS:
        for path in (1, 2, 3):
            for interp in (0, 1):
                g = _nchw(2, 3, 5, w, dtype) if planar else _nhwc(2, 5, w, 3, dtype)
                with kernel_path(pkg, path):
                    pkg.fused_preprocess_into(g.view, src, resize_dim=(w + 3, 8), interp=interp, crop_pos=(2, 1),
                                              layout="NCHW" if planar else "NHWC", base=MEAN, mul=MUL, srcCast=False)
                torch.cuda.synchronize()
                g.check(f"width {w} path {path} interp {interp}")
    # letterbox: the padded rows and columns are written by the same vector stores
    for w in (5, 17, 33, 40):
        g = _nchw(2, 3, 12, w + 6, dtype) if planar else _nhwc(2, 12, w + 6, 3, dtype)
        for path in (1, 2, 3):
            with kernel_path(pkg, path):
                pkg.fused_preprocess_into(g.view, src, resize_dim=(w, 6), interp=1, layout="NCHW" if planar else "NHWC",
                                          scale=1 / 255.0, dst_pos=(3, 4), region_size=(w, 6), pad_value=114.0)
            torch.cuda.synchronize()
            g.check(f"letterbox width {w} path {path}")
    assert pkg.read_device_error() == 0


@pytest.mark.parametrize("dtype", [np.uint8, np.float32], ids=lambda d: np.dtype(d).name)
@pytest.mark.parametrize("planar", [False, True], ids=["nhwc", "nchw"])
def test_crop_flip_normalize_writes_only_its_output(pkg, dtype, planar):
    rng = np.random.default_rng(2)
    base = to_dev(np.array(MEAN, np.float32).reshape(1, 1, 1, 3))
    scale = to_dev(np.array(MUL, np.float32).reshape(1, 1, 1, 3))
    for ch in (3, 1):
        images = [to_dev(rng.integers(0, 256, (h, wd, ch), dtype=np.uint8)) for (wd, h) in ((50, 9), (44, 11))]
        batch = pkg.ImageBatchVarShape(images)
        for w in WIDTHS:
            rects = to_dev(np.array([[1, 1, w, 6], [-2, 0, max(1, w - 1), 7]], np.int32).reshape(2, 1, 1, 4))
            flips = to_dev(np.array([1, -1], np.int32))
            g = _nchw(2, ch, 7, w, dtype) if planar else _nhwc(2, 7, w, ch, dtype)
            for path in (0, 1):
                with kernel_path(pkg, path):
                    pkg.crop_flip_normalize_reformat_into(g.view, batch, rects, flips, base[..., :ch], scale[..., :ch], 1.0, 0.0, 0.0,
                                                          0, pkg.Border.REFLECT101, 0.0, layout="NCHW" if planar else "NHWC")
                torch.cuda.synchronize()
                g.check(f"channels {ch} width {w} path {path}")


@pytest.mark.parametrize("dtype,ch", [(np.uint8, 1), (np.uint8, 3), (np.uint8, 4), (np.int16, 3), (np.float32, 4), (np.float32, 3),
                                      (np.float32, 1)],
                         ids=lambda v: str(np.dtype(v).name) if not isinstance(v, int) else str(v))
def test_standalone_operators_write_only_their_output(pkg, dtype, ch):
    rng = np.random.default_rng(3)
    info = None if dtype == np.float32 else np.iinfo(dtype)

    def data(shape):
        if info is None:
            return rng.uniform(0, 255, shape).astype(np.float32)
        return rng.integers(info.min, info.max + 1, shape).astype(dtype)

    src = to_dev(data((2, 9, 61, ch)))
    for w in WIDTHS:
        for interp in (0, 1):  # Resize
            g = _nhwc(2, 6, w, ch, dtype)
            pkg.resize_into(g.view, src, interp)
            torch.cuda.synchronize()
            g.check(f"resize width {w} interp {interp}")
        same = to_dev(data((2, 6, w, ch)))
        # Normalize (uint8 sources take the table kernel unless path 1 forces the arithmetic one), to the same type and to float32
        if True:
            b = to_dev(rng.uniform(0, 100, (1, 1, 1, ch)).astype(np.float32))
            s = to_dev(rng.uniform(0.5, 1.5, (1, 1, 1, ch)).astype(np.float32))
            for out_dt in ((dtype, np.float32) if dtype != np.float32 else (np.float32,)):  # float32 -> float32: the vector kernel
                for path in (0, 1):
                    g = _nhwc(2, 6, w, ch, out_dt)
                    with kernel_path(pkg, path):
                        pkg.normalize_into(g.view, same, b, s)
                    torch.cuda.synchronize()
                    g.check(f"normalize width {w} -> {np.dtype(out_dt).name} path {path}")
        # ConvertTo in both directions (table kernel for 8-bit sources, vector kernel for float32 sources)
        for out_dt in (np.float32, np.uint8):
            for path in (0, 1):
                g = _nhwc(2, 6, w, ch, out_dt)
                with kernel_path(pkg, path):
                    pkg.convertto_into(g.view, same, 0.5, 1.0)
                torch.cuda.synchronize()
                g.check(f"convertto width {w} -> {np.dtype(out_dt).name} path {path}")
        # CopyMakeBorder: every rule; the 16-byte groups straddle the image's edges
        for border in range(5):
            g = _nhwc(2, 6 + 3, w + 5, ch, dtype)
            pkg.copymakeborder_into(g.view, same, border, (1.0, 2.0, 3.0, 4.0), top=2, left=3)
            torch.cuda.synchronize()
            g.check(f"copymakeborder width {w} border {border}")
        # Reformat, both directions, both kernels (3-channel uint8 / 32-bit data have vector kernels)
        if ch == 3 or dtype == np.float32:
            for path in (0, 1):
                g = _nchw(2, ch, 6, w, dtype)
                with kernel_path(pkg, path):
                    pkg.reformat_into(g.view, same, src_layout="NHWC", dst_layout="NCHW")
                torch.cuda.synchronize()
                g.check(f"reformat to planar width {w} path {path}")
                planar_src = to_dev(data((2, ch, 6, w)))
                g = _nhwc(2, 6, w, ch, dtype)
                with kernel_path(pkg, path):
                    pkg.reformat_into(g.view, planar_src, src_layout="NCHW", dst_layout="NHWC")
                torch.cuda.synchronize()
                g.check(f"reformat to interleaved width {w} path {path}")


def test_guard_helper_sees_a_stray_write():
    g = _nhwc(1, 2, 3, 3, np.uint8)
    g.check("untouched")
    g.view.fill_(7)
    g.check("filled through the view")
    g.buf[g.offset_bytes + 3 * 3] = 0  # the first padding byte after row 0
    with pytest.raises(AssertionError):
        g.check("stray")
