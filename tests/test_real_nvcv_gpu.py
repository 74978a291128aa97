"""The drop-in boundary with the reference's real object model on the other side.

oracle/build_oracle.py compiles the reference's libnvcv_types and its own operators from the reference tree; a harness
written against the reference's header-only C++ API (oracle/ref_ops_harness.cpp: nvcv::Tensor, nvcv::Image,
nvcv::ImageBatchVarShape, cvcuda::ResizeCropConvertReformat, cvcuda::CropFlipNormalizeReformat) is linked once against the
B200 library and once against those reference operators. Each runs in a child process (tests/real_nvcv_worker.py) and
compares with the CPU oracle: rows of the reference's tables as real tensors and real image batches -- including images
pushed after a first call, so that ImageBatchVarShape::exportData uploads descriptors again on the call's stream
(src/nvcv/src/priv/ImageBatchVarShape.cpp:215-254) -- all 18 CropFlipNormalizeReformat rows, and status codes as the
wrappers throw them. The libraries travel prebuilt; without them the tests skip.
"""
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
_cache = {}


def _results(which, built):
    if which not in _cache:
        from oracle import ref_ops
        if not os.path.exists(ref_ops.path(which)):
            _cache[which] = None
        else:
            p = subprocess.run([sys.executable, os.path.join(HERE, "real_nvcv_worker.py"), which], capture_output=True, text=True,
                               timeout=600)
            line = next((ln for ln in p.stdout.splitlines() if ln.startswith("RESULTS ")), None)
            assert p.returncode == 0 and line, f"worker failed ({p.returncode}):\n{p.stdout[-2000:]}\n{p.stderr[-4000:]}"
            _cache[which] = json.loads(line[len("RESULTS "):])
    return _cache[which]


@pytest.mark.parametrize("which", ["b200", "ref"])
def test_reference_cxx_api_over_real_nvcv_objects(built, which):
    """which = b200: the reference's wrappers and real handles drive the B200 library (bit-equal to the oracle);
    which = ref: the same harness drives the reference's own sm_100a operators (within their own tests' bounds), which
    validates the harness and the oracle against the reference's CUDA code."""
    res = _results(which, built)
    if res is None:
        pytest.skip("the reference's libraries were not built on the machine this tree came from")
    assert len(res) == 10 + 5 + 18 + 1
    bad = {k: v for k, v in res.items() if v != "ok"}
    assert not bad, "\n".join(f"{k}: {v}" for k, v in bad.items())
