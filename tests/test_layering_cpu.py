"""CPU: the product never reaches into the test infrastructure, and refuses to run without its CUDA library."""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "cv-cuda_b200")


def _sources():
    for base, _, files in os.walk(PKG):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                yield os.path.join(base, f)
    for f in os.listdir(os.path.join(ROOT, "include", "cvcuda_b200")):
        yield os.path.join(ROOT, "include", "cvcuda_b200", f)


def test_package_never_touches_the_oracle_or_work_files():
    pat = re.compile(r"(from\s+oracle|import\s+oracle|oracle/|liboracle|libref_golden|_work/)")
    hits = [p for p in _sources() if pat.search(open(p, encoding="utf-8").read())]
    assert not hits, hits


def test_missing_library_is_a_loud_failure(pkg, monkeypatch):
    ops = pkg.ops
    monkeypatch.setattr(ops, "_lib", None)
    monkeypatch.setattr(ops, "_LIB_NAME", "libcvcuda_b200_missing.so")
    try:
        ops.lib()
    except RuntimeError as e:
        assert "no CPU or PyTorch fallback" in str(e)
    else:
        raise AssertionError("loading a missing library must raise")
    finally:
        monkeypatch.undo()
    assert ops.lib() is not None
