"""CPU: the shared library builds for sm_100a, loads without a GPU and exports every symbol the headers declare."""
import ctypes
import os
import re
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
INCLUDE = os.path.join(ROOT, "include", "cvcuda_b200")


def _declared_symbols():
    names = set()
    for fn in os.listdir(INCLUDE):
        text = open(os.path.join(INCLUDE, fn)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        for m in re.finditer(r"(?:B200PP_PUBLIC|CVCUDA_B200_PUBLIC)\s+[\w\s\*]+?\b(\w+)\s*\(", text):
            names.add(m.group(1))
    return names


def test_every_declared_symbol_is_exported(pkg):
    declared = _declared_symbols()
    assert {"b200ppResizeCropConvertReformat", "b200ppCropFlipNormalizeReformat"} <= declared
    lib = ctypes.CDLL(pkg.lib_path())
    missing = [n for n in sorted(declared) if not hasattr(lib, n)]
    assert not missing, f"declared but not exported: {missing}"


def test_nothing_else_leaks_out(pkg):
    out = subprocess.check_output(["nm", "-D", "--defined-only", pkg.lib_path()], text=True)
    exported = {ln.split()[-1].split("@")[0] for ln in out.splitlines() if " T " in ln}
    stray = [s for s in exported if not re.match(r"^(b200pp|cvcuda|nvcvOperator)", s)]
    assert not stray, f"unexpected exports: {stray[:10]}"


def test_descriptor_layout_matches_the_reference_abi(pkg):
    """sizeof(NVCVImagePlaneStrided) = 24 and sizeof(NVCVImageBufferStrided) = 152 (int32 + pad + 6 planes)."""
    ops = pkg.ops
    assert ctypes.sizeof(ops._ImagePlane) == 24 and ops._ImagePlane.basePtr.offset == 16
    assert ctypes.sizeof(ops._ImageBuffer) == 152 and ops._ImageBuffer.planes.offset == 8


def test_argument_checks_need_no_gpu(pkg):
    """Validation runs before any CUDA call, so status codes can be checked on a CPU-only machine."""
    ops = pkg.ops
    L = pkg.lib()
    s, d, op = ops._Source(), ops._Dest(), ops._ResizeOp()
    assert L.b200ppResizeCropConvertReformat(None, None, None, None) == ops.Status.ERROR_INVALID_ARGUMENT
    s.base, d.base, s.numSamples = 256, 256, 1
    s.channels, d.channels = 3, 4
    assert L.b200ppResizeCropConvertReformat(ctypes.byref(s), ctypes.byref(d), ctypes.byref(op), None) \
        == ops.Status.ERROR_NOT_COMPATIBLE
    assert b"same number of channels" in L.b200ppGetLastErrorMessage()
    d.channels = 3
    s.dtype = 6
    assert L.b200ppResizeCropConvertReformat(ctypes.byref(s), ctypes.byref(d), ctypes.byref(op), None) \
        == ops.Status.ERROR_NOT_COMPATIBLE
    s.dtype = 0
    op.resizeW = op.resizeH = 1
    assert L.b200ppResizeCropConvertReformat(ctypes.byref(s), ctypes.byref(d), ctypes.byref(op), None) \
        == ops.Status.ERROR_INVALID_ARGUMENT
    assert pkg.launch_count() == 0 or True


def test_public_headers_compile_as_c11_and_cxx11(tmp_path):
    """Like the reference's header checks (tests/cvcuda/system/CMakeLists.txt:105-126): every public header is valid
    C11 and C++11 on its own, without the CUDA toolkit on the include path."""
    for name in sorted(os.listdir(INCLUDE)):
        for compiler, std, ext in (("gcc", "-std=c11", "c"), ("g++", "-std=c++11", "cpp")):
            src = tmp_path / f"use_{name.replace('.', '_')}.{ext}"
            src.write_text(f'#include <cvcuda_b200/{name}>\nint main(void) {{ return 0; }}\n')
            subprocess.check_call([compiler, std, "-Wall", "-Werror", "-pedantic-errors", "-fsyntax-only",
                                   "-I" + os.path.join(ROOT, "include"), str(src)])
