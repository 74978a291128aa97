"""Build recipe for the CPU checkers (TEST INFRASTRUCTURE ONLY).

Two artefacts, neither of which the product library links, loads or calls:

* ``oracle/liboracle.so``            -- the C restatement in ``preproc_oracle.c`` (gcc, no dependencies).
* ``oracle/_ref/libref_golden.so``   -- the reference project's own CPU golden functions, compiled from the
  reference tree where it lies (only when that tree is present). The two golden function templates sit inside
  gtest translation units, so they are cut out by signature into a scratch directory, compiled together with
  ``ref_golden_wrap.cpp`` and the reference's header-only host helpers, and the scratch copy is removed again.
  The reference's own build system is not run.

Usage: ``python oracle/build_oracle.py [--ref-root DIR] [--force]``
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SRC = os.path.join(HERE, "preproc_oracle.c")
ORACLE_RESIZE_SRC = os.path.join(HERE, "resize_oracle.c")
ORACLE_NORMALIZE_SRC = os.path.join(HERE, "normalize_oracle.c")
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "libref_golden.so")
REF_WRAP = os.path.join(HERE, "ref_golden_wrap.cpp")
DEFAULT_REF_ROOT = os.environ.get("CVCUDA_REFERENCE_ROOT", "/root/reference")

# -ffp-contract=off: the goldens are defined by un-fused float32 arithmetic in source order.
CFLAGS = ["-O2", "-fPIC", "-shared", "-ffp-contract=off", "-fno-fast-math", "-pthread"]


def _stale(target: str, *sources: str) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(s) > t for s in sources if os.path.exists(s))


def build_oracle(force: bool = False) -> str:
    if force or _stale(ORACLE_SO, ORACLE_SRC, ORACLE_RESIZE_SRC, ORACLE_NORMALIZE_SRC, os.path.join(HERE, "preproc_oracle.h"),
                       os.path.join(HERE, "resize_oracle.h")):
        cmd = ["gcc", "-std=c11", *CFLAGS, "-o", ORACLE_SO, ORACLE_SRC, ORACLE_RESIZE_SRC, ORACLE_NORMALIZE_SRC, "-lm"]
        subprocess.check_call(cmd)
    return ORACLE_SO


def _cut_function(path: str, marker: str, start_at_template: bool = True) -> str:
    """Return the text of the top-level function (template) whose signature contains `marker`: from the
    `template<...>` line above it (or from the marker's own line) to the first line that is exactly '}'."""
    with open(path, "r", encoding="utf-8") as f:
        lines = f.read().split("\n")
    hit = next(i for i, ln in enumerate(lines) if marker in ln)
    start = hit
    while start_at_template and not lines[start].lstrip().startswith("template<"):
        start -= 1
    end = next(i for i in range(hit, len(lines)) if lines[i] == "}")
    return "\n".join(lines[start : end + 1]) + "\n"


def build_ref(ref_root: str = DEFAULT_REF_ROOT, force: bool = False) -> str | None:
    """Compile the reference's golden functions into oracle/_ref/. Returns None when the tree is absent."""
    rccr_tu = os.path.join(ref_root, "tests/cvcuda/system/TestOpResizeCropConvertReformat.cpp")
    cfnr_tu = os.path.join(ref_root, "tests/cvcuda/system/TestOpCropFlipNormalizeReformat.cpp")
    resize_tu = os.path.join(ref_root, "tests/cvcuda/system/ResizeUtils.cpp")
    norm_tu = os.path.join(ref_root, "tests/cvcuda/system/TestOpNormalize.cpp")
    border_tu = os.path.join(ref_root, "tests/cvcuda/system/TestOpCopyMakeBorder.cpp")
    crop_tu = os.path.join(ref_root, "tests/cvcuda/system/TestOpRandomResizedCrop.cpp")
    if not all(os.path.exists(f) for f in (rccr_tu, cfnr_tu, resize_tu, norm_tu, border_tu, crop_tu)):
        return REF_SO if os.path.exists(REF_SO) else None
    if not (force or _stale(REF_SO, REF_WRAP, rccr_tu, cfnr_tu, resize_tu, norm_tu, border_tu, crop_tu)):
        return REF_SO
    os.makedirs(REF_DIR, exist_ok=True)
    scratch = tempfile.mkdtemp(prefix="refgold_")
    try:
        with open(os.path.join(scratch, "rccr.inc"), "w") as f:
            f.write(_cut_function(rccr_tu, "void ResizeCropConvert(      DstT *dst,"))
        with open(os.path.join(scratch, "cfnr.inc"), "w") as f:
            f.write(_cut_function(cfnr_tu, "static void CropFlipNormalizeReformat("))
        with open(os.path.join(scratch, "resize.inc"), "w") as f:
            f.write(_cut_function(resize_tu, "void resizedCrop(T *dstPtr"))
        with open(os.path.join(scratch, "normalize.inc"), "w") as f:
            f.write(_cut_function(norm_tu, "static void Normalize(std::vector<uint8_t> &hDst", start_at_template=False))
        with open(os.path.join(scratch, "border.inc"), "w") as f:
            f.write(_cut_function(border_tu, "static void CopyMakeBorder(std::vector<T> &hDst, const std::vector<T> &hSrc,"))
        with open(os.path.join(scratch, "random_crop.inc"), "w") as f:
            f.write(_cut_function(crop_tu, "static void GetCropParams(std::mt19937 &generator", start_at_template=False))
        inc = [
            "-I" + os.path.join(ref_root, "tests"),
            "-I" + os.path.join(ref_root, "src/cvcuda/include"),
            "-I" + os.path.join(ref_root, "src/nvcv/src/include"),
            "-I/usr/local/cuda/include",
            "-I" + scratch,
        ]
        cmd = [
            "g++", "-std=c++17", *CFLAGS, "-w",
            '-DREF_GOLDEN_RCCR_INC="rccr.inc"', '-DREF_GOLDEN_CFNR_INC="cfnr.inc"', '-DREF_GOLDEN_RESIZE_INC="resize.inc"',
            '-DREF_GOLDEN_NORMALIZE_INC="normalize.inc"', '-DREF_GOLDEN_BORDER_INC="border.inc"', '-DREF_GOLDEN_RANDOM_CROP_INC="random_crop.inc"',
            *inc, "-o", REF_SO, REF_WRAP,
        ]
        subprocess.check_call(cmd)
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return REF_SO


REF_CUDA_SO = os.path.join(REF_DIR, "libref_cuda_kernels.so")
REF_CUDA_WRAP = os.path.join(HERE, "ref_cuda_wrap.cu")


def _cut_between(path: str, first_marker: str, last_marker: str, start_at_template: bool = True) -> str:
    """Lines from the `template<...>` line above the first line containing `first_marker` to the line that closes the
    definition containing `last_marker` (the first line starting with '}' after it)."""
    with open(path, "r", encoding="utf-8") as f:
        lines = f.read().split("\n")
    first = next(i for i, ln in enumerate(lines) if first_marker in ln)
    start = first
    if start_at_template:
        while not lines[start].lstrip().startswith("template"):
            start -= 1
    last = next(i for i, ln in enumerate(lines) if last_marker in ln)
    end = next(i for i in range(last, len(lines)) if lines[i].startswith("}"))
    return "\n".join(lines[start : end + 1]) + "\n"


def build_ref_cuda(ref_root: str = DEFAULT_REF_ROOT, force: bool = False) -> str | None:
    """Compile the reference's own CUDA kernels of the path for sm_100a into oracle/_ref/ (baseline and cross-check).
    Returns None when the reference tree is absent and no earlier build exists."""
    rccr = os.path.join(ref_root, "src/cvcuda/priv/OpResizeCropConvertReformat.cu")
    cfnr = os.path.join(ref_root, "src/cvcuda/priv/OpCropFlipNormalizeReformat.cu")
    if not (os.path.exists(rccr) and os.path.exists(cfnr)):
        return REF_CUDA_SO if os.path.exists(REF_CUDA_SO) else None
    if not (force or _stale(REF_CUDA_SO, REF_CUDA_WRAP, rccr, cfnr)):
        return REF_CUDA_SO
    os.makedirs(REF_DIR, exist_ok=True)
    scratch = tempfile.mkdtemp(prefix="refcuda_")
    try:
        with open(os.path.join(scratch, "rccr_kernels.inc"), "w") as f:
            f.write(_cut_between(rccr, "uchar4 remapC(const NVCVChannelManip manip)", "__global__ void resizeCrop_bilinear_varShape("))
        with open(os.path.join(scratch, "cfnr_kernels.inc"), "w") as f:
            f.write(_cut_between(cfnr, "__device__ float get_base_value(", "__global__ void slice_flip_normalize("))
        cmd = [
            os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc"), "-std=c++17", "-O3", "-gencode",
            "arch=compute_100a,code=sm_100a", "-lineinfo", "-w", "-DNDEBUG", "-Xcompiler", "-fPIC", "-shared",
            '-DREF_CUDA_RCCR_INC="rccr_kernels.inc"', '-DREF_CUDA_CFNR_INC="cfnr_kernels.inc"',
            "-I" + os.path.join(ref_root, "src/cvcuda/include"), "-I" + os.path.join(ref_root, "src/nvcv/src/include"),
            "-I" + scratch, "-o", REF_CUDA_SO, REF_CUDA_WRAP,
        ]
        subprocess.check_call(cmd)
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return REF_CUDA_SO


# ---------------------------------------------------------------------------------------------------------------------
# The reference's object model (libnvcv_types) and its own operators (a reduced libcvcuda), compiled from the reference
# tree where it lies with g++ / nvcc directly. The reference's build system is not run; the two things it would generate
# are produced here into a scratch directory: the version headers (a plain substitution of the version numbers into
# cmake/VersionDef.h.in and cmake/VersionUtils.h.in) and the linker version scripts (the list of NVCV_DEFINE_API /
# CVCUDA_DEFINE_API names per version node, which is all cmake/CreateExportsFile.cmake writes).

REF_NVCV_SO = os.path.join(REF_DIR, "libnvcv_types.so.0")
REF_CVCUDA_SO = os.path.join(REF_DIR, "libcvcuda_ref.so")
REF_VERSION = (0, 15, 0, 0)

# operators of the reduced reference library: the two of the hot path and the ones its un-fused chains are made of
REF_OPS = ["ResizeCropConvertReformat", "CropFlipNormalizeReformat", "Resize", "Normalize", "ConvertTo", "Reformat",
           "CopyMakeBorder", "RandomResizedCrop", "CustomCrop"]
REF_LEGACY = ["CvCudaLegacyHelpers.cpp", "resize_var_shape.cu", "normalize.cu", "normalize_var_shape.cu", "convert_to.cu",
              "reformat.cu", "copy_make_border.cu", "copy_make_border_var_shape.cu", "random_resized_crop.cu",
              "random_resized_crop_var_shape.cu", "custom_crop.cu"]


def _render_version_headers(ref_root: str, scratch: str) -> str:
    import re
    gen = os.path.join(scratch, "gen")
    sub = {"VERSION_MAJOR": REF_VERSION[0], "VERSION_MINOR": REF_VERSION[1], "VERSION_PATCH": REF_VERSION[2],
           "VERSION_TWEAK": REF_VERSION[3], "VERSION_SUFFIX": "", "VERSION_FULL": "%d.%d.%d" % REF_VERSION[:3],
           "VERSION_API_CODE": REF_VERSION[0] * 100 + REF_VERSION[1], "VERSION_BUILD": "%d_%d_%d-direct" % REF_VERSION[:3],
           "REPO_COMMIT": "unknown"}
    for prefix, inc in (("NVCV", "nvcv"), ("CVCUDA", "cvcuda")):
        for tmpl, out in (("VersionDef.h.in", "VersionDef.h"), ("VersionUtils.h.in", os.path.join("detail", "VersionUtils.h"))):
            text = open(os.path.join(ref_root, "cmake", tmpl)).read()
            text = re.sub(r"@(\w+)@", lambda m: str(dict(sub, LIBPREFIX=prefix).get(m.group(1), m.group(0))), text)
            dst = os.path.join(gen, inc, out)
            os.makedirs(os.path.dirname(dst), exist_ok=True)
            with open(dst, "w") as f:
                f.write(text)
    return gen


def _version_script(prefix: str, sources, out: str) -> str:
    import collections
    import re
    nodes = collections.defaultdict(set)
    for src in sources:
        for ln in open(src):
            m = re.match(r"^[A-Z_]+_DEFINE_API\(+([^,]+),([^,]+),[^,]+,([^,]+)", ln)
            if m:
                nodes[(int(m.group(1)), int(m.group(2)))].add(m.group(3).strip())
    text, prev = "", None
    for key in sorted(nodes):
        text += "%s_%d.%d {\nglobal:\n" % (prefix, *key) + "".join("    %s;\n" % fn for fn in sorted(nodes[key]))
        text += ("} %s_%d.%d;\n\n" % (prefix, *prev)) if prev else "local: *;\n};\n\n"
        prev = key
    with open(out, "w") as f:
        f.write(text)
    return out


def _compile_all(jobs, workers: int = 8):
    """jobs: list of argv lists; run them `workers` at a time, fail on the first error."""
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=workers) as pool:
        for rc, cmd in pool.map(lambda c: (subprocess.call(c), c), jobs):
            if rc != 0:
                raise subprocess.CalledProcessError(rc, cmd)


def build_ref_ops(ref_root: str = DEFAULT_REF_ROOT, force: bool = False):
    """oracle/_ref/libnvcv_types.so.0 (the reference's tensor / image / image-batch objects) and
    oracle/_ref/libcvcuda_ref.so (the reference's own operators of REF_OPS, sm_100a). Returns the two paths, or None when
    the reference tree is absent and no earlier build exists."""
    import glob
    nvcv_src = os.path.join(ref_root, "src/nvcv/src")
    cv_src = os.path.join(ref_root, "src/cvcuda")
    have = os.path.exists(REF_NVCV_SO) and os.path.exists(REF_CVCUDA_SO)
    if not os.path.isdir(nvcv_src) or not os.path.isdir(cv_src):
        return (REF_NVCV_SO, REF_CVCUDA_SO) if have else None
    if have and not force and not _stale(REF_CVCUDA_SO, __file__):
        return REF_NVCV_SO, REF_CVCUDA_SO
    os.makedirs(REF_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    scratch = tempfile.mkdtemp(prefix="refops_")
    try:
        gen = _render_version_headers(ref_root, scratch)
        util = [os.path.join(ref_root, "src/nvcv/util", f) for f in ("Assert.cpp", "CheckError.cpp", "String.cpp", "Version.cpp")]
        inc = ["-I" + os.path.join(ref_root, "src"), "-I" + os.path.join(nvcv_src, "include"), "-I" + nvcv_src, "-I" + gen,
               "-I/usr/local/cuda/include"]
        # --- libnvcv_types
        api = sorted(glob.glob(os.path.join(nvcv_src, "*.cpp")))
        srcs = api + sorted(glob.glob(os.path.join(nvcv_src, "priv", "*.cpp"))) + util
        objs, jobs = [], []
        for i, src in enumerate(srcs):
            obj = os.path.join(scratch, "nvcv_%d.o" % i)
            objs.append(obj)
            jobs.append(["g++", "-std=c++17", "-O2", "-fPIC", "-w", "-DNVCV_EXPORTING=1", *inc, "-c", src, "-o", obj])
        _compile_all(jobs)
        script = _version_script("NVCV", api, os.path.join(scratch, "nvcv.ldscript"))
        subprocess.check_call(["g++", "-shared", "-o", REF_NVCV_SO, *objs, "-Wl,--version-script=" + script,
                               "-Wl,-soname,libnvcv_types.so.0", "-L/usr/local/cuda/lib64", "-lcudart_static", "-ldl", "-lrt",
                               "-pthread"])
        link = os.path.join(REF_DIR, "libnvcv_types.so")
        if os.path.lexists(link):
            os.remove(link)
        os.symlink(os.path.basename(REF_NVCV_SO), link)
        # --- the reference's operators
        cinc = inc + ["-I" + os.path.join(cv_src, "include"), "-I" + cv_src]
        api = [os.path.join(cv_src, "Operator.cpp")] + [os.path.join(cv_src, "Op%s.cpp" % op) for op in REF_OPS]
        priv = [os.path.join(cv_src, "priv", "IOperator.cpp")]
        for op in REF_OPS:
            priv += [f for f in (os.path.join(cv_src, "priv", "Op%s.%s" % (op, ext)) for ext in ("cpp", "cu")) if os.path.exists(f)]
        legacy = [os.path.join(cv_src, "priv", "legacy", f) for f in REF_LEGACY]
        objs, jobs = [], []
        for i, src in enumerate(api + priv + legacy + util):
            obj = os.path.join(scratch, "cv_%d.o" % i)
            objs.append(obj)
            jobs.append([nvcc, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-w", "-DNDEBUG",
                         "-DCVCUDA_EXPORTING=1", "--expt-relaxed-constexpr", "--extended-lambda", "-Xcompiler", "-fPIC", *cinc,
                         "-c", src, "-o", obj])
        _compile_all(jobs)
        script = _version_script("CVCUDA", api, os.path.join(scratch, "cvcuda.ldscript"))
        subprocess.check_call([nvcc, "-shared", "-o", REF_CVCUDA_SO, *objs, "-Xlinker", "--version-script=" + script,
                               "-Xlinker", "-rpath,$ORIGIN", "-L" + REF_DIR, "-l:libnvcv_types.so.0"])
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return REF_NVCV_SO, REF_CVCUDA_SO


REF_HARNESS_SRC = os.path.join(HERE, "ref_ops_harness.cpp")
HARNESS_B200_SO = os.path.join(REF_DIR, "libharness_b200.so")
HARNESS_REF_SO = os.path.join(REF_DIR, "libharness_ref.so")


def build_ref_harness(ref_root: str = DEFAULT_REF_ROOT, force: bool = False):
    """oracle/_ref/libharness_b200.so and libharness_ref.so: ref_ops_harness.cpp (written against the reference's header-only
    C++ API) linked once against the B200 library and once against the reference's own operators, both over the
    reference's real libnvcv_types. Needs build_ref_ops' outputs and the B200 library."""
    b200 = os.path.join(os.path.dirname(HERE), "cv-cuda_b200", "libcvcuda_b200.so")
    have = os.path.exists(HARNESS_B200_SO) and os.path.exists(HARNESS_REF_SO)
    if not os.path.isdir(os.path.join(ref_root, "src/cvcuda/include")) or not os.path.exists(REF_CVCUDA_SO) or not os.path.exists(b200):
        return (HARNESS_B200_SO, HARNESS_REF_SO) if have else None
    if have and not force and not _stale(HARNESS_B200_SO, REF_HARNESS_SRC, REF_CVCUDA_SO) and not _stale(HARNESS_REF_SO, REF_HARNESS_SRC):
        return HARNESS_B200_SO, HARNESS_REF_SO
    scratch = tempfile.mkdtemp(prefix="refharness_")
    try:
        gen = _render_version_headers(ref_root, scratch)
        common = ["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-w", "-I" + os.path.join(ref_root, "src/cvcuda/include"),
                  "-I" + os.path.join(ref_root, "src/nvcv/src/include"), "-I" + gen, "-I/usr/local/cuda/include",
                  "-I" + os.path.join(os.path.dirname(HERE), "include"), REF_HARNESS_SRC]
        tail = ["-L" + REF_DIR, "-l:libnvcv_types.so.0", "-L/usr/local/cuda/lib64", "-lcudart_static", "-ldl", "-lrt", "-pthread"]
        # $ORIGIN = oracle/_ref; the B200 library sits in ../../cv-cuda_b200
        subprocess.check_call(common + ["-DHARNESS_B200", "-o", HARNESS_B200_SO, "-L" + os.path.dirname(b200), "-l:libcvcuda_b200.so",
                                        "-Wl,-rpath,$ORIGIN:$ORIGIN/../../cv-cuda_b200"] + tail)
        subprocess.check_call(common + ["-o", HARNESS_REF_SO, "-l:libcvcuda_ref.so", "-Wl,-rpath,$ORIGIN"] + tail)
    finally:
        shutil.rmtree(scratch, ignore_errors=True)
    return HARNESS_B200_SO, HARNESS_REF_SO


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-root", default=DEFAULT_REF_ROOT)
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    print("oracle:", build_oracle(a.force))
    print("reference golden:", build_ref(a.ref_root, a.force) or "reference tree absent, not built")
    print("reference CUDA kernels:", build_ref_cuda(a.ref_root, a.force) or "reference tree absent, not built")
    print("reference object model + operators:", build_ref_ops(a.ref_root, a.force) or "reference tree absent, not built")
    print("harness over the reference's C++ API:", build_ref_harness(a.ref_root, a.force) or "not built")
    return 0


if __name__ == "__main__":
    sys.exit(main())
