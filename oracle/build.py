"""Build recipes for the checker side: the CPU oracle and the reference's own CUDA build.

Both outputs are test infrastructure. ``libfgs_oracle.so`` is the C++/OpenMP
restatement in ``fgs_oracle.cpp``. ``_ref/flash_gaussian_splatting*.so`` is the
unmodified reference compiled from its own sources where they lie (never copied
into this repository) with the flags its ``setup.py`` uses (``-O1``,
``-Xptxas=-O1``, setup.py:19-20); it needs the reference checkout and is
skipped when that is absent.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "libfgs_oracle.so")
REF_DIR = os.path.join(HERE, "_ref")
REF_SO = os.path.join(REF_DIR, "flash_gaussian_splatting.so")
# Tool and source locations; each can be overridden from the environment.
CXX = os.environ.get("FLASHGS_CXX", "/usr/bin/g++")   # the system compiler; a wrapped compiler produced a reference module that crashed in loadPly
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")
# the reference checkout: by default a directory named "reference" beside this repository
REFERENCE_ROOT = os.environ.get("FLASHGS_REFERENCE_ROOT", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference"))
REF_EXAMPLE = os.path.join(REF_DIR, "example.py")   # the reference's example script, beside its build (untracked like it)


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "fgs_oracle.cpp")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    cmd = [CXX, "-O2", "-std=c++17", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
           "-shared", "-fPIC", src, "-o", ORACLE_SO]
    subprocess.check_call(cmd)
    return ORACLE_SO


def build_reference(ref_root: str = REFERENCE_ROOT, force: bool = False):
    """Compile the reference extension from its own sources into ``oracle/_ref``. Returns the path or None.
    The reference's example script is placed beside the build (a test runs it, unmodified, against this
    repository's drop-in module); like the build it stays out of the history."""
    example = os.path.join(ref_root, "example.py")
    if os.path.exists(example):
        import shutil
        os.makedirs(REF_DIR, exist_ok=True)
        if not os.path.exists(REF_EXAMPLE) or os.path.getmtime(REF_EXAMPLE) < os.path.getmtime(example):
            shutil.copyfile(example, REF_EXAMPLE)
    srcs = [os.path.join(ref_root, "csrc", "cuda_rasterizer", f) for f in ("preprocess.cu", "sort.cu", "render.cu")]
    binding = os.path.join(ref_root, "csrc", "pybind.cpp")
    if not all(os.path.exists(s) for s in srcs + [binding]):
        return REF_SO if os.path.exists(REF_SO) else None
    if not force and _newer(REF_SO, srcs + [binding]):
        return REF_SO
    import torch
    from torch.utils import cpp_extension as ce

    os.makedirs(REF_DIR, exist_ok=True)
    inc = []
    for d in ce.include_paths() + [sysconfig.get_paths()["include"], os.path.join(CUDA_HOME, "include")]:
        inc += ["-isystem", d]
    defs = ["-DTORCH_EXTENSION_NAME=flash_gaussian_splatting", "-DTORCH_API_INCLUDE_EXTENSION_H",
            "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)]
    objs = []
    for s in srcs:
        o = os.path.join(REF_DIR, os.path.basename(s) + ".o")
        cmd = ["nvcc", "-ccbin", CXX, "-c", s, "-o", o, "-O1", "-Xptxas=-O1", "-std=c++17",
               "--expt-relaxed-constexpr", "-gencode=arch=compute_100,code=sm_100",
               "-D__CUDA_NO_HALF_OPERATORS__", "-D__CUDA_NO_HALF_CONVERSIONS__",
               "-D__CUDA_NO_BFLOAT16_CONVERSIONS__", "-D__CUDA_NO_HALF2_OPERATORS__",
               "--compiler-options", "-fPIC"] + defs + inc
        subprocess.check_call(cmd)
        objs.append(o)
    o = os.path.join(REF_DIR, "pybind.o")
    subprocess.check_call([CXX, "-c", binding, "-o", o, "-g", "-O1", "-std=c++17", "-fPIC"] + defs + inc)
    objs.append(o)
    libdirs = ce.library_paths() + [os.path.join(CUDA_HOME, "lib64")]
    link = [CXX, "-shared", "-o", REF_SO] + objs
    for d in libdirs:
        link += ["-L" + d, "-Wl,-rpath," + d]
    link += ["-lc10", "-ltorch_cpu", "-ltorch", "-ltorch_python", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
    subprocess.check_call(link)
    return REF_SO


if __name__ == "__main__":
    print(build_oracle(force="--force" in sys.argv))
    if "--ref" in sys.argv:
        print(build_reference(force="--force" in sys.argv))
