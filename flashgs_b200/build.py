"""In-tree build of ``libflashgs_b200.so`` (hand-written CUDA for sm_100a behind a C ABI).

``python -m flashgs_b200.build`` compiles every ``csrc/*.cu`` with
``nvcc -gencode arch=compute_100a,code=sm_100a`` and links one shared library next to
this file. nvcc cross-compiles without a GPU, so the build also serves as the
"does it compile" check on machines that have none.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libflashgs_b200.so")
LIB_CHECKED = os.path.join(HERE, "libflashgs_b200_checked.so")
OBJ_DIR = os.path.join(HERE, "build")

CXX = os.environ.get("FLASHGS_CXX", "/usr/bin/g++")     # host compiler behind nvcc
NVCC = os.environ.get("FLASHGS_NVCC", "nvcc")
EXTRA = os.environ.get("FLASHGS_NVCC_FLAGS", "").split()   # e.g. -DFGS_DEBUG_BOUNDS for the checked build

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-ccbin", CXX,
    "-Xcompiler", "-fPIC", "-Xcompiler", "-ffp-contract=off",  # host matrices: one rounding per operation
    "-Xptxas", "-v",
]


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, checked: bool = False) -> str:
    """Compile and link the library. ``checked=True`` builds the flavour with ``-DFGS_DEBUG_BOUNDS`` (every store and
    computed index compared with its extent first, violations reported through the device status word) into
    ``libflashgs_b200_checked.so``; the tests run their small cases under it."""
    srcs = sorted(glob.glob(os.path.join(CSRC, "*.cu")))
    hdrs = glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "*.h"))
    obj_dir = OBJ_DIR + ("_checked" if checked else "")
    lib = LIB_CHECKED if checked else LIB
    flags = NVCC_FLAGS + EXTRA + (["-DFGS_DEBUG_BOUNDS"] if checked else [])
    os.makedirs(obj_dir, exist_ok=True)
    jobs = []
    for s in srcs:
        o = os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o")
        if force or _stale(o, [s] + hdrs):
            jobs.append((s, o))

    def compile_one(job):
        s, o = job
        r = subprocess.run([NVCC, "-c", s, "-o", o] + flags, capture_output=True, text=True)
        with open(o + ".log", "w") as f:
            f.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError("nvcc failed on %s:\n%s" % (s, r.stdout + r.stderr))
        return r.stderr

    with cf.ThreadPoolExecutor(max_workers=4) as ex:
        for log in ex.map(compile_one, jobs):
            if verbose:
                print(log)
    objs = [os.path.join(obj_dir, os.path.basename(s)[:-3] + ".o") for s in srcs]
    if force or jobs or _stale(lib, objs):
        subprocess.check_call([NVCC, "-shared", "-o", lib] + objs + ["-ccbin", CXX, "-lcudart"])
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, checked="--checked" in sys.argv))
