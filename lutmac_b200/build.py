"""Builds the CUDA library in-tree: lutmac_b200/liblutmac_b200.so (sm_100a only)."""
from __future__ import annotations

import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "liblutmac_b200.so")
LIB_DEBUG_BOUNDS = os.path.join(HERE, "liblutmac_b200_dbg.so")  # range-checking build, see include/lutmac_b200.h: lmb_debug_bounds

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-O2",
]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def needs_build(lib: str = LIB) -> bool:
    if not os.path.exists(lib):
        return True
    t = os.path.getmtime(lib)
    deps = sources() + glob.glob(os.path.join(CSRC, "*.cuh")) + [os.path.join(HERE, "..", "include", "lutmac_b200.h")]
    return any(os.path.getmtime(d) > t for d in deps)


def build(force: bool = False, verbose: bool = False, debug_bounds: bool = False) -> str:
    """Compile every .cu under csrc/ for sm_100a and link them into one shared library.
    debug_bounds: the range-checking variant (-DLMB_DEBUG_BOUNDS) as liblutmac_b200_dbg.so."""
    lib = LIB_DEBUG_BOUNDS if debug_bounds else LIB
    if not force and not needs_build(lib):
        return lib
    nvcc = os.environ.get("NVCC", "nvcc")
    objdir = os.path.join(HERE, "build", "dbg") if debug_bounds else os.path.join(HERE, "build")
    os.makedirs(objdir, exist_ok=True)
    objs = []
    procs = []
    for src in sources():
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        objs.append(obj)
        cmd = [nvcc] + NVCC_FLAGS + (["-DLMB_DEBUG_BOUNDS=1"] if debug_bounds else []) + (["-Xptxas", "-v"] if verbose else []) + ["-c", src, "-o", obj]
        procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    for cmd, p in procs:
        out, _ = p.communicate()
        if verbose or p.returncode != 0:
            sys.stderr.write(out)
        if p.returncode != 0:
            raise RuntimeError("nvcc failed: " + " ".join(cmd))
    link = [nvcc, "-shared", "-o", lib] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"]
    subprocess.run(link, check=True)
    return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, debug_bounds="--debug-bounds" in sys.argv))
