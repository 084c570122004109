"""Compile libsp_moe_b200 for sm_100a, in-tree (kairos_engine_b200/lib/): the shared library the
Python mirror and the tests load, and the static archive a daemon links the way the reference links
its own backend (`cargo:rustc-link-lib=static=...`, tools/sp_daemon/build.rs:396-454).

nvcc cross-compiles without a GPU. Run as `python -m kairos_engine_b200.build [--force] [-v]`.
"""
import glob
import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "lib")
OBJDIR = os.path.join(LIBDIR, "obj")
LIB = os.path.join(LIBDIR, "libsp_moe_b200.so")
ARCHIVE = os.path.join(LIBDIR, "libsp_moe_b200.a")

CC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC"]
# flags of the one-step build the objects replace; kept for scripts that compile a debug variant themselves
NVCC_FLAGS = CC_FLAGS + ["-shared", "-cudart", "static"]


def sources():
    return sorted(glob.glob(os.path.join(CSRC, "*.cu")))


def _headers():
    return glob.glob(os.path.join(CSRC, "*.cuh")) + glob.glob(os.path.join(HERE, "..", "include", "sp_engine", "*.h"))


def _obj(src):
    return os.path.join(OBJDIR, os.path.basename(src)[:-3] + ".o")


def stale():
    if not (os.path.exists(LIB) and os.path.exists(ARCHIVE)):
        return True
    t = min(os.path.getmtime(LIB), os.path.getmtime(ARCHIVE))
    return any(os.path.getmtime(p) > t for p in sources() + _headers())


def _run(cmd):
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed: " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    return r.stderr


def build(force=False, verbose=False):
    if not force and not stale():
        return LIB
    os.makedirs(OBJDIR, exist_ok=True)
    hdr_t = max(os.path.getmtime(p) for p in _headers())
    todo = [s for s in sources() if force or not os.path.exists(_obj(s)) or os.path.getmtime(_obj(s)) < max(os.path.getmtime(s), hdr_t)]
    extra = ["-Xptxas", "-v"] if verbose else []
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(todo)))) as ex:
        logs = list(ex.map(lambda s: _run(["nvcc"] + CC_FLAGS + extra + ["-c", s, "-o", _obj(s)]), todo))
    if verbose:
        print("".join(logs))
    live = {_obj(s) for s in sources()}
    for o in glob.glob(os.path.join(OBJDIR, "*.o")):          # an object whose source is gone must not be linked
        if o not in live:
            os.remove(o)
    objs = sorted(live)
    _run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-cudart", "static", "-o", LIB] + objs)
    if os.path.exists(ARCHIVE):
        os.remove(ARCHIVE)
    _run(["ar", "rcs", ARCHIVE] + objs)
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv))
