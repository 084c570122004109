"""Builds tests/abi_harness.c with gcc against include/sp_engine/moe_backend.h and runs it twice:
linked against the shared library and against the static archive (the form the reference's daemon
links its backend in, tools/sp_daemon/build.rs:396-454). The harness calls every exported entry
from plain C, with the structs laid out by the C compiler."""
import os
import shutil
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CUDA = os.environ.get("CUDA_HOME", "/usr/local/cuda")


def _build_and_run(tmp_path, static):
    from kairos_engine_b200 import build
    build.build()
    exe = str(tmp_path / ("harness_static" if static else "harness_shared"))
    libdir = os.path.dirname(build.LIB)
    cmd = ["gcc", "-O1", "-std=gnu11", "-I" + os.path.join(ROOT, "include"), "-I" + os.path.join(CUDA, "include"),
           os.path.join(ROOT, "tests", "abi_harness.c"), "-o", exe]
    if static:
        cmd += [build.ARCHIVE, "-L" + os.path.join(CUDA, "lib64"), "-lcudart_static", "-lstdc++", "-lm", "-ldl", "-lrt", "-lpthread"]
    else:
        cmd += ["-L" + libdir, "-lsp_moe_b200", "-Wl,-rpath," + libdir, "-L" + os.path.join(CUDA, "lib64"), "-lcudart", "-Wl,-rpath," + os.path.join(CUDA, "lib64"), "-lm"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, "gcc failed:\n" + r.stdout + r.stderr
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, "harness failed:\n" + r.stdout[-4000:] + r.stderr[-2000:]
    assert r.stdout.strip().splitlines()[-1].startswith("OK:"), r.stdout[-2000:]


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_c_harness_against_the_shared_library(tmp_path):
    _build_and_run(tmp_path, static=False)


@pytest.mark.skipif(shutil.which("gcc") is None, reason="needs gcc")
def test_c_harness_against_the_static_archive(tmp_path):
    _build_and_run(tmp_path, static=True)
