"""No-GPU checks of the C-ABI library: it loads, exports every symbol the header declares, and
every entry fails loudly (no CPU fallback) when there is no CUDA device."""
import ctypes as C
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _lib():
    from kairos_engine_b200 import _lib, build
    build.build()
    return _lib


def test_library_exports_every_declared_symbol():
    L = _lib()
    header = open(os.path.join(ROOT, "include", "sp_engine", "moe_backend.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b((?:sp_|gemma4_)\w+)\s*\(", header))
    declared -= {"sp_moe"}                       # the opaque type
    assert declared, "no declarations found"
    lib = L.lib()
    missing = [s for s in sorted(declared) if not hasattr(lib, s)]
    assert not missing, f"declared in the header but not exported: {missing}"
    assert set(L.EXPORTS) == declared, (set(L.EXPORTS) ^ declared)


def test_error_text_is_thread_local_and_settable():
    L = _lib().lib()
    L.sp_set_error(b"hello")
    assert L.sp_last_error() == b"hello"


def _no_gpu():
    import torch
    return not torch.cuda.is_available()


@pytest.mark.skipif(not _no_gpu(), reason="checks the no-device failure mode")
def test_open_fails_loudly_without_a_device():
    from kairos_engine_b200 import MoeEngine, SpMoeError
    with pytest.raises(SpMoeError) as ei:
        MoeEngine(128, 8, 2, 32, 64, 1)
    assert ei.value.code == -40 and "no CPU path" in ei.value.text


def test_bad_arguments_are_rejected_before_any_cuda_call():
    from kairos_engine_b200 import MoeEngine, SpMoeError
    for kw in (dict(E=100, NE=8, NU=2, FFE=32, FFS=64), dict(E=128, NE=8, NU=9, FFE=32, FFS=64),
               dict(E=128, NE=2, NU=4, FFE=32, FFS=64), dict(E=8192, NE=8, NU=2, FFE=32, FFS=64),
               dict(E=128, NE=8, NU=2, FFE=48, FFS=64)):
        with pytest.raises(SpMoeError) as ei:
            MoeEngine(n_layers=1, **kw)
        assert ei.value.code == -3, kw
    L = _lib().lib()
    assert L.sp_moe_close(None) == 0                 # NULL-safe, like the reference's close (glue:390-393)
    assert L.gemma4_moe_ffn_q4b_cuda(100, 8, 2, 32, C.c_float(1e-6), *([None] * 9)) == 1     # E % 32 != 0, CF:13828
    assert b"%32" in L.sp_last_error()
    assert L.sp_moe_q4b_quantize_dev(None, 1, 32, None, None, None) == -3
