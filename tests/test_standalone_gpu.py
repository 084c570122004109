"""gemma4_moe_ffn_q4b_cuda — the reference's self-contained single-token operator, exported with
its own signature (src/backends/cuda/cuda_forward.cu:13821-13977) — against the CPU checker's
restatement of the same lines. Its semantics are NOT the served layer's: one weightless RMS norm
with a float sum, float expf softmax, no clamp on the renormalisation, experts accumulated in
descending-probability order."""
import ctypes as C

import numpy as np
import pytest

import orc
from gpu_common import assert_close

pytestmark = pytest.mark.gpu


def _random_q4b(rng, rows, cols):
    """Valid Q4B bytes without running a quantiser over half a billion weights: codes in [-7, 7]
    (two's-complement nibbles, low nibble = even column), f16 block scales around 0.02 * 3 / 7."""
    v = rng.integers(-7, 8, size=(rows, cols), dtype=np.int8)
    codes = ((v[:, 0::2] & 0xF) | ((v[:, 1::2] & 0xF) << 4)).astype(np.uint8)
    bs = rng.uniform(0.004, 0.012, size=(rows, cols // 32)).astype(np.float16).view(np.uint16)
    return np.ascontiguousarray(codes), np.ascontiguousarray(bs)


@pytest.mark.parametrize("E,NE,NU,FF", [(256, 16, 4, 64), (2816, 128, 8, 704)])
def test_standalone_operator_matches_checker(E, NE, NU, FF):
    from kairos_engine_b200 import _lib
    L = _lib.lib()
    rng = np.random.default_rng(E + NE)
    eps = 1e-6
    gate_inp = (rng.standard_normal((NE, E)) * 0.02).astype(np.float32)
    gate_scale = rng.uniform(0.5, 1.5, E).astype(np.float32)
    gu_codes, gu_bs = _random_q4b(rng, NE * 2 * FF, E)
    dn_codes, dn_bs = _random_q4b(rng, NE * E, FF)
    for trial in range(2):
        hidden = rng.standard_normal(E).astype(np.float32) * (1.0 + trial)
        out = np.full(E, np.nan, np.float32)
        sel = np.full(NU, -1, np.int32)
        rc = L.gemma4_moe_ffn_q4b_cuda(E, NE, NU, FF, C.c_float(eps), gate_inp.ctypes.data, gate_scale.ctypes.data,
                                       gu_codes.ctypes.data, gu_bs.ctypes.data, dn_codes.ctypes.data, dn_bs.ctypes.data,
                                       hidden.ctypes.data, out.ctypes.data, sel.ctypes.data)
        assert rc == 0, L.sp_last_error()
        rrc, rout, rsel = orc.standalone_q4b(E, NE, NU, FF, eps, gate_inp, gate_scale, gu_codes, gu_bs, dn_codes, dn_bs, hidden)
        assert rrc == 0
        assert np.array_equal(sel, rsel), "expert ids (descending probability) differ from the checker"
        assert_close(out, rout, f"standalone operator E={E} trial {trial}")


def test_standalone_operator_sel_out_is_optional():
    from kairos_engine_b200 import _lib
    L = _lib.lib()
    E, NE, NU, FF = 128, 8, 2, 32
    rng = np.random.default_rng(5)
    gate_inp = (rng.standard_normal((NE, E)) * 0.02).astype(np.float32)
    gate_scale = np.ones(E, np.float32)
    gu_codes, gu_bs = _random_q4b(rng, NE * 2 * FF, E)
    dn_codes, dn_bs = _random_q4b(rng, NE * E, FF)
    hidden = rng.standard_normal(E).astype(np.float32)
    out = np.empty(E, np.float32)
    rc = L.gemma4_moe_ffn_q4b_cuda(E, NE, NU, FF, C.c_float(1e-6), gate_inp.ctypes.data, gate_scale.ctypes.data,
                                   gu_codes.ctypes.data, gu_bs.ctypes.data, dn_codes.ctypes.data, dn_bs.ctypes.data,
                                   hidden.ctypes.data, out.ctypes.data, None)
    assert rc == 0, L.sp_last_error()
    _, rout, _ = orc.standalone_q4b(E, NE, NU, FF, 1e-6, gate_inp, gate_scale, gu_codes, gu_bs, dn_codes, dn_bs, hidden)
    assert_close(out, rout, "standalone operator, no sel_out")
