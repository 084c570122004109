"""Tensor-core prefill GEMMs (tcgen05 path) against the CPU checker and against the CUDA-core
fp32 kernels of the same library, through the C ABI."""
import os

import numpy as np
import pytest

import orc
from gpu_common import assert_close, assert_same_experts, make_stack, oracle_stack

pytestmark = pytest.mark.gpu
B = 1


def _simt_stack(cfg, n_layers, seed, max_tokens, **kw):
    os.environ["SP_MOE_PREFILL_IMPL"] = "simt"
    try:
        return make_stack(cfg, n_layers, seed=seed, max_tokens=max_tokens, **kw)
    finally:
        del os.environ["SP_MOE_PREFILL_IMPL"]


@pytest.mark.parametrize("M", [5, 1, 16, 129, 300])
def test_small_geometry_matches_checker_and_simt(M):
    cfg = orc.SMALL
    eng, host = make_stack(cfg, 2, seed=41, rand_norms=True, max_tokens=max(M, 2))
    ref_eng, _ = _simt_stack(cfg, 2, 41, max(M, 2), rand_norms=True)
    x = np.random.default_rng(M).standard_normal((M, cfg["E"])).astype(np.float32)
    l0, s0 = eng.kernel_launches, ref_eng.kernel_launches
    y, sel, wts = eng.forward(x, flavour=B)
    ys, sels, _ = ref_eng.forward(x, flavour=B)
    if M > 1:       # the two engines really ran different kernels: 14 launches per layer with the grouped GEMMs, 8 without
        assert (eng.kernel_launches - l0, ref_eng.kernel_launches - s0) == (28, 16)
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, B)
    assert_same_experts(sel, rsel, wts, rwts, margin)
    assert_close(y, ry, f"tensor-core prefill vs checker, M={M}")
    # the split-fp16 arithmetic carries ~22 bits: far inside the gate, close to the fp32 kernels
    assert np.abs(y - ys).max() <= 2e-4
    eng.close(); ref_eng.close()


@pytest.mark.parametrize("M", [24, 200])
def test_gemma_geometry(M):
    cfg = orc.GEMMA
    eng, host = make_stack(cfg, 1, seed=6, max_tokens=M)
    x = np.random.default_rng(10 + M).standard_normal((M, cfg["E"])).astype(np.float32)
    y, sel, wts = eng.forward(x, flavour=B)
    n_ref = min(M, 32)                                    # the checker takes seconds per 32 tokens at this size
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x[:n_ref], B)
    assert np.array_equal(sel[:, :n_ref], rsel), f"expert ids differ (min margin {margin:.3e})"
    assert_close(y[:n_ref], ry, f"gemma geometry, tensor-core prefill, M={M}")
    # rows do not depend on which other rows share the batch
    y2, _, _ = eng.forward(x[: M // 2], flavour=B)
    assert np.array_equal(y2.view(np.uint32), y[: M // 2].view(np.uint32))
    eng.close()


@pytest.mark.parametrize("terms", [2, 1])
def test_fewer_terms_one_layer(terms, monkeypatch):
    """SP_MOE_PREFILL_TERMS=2 rounds the dequantised weight to fp16, =1 rounds the activation as well (the
    reference's SP_G4_GEMM_F16 mode). One Gemma-geometry layer stays inside the gate; the measured error is
    reported so the cost of each dropped term is on record. Expert ids do not depend on the GEMMs."""
    cfg = orc.GEMMA
    M = 32
    monkeypatch.setenv("SP_MOE_PREFILL_TERMS", str(terms))
    eng, host = make_stack(cfg, 1, seed=6, max_tokens=M)
    x = np.random.default_rng(77).standard_normal((M, cfg["E"])).astype(np.float32)
    y, sel, wts = eng.forward(x, flavour=B)
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, B)
    assert np.array_equal(sel, rsel)
    d = y.astype(np.float64) - ry.astype(np.float64)
    max_abs, rel = np.abs(d).max(), np.linalg.norm(d) / np.linalg.norm(ry.astype(np.float64))
    print(f"terms={terms}: max-abs {max_abs:.3e} rel-L2 {rel:.3e}")
    if terms == 2:
        assert_close(y, ry, "tensor-core prefill, weight rounded to fp16")           # inside the gate
    else:
        # fp16 x fp16 leaves the gate on max-abs (about 2.4e-3 against 2e-3 here): an opt-in mode, never the default
        assert rel <= 1e-3 and max_abs <= 5e-3
    eng.close()


def test_skewed_routing_many_rows_on_one_expert():
    from kairos_engine_b200 import synth
    cfg = orc.SMALL
    bias = synth.zipf_bias(cfg["NE"], s=2.0, seed=4) * 4.0
    M = 400
    eng, host = make_stack(cfg, 1, seed=43, max_tokens=M, bias=bias)
    x = np.random.default_rng(2).standard_normal((M, cfg["E"])).astype(np.float32)
    y, sel, _ = eng.forward(x, flavour=B)
    ry, rsel, _, margin = oracle_stack(cfg, host, x, B)
    assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
    assert np.bincount(sel.reshape(-1), minlength=cfg["NE"]).max() > 128      # some expert needs more than one tile
    assert_close(y, ry, "skewed routing")
    eng.close()
