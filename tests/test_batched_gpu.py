"""GPU parity of the M > 1 paths (through the C ABI) against the CPU checker, both arithmetic
flavours, plus consistency between the batched decode arithmetic and the M=1 decode kernel."""
import numpy as np
import pytest

import orc
from gpu_common import assert_close, assert_same_experts, make_stack, oracle_stack

pytestmark = pytest.mark.gpu
A, B = 0, 1


@pytest.mark.parametrize("cfg,n_layers,M", [(orc.TINY, 2, 2), (orc.TINY, 1, 7), (orc.SMALL, 3, 16), (orc.SMALL, 1, 33)])
def test_batched_decode_flavour_small(cfg, n_layers, M):
    eng, host = make_stack(cfg, n_layers, seed=21, rand_norms=True, max_tokens=M)
    x = np.random.default_rng(M).standard_normal((M, cfg["E"])).astype(np.float32)
    y, sel, wts = eng.forward(x, flavour=A)
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, A)
    assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
    assert_close(y, ry, "batched decode flavour")
    # each row equals what the single-token decode kernel gives for that token, bit for bit
    for t in range(min(M, 3)):
        y1, sel1, _ = eng.forward(x[t:t + 1], flavour=A)
        assert np.array_equal(sel1[:, 0], sel[:, t])
        assert np.array_equal(y1[0].view(np.uint32), y[t].view(np.uint32))
    eng.close()


@pytest.mark.parametrize("cfg,n_layers,M", [(orc.TINY, 2, 2), (orc.SMALL, 2, 5), (orc.GEMMA, 1, 3)])
def test_small_decode_batch_both_routes(cfg, n_layers, M, monkeypatch):
    """A decode batch of a few tokens runs token by token through the single-token graph by default;
    SP_MOE_SEQ_TOKENS=1 sends it to the batched kernels instead (tensor-core row dots, per-expert router
    blocks). Both give the checker's result and each other's, bit for bit, routing tables included."""
    x = np.random.default_rng(50 + M).standard_normal((M, cfg["E"])).astype(np.float32)
    outs = []
    for seq in ("8", "1"):
        monkeypatch.setenv("SP_MOE_SEQ_TOKENS", seq)
        eng, host = make_stack(cfg, n_layers, seed=23, rand_norms=True, max_tokens=M)
        outs.append(eng.forward(x, flavour=A))
        eng.close()
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, A)
    for y, sel, wts in outs:
        assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
        assert_close(y, ry, "small decode batch")
    assert np.array_equal(outs[0][0].view(np.uint32), outs[1][0].view(np.uint32))
    assert np.array_equal(outs[0][2].view(np.uint32), outs[1][2].view(np.uint32))


@pytest.mark.parametrize("cfg,n_layers,M", [(orc.TINY, 2, 3), (orc.SMALL, 2, 40), (orc.SMALL, 1, 1)])
def test_batched_prefill_flavour_small(cfg, n_layers, M):
    eng, host = make_stack(cfg, n_layers, seed=22, rand_norms=True, max_tokens=M)
    x = np.random.default_rng(M + 100).standard_normal((M, cfg["E"])).astype(np.float32)
    y, sel, wts = eng.forward(x, flavour=B)
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, B)
    assert_same_experts(sel, rsel, wts, rwts, margin)
    np.testing.assert_allclose(np.sort(wts, axis=-1), np.sort(rwts, axis=-1), rtol=1e-5, atol=1e-7)
    assert_close(y, ry, "batched prefill flavour")
    eng.close()


@pytest.mark.parametrize("flavour,M", [(A, 8), (B, 24)])
def test_batched_gemma_geometry(flavour, M):
    cfg = orc.GEMMA
    eng, host = make_stack(cfg, 1, seed=5, max_tokens=M)
    x = np.random.default_rng(9).standard_normal((M, cfg["E"])).astype(np.float32)
    y, sel, wts = eng.forward(x, flavour=flavour)
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, flavour)
    assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
    assert_close(y, ry, f"gemma geometry flavour {flavour} M={M}")
    # every token chose NU distinct experts
    assert all(len(set(row)) == cfg["NU"] for row in sel[0])
    eng.close()


def test_zipf_bias_skews_routing_and_stays_exact():
    import torch
    from kairos_engine_b200 import synth
    cfg = orc.SMALL
    bias = synth.zipf_bias(cfg["NE"], s=1.2, seed=3)
    eng, host = make_stack(cfg, 1, seed=8, max_tokens=64, bias=bias)
    x = np.random.default_rng(1).standard_normal((64, cfg["E"])).astype(np.float32)
    y, sel, _ = eng.forward(x, flavour=A)
    ry, rsel, _, _ = oracle_stack(cfg, host, x, A)
    assert np.array_equal(sel, rsel)
    assert_close(y, ry, "zipf")
    counts = np.bincount(sel.reshape(-1), minlength=cfg["NE"])
    assert counts.max() >= 4 * max(1, np.median(counts))      # a few experts take most tokens
    eng.close()
