"""Edge cases of the layer through the C ABI, against the CPU checker: exact routing ties, an
all-zero token, large activations, the largest batch a handle accepts, a one-expert-takes-all router."""
import numpy as np
import pytest

import orc
from gpu_common import assert_close, assert_same_experts, oracle_stack

pytestmark = pytest.mark.gpu
A, B = 0, 1


def _stack(cfg, layers_host, max_tokens):
    from kairos_engine_b200 import MoeEngine
    eng = MoeEngine(n_layers=len(layers_host), max_tokens=max_tokens, **cfg)
    for L, lay in enumerate(layers_host):
        eng.upload_layer(L, lay)
    return eng, [orc.LayerWeights(**lay) for lay in layers_host]


def _host_layer(cfg, seed, **kw):
    from kairos_engine_b200 import synth
    return synth.layer_to_host(synth.make_layer(cfg, seed, rand_norms=True, **kw))


def test_exact_probability_ties_go_to_the_lower_expert_id():
    cfg = orc.SMALL
    lay = _host_layer(cfg, 61)
    lay["router_w"] = lay["router_w"].copy()
    lay["router_w"][1::2] = lay["router_w"][0::2]          # experts 2k and 2k+1 get identical logits
    eng, host = _stack(cfg, [lay], 8)
    x = np.random.default_rng(1).standard_normal((8, cfg["E"])).astype(np.float32)
    for M, flavour in ((1, A), (8, A), (8, B)):
        y, sel, wts = eng.forward(x[:M], flavour=flavour)
        ry, rsel, rwts, _ = oracle_stack(cfg, host, x[:M], flavour)
        assert np.array_equal(sel, rsel)
        # inside the selection a tied pair appears lower id first
        for row, w in zip(sel[0], wts[0]):
            for k in range(cfg["NU"] - 1):
                if w[k] == w[k + 1]:
                    assert row[k] < row[k + 1]
        assert_close(y, ry, f"ties M={M} flavour={flavour}")
    eng.close()


@pytest.mark.parametrize("flavour", [A, B])
def test_zero_token_and_large_activations(flavour):
    cfg = orc.SMALL
    eng, host = _stack(cfg, [_host_layer(cfg, 62), _host_layer(cfg, 63)], 4)
    x = np.random.default_rng(2).standard_normal((4, cfg["E"])).astype(np.float32)
    x[1] = 0.0                                              # rms(0) = 0 * 1/sqrt(eps): stays 0 through the layer
    x[2] *= 1e4
    x[3] *= 1e-4
    y, sel, wts = eng.forward(x, flavour=flavour)
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, flavour)
    assert np.isfinite(y).all()
    if flavour == A:
        assert np.array_equal(sel, rsel)
        assert np.array_equal(y.view(np.uint32), ry.view(np.uint32))       # the decode arithmetic is bit-exact
    else:
        assert_same_experts(sel, rsel, wts, rwts, margin)
        d = np.abs(y.astype(np.float64) - ry)
        assert (d <= 2e-3 + 1e-6 * np.abs(ry)).all()        # the gate, scaled for the 1e4-magnitude row
    eng.close()


def test_largest_batch_and_one_more_is_refused():
    from kairos_engine_b200 import SpMoeError
    cfg = orc.TINY
    eng, host = _stack(cfg, [_host_layer(cfg, 64)], 33)
    x = np.random.default_rng(3).standard_normal((34, cfg["E"])).astype(np.float32)
    y, sel, _ = eng.forward(x[:33], flavour=A)
    ry, rsel, _, _ = oracle_stack(cfg, host, x[:33], A)
    assert np.array_equal(sel, rsel) and np.array_equal(y.view(np.uint32), ry.view(np.uint32))
    with pytest.raises(SpMoeError):
        eng.forward(x, flavour=A)
    eng.close()


def test_router_that_sends_every_token_to_the_same_experts():
    import torch
    cfg = orc.SMALL
    bias = torch.full((cfg["NE"],), -30.0)
    bias[:cfg["NU"]] = 30.0                                 # the first NU experts always win
    lay = _host_layer(cfg, 65, bias=bias.cuda())
    eng, host = _stack(cfg, [lay], 200)
    x = np.random.default_rng(4).standard_normal((200, cfg["E"])).astype(np.float32)
    y, sel, wts = eng.forward(x, flavour=B)
    assert set(sel.reshape(-1).tolist()) == set(range(cfg["NU"]))
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, B)
    assert_same_experts(sel, rsel, wts, rwts, margin)
    assert_close(y, ry, "all tokens on the same experts")
    eng.close()
