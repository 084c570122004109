"""Shared helpers of the GPU parity tests: build the same seeded layers on the device (for the
CUDA library) and on the host (for the CPU checker), and compare within the stated tolerance."""
import numpy as np

import orc

# tolerance of the parity gate: hidden states max-abs 2e-3 and rel-L2 1e-3; expert ids bit-exact
MAX_ABS = 2e-3
REL_L2 = 1e-3


def make_stack(cfg, n_layers, seed=0, rand_norms=False, max_tokens=1, bias=None, **engine_kw):
    """-> (engine, [orc.LayerWeights per layer]) holding identical bytes."""
    import torch
    from kairos_engine_b200 import MoeEngine, synth
    eng = MoeEngine(n_layers=n_layers, max_tokens=max_tokens, **engine_kw, **cfg)
    host_layers = []
    for L in range(n_layers):
        layer = synth.make_layer(cfg, seed + 1000 * L, rand_norms=rand_norms, bias=bias)
        eng.upload_layer(L, layer, on_device=True)
        host_layers.append(orc.LayerWeights(**synth.layer_to_host(layer)))
        del layer
    torch.cuda.synchronize()
    return eng, host_layers


def oracle_stack(cfg, host_layers, x, flavour, first=0, n=None):
    """Runs the checker layer by layer; returns y, sel [n][M][NU], wts, min routing margin."""
    n = len(host_layers) - first if n is None else n
    cur = np.ascontiguousarray(x, np.float32)
    sels, wts, margin = [], [], np.inf
    for L in range(first, first + n):
        r = orc.layer_forward(cfg, host_layers[L], cur, flavour, want_margin=True)
        assert r["rc"] == 0
        cur = r["y"]
        sels.append(r["sel"]); wts.append(r["wts"]); margin = min(margin, float(r["margin"].min()))
    return cur, np.stack(sels), np.stack(wts), margin


def assert_close(y, ref, what=""):
    d = y.astype(np.float64) - ref.astype(np.float64)
    max_abs = np.abs(d).max()
    rel = np.linalg.norm(d) / max(np.linalg.norm(ref.astype(np.float64)), 1e-30)
    assert max_abs <= MAX_ABS and rel <= REL_L2, f"{what}: max-abs {max_abs:.3e} (<= {MAX_ABS}), rel-L2 {rel:.3e} (<= {REL_L2})"
    return max_abs, rel


def assert_same_experts(sel, rsel, wts, rwts, margin, tie=1e-6):
    """Prefill arithmetic (floating-point GEMMs whose summation order differs from the checker's):
    every token must pick the same SET of experts; the descending-probability order inside the
    set may differ from the checker's only between experts whose weights tie within `tie`."""
    assert np.array_equal(np.sort(sel, axis=-1), np.sort(rsel, axis=-1)), f"expert sets differ (min top-8/9 margin {margin:.3e})"
    swapped = sel != rsel
    if swapped.any():
        assert np.abs(np.sort(wts, axis=-1) - np.sort(rwts, axis=-1))[swapped.any(axis=-1)].max() <= tie
        assert np.abs(wts - rwts)[swapped].max() <= tie, "order inside the selection differs beyond a tie"
