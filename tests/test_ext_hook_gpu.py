"""The MoE plugin hook (SwiGLU experts, separate gate/up/down tensors, host-chosen experts) against
the CPU checker's quantiser + Q4B GEMV composed the way the reference's hook composes them
(src/backends/cuda/cuda_forward.cu:16257-16289)."""
import numpy as np
import pytest

import orc
from gpu_common import MAX_ABS, REL_L2

pytestmark = pytest.mark.gpu


def _q4b(rng, rows, cols, std=0.05):
    w = (rng.standard_normal((rows, cols)) * std).astype(np.float32)
    return orc.q4b_quantize(w)


def _reference(x, idx, wt, g, gs, u, us, d, ds, E, FF):
    y = np.zeros(E, np.float32)
    qx, sx = orc.quant_act(x)
    for k, e in enumerate(idx):
        gv = orc.gemv_a(g[e], gs[e], FF, E, qx, sx)
        uv = orc.gemv_a(u[e], us[e], FF, E, qx, sx)
        h = ((gv / (np.float32(1.0) + np.exp(-gv, dtype=np.float32))) * uv).astype(np.float32)
        qh, sh = orc.quant_act(h)
        de = orc.gemv_a(d[e], ds[e], E, FF, qh, sh)
        y = (np.float32(wt[k]) * de + y).astype(np.float32)
    return y


@pytest.mark.parametrize("E,FF,NE,NU", [(128, 64, 6, 2), (2048, 512, 16, 8)])       # the second is the qwen36 expert shape
def test_hook_matches_checker_and_says_not_mine(E, FF, NE, NU):
    from kairos_engine_b200 import MoeExt
    rng = np.random.default_rng(E)
    g, gs, u, us, d, ds = [], [], [], [], [], []
    for e in range(NE):
        c, s = _q4b(rng, FF, E); g.append(c); gs.append(s)
        c, s = _q4b(rng, FF, E); u.append(c); us.append(s)
        c, s = _q4b(rng, E, FF); d.append(c); ds.append(s)
    ext = MoeExt()
    ext.upload_experts("blk.3.ffn_gate_exps.weight", np.stack(g), np.stack(gs), np.stack(u), np.stack(us), np.stack(d), np.stack(ds), NE, FF, E)
    x = rng.standard_normal(E).astype(np.float32)
    idx = rng.choice(NE, NU, replace=False).astype(np.int32)
    wt = rng.random(NU).astype(np.float32); wt /= wt.sum()
    y = ext.moe("blk.3.ffn_gate_exps.weight", idx, wt, x, FF)
    ref = _reference(x, idx, wt, g, gs, u, us, d, ds, E, FF)
    diff = y.astype(np.float64) - ref
    # tolerance of the parity gate (silu goes through expf, which CPU and GPU round differently)
    assert np.abs(diff).max() <= MAX_ABS and np.linalg.norm(diff) / np.linalg.norm(ref) <= REL_L2
    assert ext.moe("blk.4.ffn_gate_exps.weight", idx, wt, x, FF) is None           # unknown tag: not mine
    assert ext.moe("blk.3.ffn_gate_exps.weight", idx, wt, x, FF * 2) is None       # other shape: not mine
    ext.close()
