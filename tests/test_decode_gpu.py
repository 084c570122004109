"""GPU parity of the M=1 decode path (through the C ABI) against the CPU checker."""
import numpy as np
import pytest

import orc
from gpu_common import assert_close, make_stack, oracle_stack

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cfg,n_layers,rand_norms", [(orc.TINY, 1, False), (orc.TINY, 3, True),
                                                     (orc.SMALL, 1, True), (orc.SMALL, 4, True)])
def test_decode_small_geometries(cfg, n_layers, rand_norms):
    eng, host = make_stack(cfg, n_layers, seed=7, rand_norms=rand_norms)
    rng = np.random.default_rng(3)
    for trial in range(4):
        x = rng.standard_normal((1, cfg["E"])).astype(np.float32)
        y, sel, wts = eng.forward(x)
        ry, rsel, rwts, margin = oracle_stack(cfg, host, x, orc.ORC_A if hasattr(orc, "ORC_A") else 0)
        assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
        np.testing.assert_allclose(wts, rwts, rtol=1e-6, atol=1e-7)
        assert_close(y, ry, f"{cfg} x{n_layers} trial {trial}")
    eng.close()


def test_decode_gemma_geometry_one_layer():
    cfg = orc.GEMMA
    eng, host = make_stack(cfg, 1, seed=0)
    rng = np.random.default_rng(0)
    for trial in range(3):
        x = rng.standard_normal((1, cfg["E"])).astype(np.float32)
        if trial == 0:       # the single-layer configuration RMS-norms its input once
            x = x / np.sqrt((x * x).mean() + 1e-6)
        y, sel, wts = eng.forward(x)
        ry, rsel, rwts, margin = oracle_stack(cfg, host, x, 0)
        assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
        assert_close(y, ry, f"gemma 1 layer trial {trial}")
    eng.close()


def test_decode_gemma_geometry_stack_of_three():
    cfg = orc.GEMMA
    eng, host = make_stack(cfg, 3, seed=11, rand_norms=True)
    x = np.random.default_rng(5).standard_normal((1, cfg["E"])).astype(np.float32)
    y, sel, wts = eng.forward(x)
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, 0)
    assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
    assert_close(y, ry, "gemma 3 layers")
    # a sub-range of layers is the per-layer drop-in call (g4_ffn_block): layer 1 alone
    x1 = oracle_stack(cfg, host, x, 0, first=0, n=1)[0]
    y1, sel1, _ = eng.forward(x1, layer_first=1, n_layers=1)
    r1 = oracle_stack(cfg, host, x1, 0, first=1, n=1)
    assert np.array_equal(sel1, r1[1])
    assert_close(y1, r1[0], "gemma layer 1 alone")
    eng.close()


def test_quantiser_matches_checker_bitwise():
    import torch
    from kairos_engine_b200 import q4b_dequantize, q4b_quantize
    g = torch.Generator(device="cuda").manual_seed(1)
    w = torch.randn((257, 704), generator=g, device="cuda") * 0.02
    w[3, :32] = 0.0                                    # an all-zero block: scale 0, codes 0
    codes, bs = q4b_quantize(w)
    rc, rbs = orc.q4b_quantize(w.cpu().numpy())
    assert np.array_equal(codes.cpu().numpy(), rc)
    assert np.array_equal(bs.cpu().numpy().view(np.uint16), rbs)
    deq = q4b_dequantize(codes, bs).cpu().numpy()
    assert np.array_equal(deq, orc.q4b_dequantize(rc, rbs))
    assert np.abs(deq - w.cpu().numpy()).max() <= 0.02 * 6 / 7 / 2 * 1.01 + 1e-6


def test_router_nan_is_reported_not_silent():
    from kairos_engine_b200 import SpMoeError
    cfg = orc.TINY
    eng, host = make_stack(cfg, 1, seed=2)
    x = np.full((1, cfg["E"]), np.nan, np.float32)
    with pytest.raises(SpMoeError) as ei:
        eng.forward(x)
    assert "NaN" in str(ei.value)
    # the handle stays usable afterwards
    x = np.random.default_rng(1).standard_normal((1, cfg["E"])).astype(np.float32)
    y, sel, _ = eng.forward(x)
    ry, rsel, _, _ = oracle_stack(cfg, host, x, 0)
    assert np.array_equal(sel, rsel)
    assert_close(y, ry, "after NaN")
    eng.close()


def test_gelu_is_bit_identical_to_checker():
    import torch
    from kairos_engine_b200 import gelu_mul
    g = torch.Generator(device="cuda").manual_seed(4)
    x = torch.cat([torch.randn(200000, generator=g, device="cuda") * 3,
                   torch.linspace(-12, 12, 100001, device="cuda"),
                   torch.tensor([0.0, -0.0, 0.55, -0.55, 9.01, 30.0, -30.0, 1e-30], device="cuda")])
    up = torch.randn(x.numel(), generator=g, device="cuda")
    got = gelu_mul(x, up).cpu().numpy()
    xs, us = x.cpu().numpy(), up.cpu().numpy()
    L = orc.lib()
    ref = np.array([L.orc_gelu_mul(float(a), float(b)) for a, b in zip(xs[::7], us[::7])], np.float32)
    assert np.array_equal(got[::7].view(np.uint32), ref.view(np.uint32))


def test_gemv_q4b_entry_matches_checker_bitwise():
    import torch
    from kairos_engine_b200 import gemv_q4b, q4b_quantize
    g = torch.Generator(device="cuda").manual_seed(9)
    for rows, cols in ((1408, 2816), (2816, 704), (33, 64)):
        w = torch.randn((rows, cols), generator=g, device="cuda") * 0.02
        codes, bs = q4b_quantize(w)
        x = torch.randn(cols, generator=g, device="cuda")
        y = gemv_q4b(codes, bs, x).cpu().numpy()
        qx, sx = orc.quant_act(x.cpu().numpy())
        ref = orc.gemv_a(codes.cpu().numpy(), bs.cpu().numpy().view(np.uint16), rows, cols, qx, sx)
        assert np.array_equal(y.view(np.uint32), ref.view(np.uint32))


@pytest.mark.parametrize("cfg,n_layers", [(orc.SMALL, 4), (orc.GEMMA, 2)])
def test_decode_direct_rows_path(cfg, n_layers, monkeypatch):
    """SP_MOE_DECODE_IMPL=direct: the kernels that read weight rows straight from global memory (the
    path for geometries whose per-CTA slices do not fit shared memory). Same checker, and bit-identical
    to the default path that stages rows through shared memory."""
    x = np.random.default_rng(23).standard_normal((1, cfg["E"])).astype(np.float32)
    monkeypatch.setenv("SP_MOE_DECODE_IMPL", "direct")
    eng, host = make_stack(cfg, n_layers, seed=13, rand_norms=True)
    monkeypatch.delenv("SP_MOE_DECODE_IMPL")
    y, sel, wts = eng.forward(x)
    eng.close()
    ry, rsel, rwts, margin = oracle_stack(cfg, host, x, 0)
    assert np.array_equal(sel, rsel), f"expert ids differ (min margin {margin:.3e})"
    assert_close(y, ry, "direct rows path")
    eng2, _ = make_stack(cfg, n_layers, seed=13, rand_norms=True)
    y2, sel2, wts2 = eng2.forward(x)
    eng2.close()
    assert np.array_equal(sel2, sel) and np.array_equal(wts2.view(np.uint32), wts.view(np.uint32))
    assert np.array_equal(y2.view(np.uint32), y.view(np.uint32))


def test_bounded_wait_that_runs_out_is_reported_and_survivable():
    """A device-side wait that can never be satisfied gives up after its poll limit, the kernel returns,
    and the host reads the timeout through the status call; the handle keeps working."""
    from kairos_engine_b200 import SpMoeError
    cfg = orc.TINY
    eng, host = make_stack(cfg, 1, seed=3)
    eng.debug_wait_timeout(polls=2000)
    with pytest.raises(SpMoeError) as ei:
        eng.status()
    assert ei.value.code == -40 and "bounded device-side wait ran out" in ei.value.text
    eng.status()                                       # the error word was cleared
    x = np.random.default_rng(2).standard_normal((1, cfg["E"])).astype(np.float32)
    y, sel, _ = eng.forward(x)
    ry, rsel, _, _ = oracle_stack(cfg, host, x, 0)
    assert np.array_equal(sel, rsel)
    assert_close(y, ry, "after a timed-out wait")
    eng.close()


def test_decode_phase_timing_entry(monkeypatch):
    from kairos_engine_b200 import SpMoeError
    cfg = orc.SMALL
    eng, _ = make_stack(cfg, 2, seed=4)
    with pytest.raises(SpMoeError):                    # not switched on: no clock is read, the call says so
        eng.decode_timing()
    eng.close()
    monkeypatch.setenv("SP_MOE_TIMING", "1")
    eng, _ = make_stack(cfg, 2, seed=4)
    monkeypatch.delenv("SP_MOE_TIMING")
    x = np.random.default_rng(2).standard_normal((1, cfg["E"])).astype(np.float32)
    eng.forward(x)
    t = eng.decode_timing()
    assert 0.0 < t["layer_us"] < 1e4
    for k in t["kernels"].values():
        assert k["wait_us"] >= 0.0 and k["prologue_us"] > 0.0 and k["rows_us"] >= 0.0
    eng.close()


def test_reupload_with_and_without_bias_drops_the_captured_graph():
    """A captured decode graph holds the layer's view by value; uploading the layer again with a router
    bias it lacked (or without one it had) must take effect on the next call."""
    import torch
    from kairos_engine_b200 import MoeEngine, synth
    cfg = orc.SMALL
    eng = MoeEngine(n_layers=1, **cfg)
    layer = synth.make_layer(cfg, 5)
    eng.upload_layer(0, layer, on_device=True)
    x = np.random.default_rng(8).standard_normal((1, cfg["E"])).astype(np.float32)
    y0, sel0, _ = eng.forward(x)
    biased = dict(layer); biased["router_bias"] = synth.zipf_bias(cfg["NE"], s=2.0, seed=1) * 8.0
    eng.upload_layer(0, biased, on_device=True)
    y1, sel1, _ = eng.forward(x)
    ref = orc.layer_forward(cfg, orc.LayerWeights(**synth.layer_to_host(biased)), x, 0)
    assert np.array_equal(sel1[0], ref["sel"]) and not np.array_equal(sel1, sel0)
    eng.upload_layer(0, layer, on_device=True)
    y2, sel2, _ = eng.forward(x)
    assert np.array_equal(sel2, sel0) and np.array_equal(y2.view(np.uint32), y0.view(np.uint32))
    eng.close()


def test_handles_on_two_devices_in_one_process():
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    from kairos_engine_b200 import MoeEngine, synth
    cfg = orc.SMALL
    x = np.random.default_rng(3).standard_normal((1, cfg["E"])).astype(np.float32)
    outs = []
    for dev in (0, 1):
        with torch.cuda.device(dev):
            eng = MoeEngine(n_layers=2, device=dev, **cfg)
            for L in range(2):
                eng.upload_layer(L, synth.make_layer(cfg, 30 + L, device=f"cuda:{dev}"), on_device=True)
            outs.append(eng.forward(x)[0])
            eng.close()
    assert np.array_equal(outs[0].view(np.uint32), outs[1].view(np.uint32))
