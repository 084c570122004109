"""CPU tests of the checker itself: pinned against the reference's own CPU expert code
(oracle/_ref, built from the reference tree in place) and against committed golden vectors."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _bench_inputs(seed, E=2816, FFE=704):
    """The reference micro-benches' own distribution (tools/moe_cpu_bench/moe_cpu_bench.cu:211-226):
    random nibbles, scales f16(0.004*(1+0.3|N(0,1)|)), x ~ N(0,1) with 8 entries x25."""
    r = np.random.default_rng(seed)
    gc = r.integers(0, 256, (2 * FFE, E // 2), dtype=np.uint8)
    dc = r.integers(0, 256, (E, FFE // 2), dtype=np.uint8)
    gs = (0.004 * (1 + 0.3 * np.abs(r.standard_normal((2 * FFE, E // 32))))).astype(np.float16).view(np.uint16)
    ds = (0.004 * (1 + 0.3 * np.abs(r.standard_normal((E, FFE // 32))))).astype(np.float16).view(np.uint16)
    x = r.standard_normal(E).astype(np.float32)
    x[r.integers(0, E, 8)] *= 25.0
    return gc, gs, dc, ds, x


def _ref_or_skip():
    R = orc.ref_lib()
    if R is None:
        pytest.skip("oracle/_ref not built or CPU lacks AVX-512 VNNI")
    return R


@pytest.mark.parametrize("seed", [1234, 1, 2])
def test_quant_and_gemv_bitwise_vs_reference_cpu_code(seed):
    """moe_exact_bench.cu:121-149's acceptance: int8 codes and scales identical, gate_up and down
    GEMV bitwise identical — here between the restatement and the reference's own file."""
    R = _ref_or_skip()
    E, FFE = 2816, 704
    gc, gs, dc, ds, x = _bench_inputs(seed)
    qx, sx = orc.quant_act(x)
    rq, rs = np.empty(E, np.int8), np.empty(E // 16, np.float32)
    assert R.sp_moe_cpu_quant(orc.p(x, orc.f32p), E, orc.p(rq, orc.i8p), orc.p(rs, orc.f32p)) == 0
    assert np.array_equal(rq, qx) and np.array_equal(rs.view(np.uint32), sx.view(np.uint32))
    y = orc.gemv_a(gc, gs, 2 * FFE, E, qx, sx)
    ry = np.empty(2 * FFE, np.float32)
    assert R.sp_moe_cpu_gemv(orc.p(gc, orc.u8p), orc.p(gs, orc.u16p), E, 2 * FFE, orc.p(qx, orc.i8p), orc.p(sx, orc.f32p), orc.p(ry, orc.f32p)) == 0
    assert np.array_equal(ry.view(np.uint32), y.view(np.uint32))
    h = np.array([orc.lib().orc_gelu_mul(float(y[i]), float(y[FFE + i])) for i in range(FFE)], np.float32)
    qh, sh = orc.quant_act(h)
    o = orc.gemv_a(dc, ds, E, FFE, qh, sh)
    ro = np.empty(E, np.float32)
    assert R.sp_moe_cpu_gemv(orc.p(dc, orc.u8p), orc.p(ds, orc.u16p), FFE, E, orc.p(qh, orc.i8p), orc.p(sh, orc.f32p), orc.p(ro, orc.f32p)) == 0
    assert np.array_equal(ro.view(np.uint32), o.view(np.uint32))
    # whole expert through the reference's v1 path (libm tanhf, different float order): relL2 ~2e-7
    re = np.empty(E, np.float32)
    assert R.sp_moe_cpu_expert(orc.p(x, orc.f32p), E, FFE, orc.p(gc, orc.u8p), orc.p(gs, orc.u16p),
                               orc.p(dc, orc.u8p), orc.p(ds, orc.u16p), orc.p(re, orc.f32p)) == 0
    assert np.linalg.norm(re - o) / np.linalg.norm(o) < 2e-6


def test_tanh_within_two_ulp_of_libm():
    L = orc.lib()
    ys = np.concatenate([np.linspace(-10, 10, 40001), np.linspace(-0.6, 0.6, 20001),
                         np.random.default_rng(0).standard_normal(20000) * 2]).astype(np.float32)
    got = np.array([L.orc_tanhf(float(v)) for v in ys], np.float64)
    ref = np.tanh(ys.astype(np.float64))
    ulp = np.spacing(np.abs(ref).astype(np.float32)).astype(np.float64)
    assert (np.abs(got - ref) / ulp).max() <= 2.0
    assert L.orc_tanhf(0.0) == 0.0 and L.orc_tanhf(40.0) == 1.0 and L.orc_tanhf(-40.0) == -1.0
    assert np.isnan(L.orc_tanhf(float("nan")))


def test_half_conversions_match_numpy():
    L = orc.lib()
    hs = np.arange(0, 65536, 7, dtype=np.uint32).astype(np.uint16)
    ref = hs.view(np.float16).astype(np.float32)
    got = np.array([L.orc_half_to_float(int(h)) for h in hs], np.float32)
    ok = ~np.isnan(ref)
    assert np.array_equal(got[ok].view(np.uint32), ref[ok].view(np.uint32))
    fs = (np.random.default_rng(0).standard_normal(5000) * np.logspace(-8, 5, 5000)).astype(np.float32)
    assert np.array_equal(np.array([L.orc_float_to_half(float(f)) for f in fs], np.uint16), fs.astype(np.float16).view(np.uint16))


def test_topk_semantics():
    # descending p, strict > so ties keep the lower id (CF:6229); renormalised weights sum to 1
    lg = np.zeros(16, np.float32); lg[[3, 9, 12]] = [2.0, 2.0, 1.0]
    rc, idx, wt = orc.topk(lg, 4)
    assert rc == 0 and list(idx) == [3, 9, 12, 0]
    assert abs(wt.sum() - 1.0) < 1e-6 and wt[0] == wt[1]
    lg[5] = np.nan                                      # a NaN row is a hard error (CF:8596-8620)
    assert orc.topk(lg, 4)[0] == -1
    # the clamp (CF:6237): selected probabilities that underflow to 0 divide by 2^-14, not by 0
    lg = np.full(8, -200.0, np.float32); lg[0] = 200.0
    rc, idx, wt = orc.topk(lg, 2)
    assert rc == 0 and idx[0] == 0 and wt[0] == 1.0 and wt[1] == 0.0


def test_q4b_quantiser_recipe():
    r = np.random.default_rng(0)
    w = (r.standard_normal((33, 256)) * 0.02).astype(np.float32)
    w[5, 32:64] = 0.0
    codes, bs = orc.q4b_quantize(w)
    deq = orc.q4b_dequantize(codes, bs)
    nib = np.stack([codes & 0xF, codes >> 4], -1).reshape(33, 256).astype(np.int32)
    code = (nib ^ 8) - 8
    assert code.min() >= -7 and code.max() <= 7
    s = bs.view(np.float16).astype(np.float32)
    assert np.array_equal(deq, code.astype(np.float32) * np.repeat(s, 32, axis=1))     # w = code * f16 scale exactly
    assert np.all(np.abs(deq - w) <= np.repeat(s, 32, axis=1) * 0.5 + 1e-9)
    assert np.all(deq[5, 32:64] == 0)


def test_layer_flavours_agree_and_routing_matches():
    cfg = orc.SMALL
    w = orc.make_layer(cfg, 0, rand_norms=True)
    x = np.random.default_rng(1).standard_normal((6, cfg["E"])).astype(np.float32)
    a, b = orc.layer_forward(cfg, w, x, 0, True), orc.layer_forward(cfg, w, x, 1, True)
    assert a["rc"] == 0 and b["rc"] == 0
    assert np.array_equal(a["sel"], b["sel"])            # the router does not depend on the matmul flavour
    assert np.linalg.norm(a["y"] - b["y"]) / np.linalg.norm(b["y"]) < 2e-2   # int8 activations: ~1e-2, by construction (CF:13808-13814)
    assert np.all(a["margin"] > 0)
    # ids are the top-NU of the logits
    for t in range(6):
        assert set(np.argsort(-a["logits"][t], kind="stable")[: cfg["NU"]]) == set(a["sel"][t])


def test_layer_empty_and_nan_inputs():
    cfg = orc.TINY
    w = orc.make_layer(cfg, 3)
    assert orc.layer_forward(cfg, w, np.zeros((0, cfg["E"]), np.float32))["y"].shape == (0, cfg["E"])
    z = orc.layer_forward(cfg, w, np.zeros((1, cfg["E"]), np.float32))      # all-zero row: scale path m == 0 -> 1.0
    assert z["rc"] == 0 and np.all(np.isfinite(z["y"]))
    assert orc.layer_forward(cfg, w, np.full((1, cfg["E"]), np.nan, np.float32))["rc"] == -1


def test_int_gemm_scaled_matches_numpy():
    r = np.random.default_rng(0)
    M, N, K = 16, 24, 64
    A = r.integers(-8, 8, (M, K)).astype(np.int8); B = r.integers(-8, 8, (N, K)).astype(np.int8)
    sa = (0.5 + r.integers(0, 256, M) / 512).astype(np.float32); sb = (0.5 + r.integers(0, 256, N) / 512).astype(np.float32)
    Cc = np.empty((M, N), np.uint16)
    orc.lib().orc_int_gemm_scaled(orc.p(A, orc.i8p), orc.p(B, orc.i8p), M, N, K, orc.p(sa, orc.f32p), orc.p(sb, orc.f32p), orc.p(Cc, orc.u16p))
    ref = ((A.astype(np.int32) @ B.astype(np.int32).T).astype(np.float32) * sa[:, None] * sb[None, :]).astype(np.float16)
    assert np.array_equal(Cc, ref.view(np.uint16))


# ---- committed golden vectors (generated by tests/golden/make_golden.py from this checker; they
# ---- freeze its behaviour so a later edit cannot drift unnoticed, and travel to machines
# ---- without the reference tree)
@pytest.mark.parametrize("name", ["tiny_A", "tiny_B", "small_A", "small_B"])
def test_golden_layer_vectors(name):
    path = os.path.join(GOLDEN, f"layer_{name}.npz")
    g = np.load(path)
    meta = json.loads(str(g["meta"]))
    cfg = meta["cfg"]
    w = orc.make_layer(cfg, meta["seed"], rand_norms=True)
    r = orc.layer_forward(cfg, w, g["x"], meta["flavour"], True)
    assert np.array_equal(r["sel"], g["sel"])
    assert np.array_equal(r["y"].view(np.uint32), g["y"].view(np.uint32))
    assert np.array_equal(r["wts"].view(np.uint32), g["wts"].view(np.uint32))


def test_golden_reference_expert_vectors():
    """Outputs of the reference's own moe_cpu_expert.c recorded in this container
    (tests/golden/make_golden.py); the restatement must keep reproducing them."""
    _ref_or_skip()
    g = np.load(os.path.join(GOLDEN, "ref_expert.npz"))
    gc, gs, dc, ds, x = _bench_inputs(int(g["seed"]))
    qx, sx = orc.quant_act(x)
    assert np.array_equal(qx, g["qx"]) and np.array_equal(sx.view(np.uint32), g["sx"].view(np.uint32))
    y = orc.gemv_a(gc, gs, 2 * 704, 2816, qx, sx)
    assert np.array_equal(y.view(np.uint32), g["gate_up"].view(np.uint32))


def test_golden_reference_expert_vectors_without_ref_lib():
    """Same fixture, checked without loading oracle/_ref (machines without AVX-512 VNNI)."""
    g = np.load(os.path.join(GOLDEN, "ref_expert.npz"))
    gc, gs, dc, ds, x = _bench_inputs(int(g["seed"]))
    qx, sx = orc.quant_act(x)
    assert np.array_equal(qx, g["qx"])
    y = orc.gemv_a(gc, gs, 2 * 704, 2816, qx, sx)
    assert np.array_equal(y.view(np.uint32), g["gate_up"].view(np.uint32))
    hq, hs = g["hq"], g["hs"]
    o = orc.gemv_a(dc, ds, 2816, 704, hq, hs)
    assert np.array_equal(o.view(np.uint32), g["down"].view(np.uint32))
