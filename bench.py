#!/usr/bin/env python
"""bench.py — MoE-FFN decode throughput of the 30-layer Gemma-4-26B-A4B-geometry stack on B200.

Workload (N=1 default): the full 30-layer MoE FFN stack, decode M=1, all 30*128 experts resident
in HBM, random-init Q4B weights (router N(0,0.02) f32; expert/shared weights N(0,0.02) then Q4B),
seeded N(0,1) hidden states. One bench STEP = 256 sequential single-token decode steps through
all 30 layers. `value` = tokens/s with inputs resident in HBM, timed with CUDA events on the
launching stream; `e2e` = the same through the host-pointer C-ABI call (H2D of the token's hidden
state and D2H of the result inside the timed region, every token). N>1 runs N independent
replicas for the decode metric (decode does not shard); the expert-parallel prefill, which does,
is reported in the `prefill` object, and the load-imbalance stress in `zipf`.

Beside the headline the line carries: `parity` (results checked against the CPU checker and
against the library's own second path, outside every timed region), `prefill`, `small_batch`
(M = 4..64 in the decode arithmetic, roofline with the measured number of distinct experts),
`prefill_terms` (the opt-in 2- and 1-term GEMM modes beside the exact default), `int_gemm`,
`cpu_baseline`, `ref_gpu_kernels` (the reference's own decode kernels, compiled for this GPU, timed
on the same shapes); at N>1 `zipf` and `ep_stage_times` (CUDA-event times of the stages of one
expert-parallel layer: route, dispatch, experts, combine, finish).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

--impl reference times the reference's own CPU expert code (oracle/_ref: moe_cpu_expert.c compiled
in place, with the restated layer glue around it) on this host's cores on a bounded sample.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(E=2816, NE=128, NU=8, FFE=704, FFS=2112, eps=1e-6)
N_LAYERS = 30
TOKENS_PER_STEP = 256
FALLBACK_HBM_GBS = 6650.0
# dram__bytes_read.sum + dram__bytes_write.sum of the three decode kernels of one layer, from one ncu capture of a
# 2-layer stack (six launches = one token; L2 flushed before each kernel, prefetch hints off):
#   SP_MOE_STAGED_FLAGS=8 ncu --metrics dram__bytes_read.sum,dram__bytes_write.sum --clock-control none -k regex:k_ds_ -s 18 -c 6
#       python bench.py --steps 1 --warmup 3 --tokens-per-step 1 --layers 2 --no-cpu --no-prefill
# 38,520,832 B per layer against 38,331,904 algorithmic; the traffic is the same for every layer, so a launch is 30x that.
NCU_TRAFFIC_BYTES_PER_LAYER = 38520832


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), float(d.get("bf16_tflops_sustained", 0.0)) or None, "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, 1400.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled every 200 ms while the timed region runs."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.proc, self.lines = index, None, []

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=lambda: self.lines.extend(self.proc.stdout), daemon=True)
            self.t.start()
        except Exception:
            self.proc = None
        return self

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.25)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            self.t.join(timeout=2)

    def summary(self):
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [c.strip() for c in ln.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------- CPU legs (the checker / the reference's CPU code)
def _orc():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import orc
    return orc


def random_q4b(rng, rows, cols):
    """Valid Q4B bytes drawn directly (codes in [-7, 7] as two's-complement nibbles, f16 block scales around
    0.02 * 3 / 7): the CPU arm's time does not depend on the values, and no quantiser has to run."""
    import numpy as np
    v = rng.integers(-7, 8, size=(rows, cols), dtype=np.int8)
    codes = ((v[:, 0::2] & 0xF) | ((v[:, 1::2] & 0xF) << 4)).astype(np.uint8)
    bs = rng.uniform(0.004, 0.012, size=(rows, cols // 32)).astype(np.float16).view(np.uint16)
    return np.ascontiguousarray(codes), np.ascontiguousarray(bs)


def cpu_layers_random(n_pool):
    """n_pool layers of the benchmark geometry built on the CPU alone (the reference arm must not need the product)."""
    import numpy as np
    orc = _orc()
    E, NE, FFE, FFS = CFG["E"], CFG["NE"], CFG["FFE"], CFG["FFS"]
    out = []
    for L in range(n_pool):
        r = np.random.default_rng(1000 * L)
        one = lambda n: np.ones(n, np.float32)
        gu_c, gu_s = random_q4b(r, NE * 2 * FFE, E); dn_c, dn_s = random_q4b(r, NE * E, FFE)
        sg_c, sg_s = random_q4b(r, FFS, E); su_c, su_s = random_q4b(r, FFS, E); sd_c, sd_s = random_q4b(r, E, FFS)
        out.append(orc.LayerWeights(router_w=(r.standard_normal((NE, E)) * 0.02).astype(np.float32), router_scale=one(E), router_bias=None,
                                    ffn_norm=one(E), post_ffw1=one(E), pre_ffw2=one(E), post_ffw2=one(E), post_ffw=one(E), dexps_scale=one(NE),
                                    gu_codes=gu_c, gu_bs=gu_s, dn_codes=dn_c, dn_bs=dn_s, sg_codes=sg_c, sg_bs=sg_s, su_codes=su_c, su_bs=su_s,
                                    sd_codes=sd_c, sd_bs=sd_s))
    return out


def cpu_time_tokens(layers, n_tokens, threads, seed=0):
    """Runs n_tokens single-token passes of the 30-layer stack on the CPU, cycling the layer pool
    (weights stay cold: the pool is far larger than the last-level cache). Returns (seconds, kind)."""
    import numpy as np
    orc = _orc()
    kind = orc.use_reference_gemv(threads)
    rng = np.random.default_rng(seed)
    t0 = time.perf_counter()
    for t in range(n_tokens):
        x = rng.standard_normal((1, CFG["E"])).astype(np.float32)
        for L in range(N_LAYERS):
            x = orc.layer_forward(CFG, layers[L % len(layers)], x, 0)["y"]
    return time.perf_counter() - t0, kind


def run_reference(args, rank, world):
    if rank != 0:                                      # rank 0 alone runs the CPU arm; the others leave without work
        return
    threads = min(os.cpu_count() or 1, 16)            # the reference pool's cap (moe_cpu_expert.c:225)
    layers = cpu_layers_random(4)
    tok = 1                                            # one step = one token through 30 layers
    for _ in range(args.warmup):
        cpu_time_tokens(layers, tok, threads)
    secs, kind = cpu_time_tokens(layers, tok * args.steps, threads, seed=1)
    v = tok * args.steps / secs
    sample = f"{tok} token x 30 layers per step, {args.steps} steps, layer pool of 4 cycled (cold weights), random valid Q4B bytes built on the CPU"
    line = {"impl": "reference", "metric": "MoE-FFN decode tokens/s (30-layer stack, M=1)", "value": v, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 activations x int4 weights, f32 accumulate",
            "data": "synthetic", "config": {"workload": "configs[1]: 30-layer MoE FFN stack, decode M=1", "cpu_sample": sample},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def cpu_baseline_leg(eng, torch):
    """The CPU arm on this host's cores (bounded sample) and, in the same leg, the checker compared with the
    library on the benchmark's own weights: 4 tokens through the first 3 layers, ids and hidden state bit for bit."""
    import numpy as np
    from kairos_engine_b200 import synth
    orc = _orc()
    threads = min(os.cpu_count() or 1, 16)
    layers = []
    for L in range(3):                                 # the very layers 0..2 the engine holds (same seeds, same quantiser)
        layer = synth.make_layer(CFG, 1000 * L)
        layers.append(orc.LayerWeights(**synth.layer_to_host(layer)))
        del layer
    torch.cuda.empty_cache()
    parity = {"checked": "4 tokens x layers 0..2 of the benchmark stack against the CPU checker", "ids_exact": True, "bit_identical": True, "max_abs": 0.0}
    orc.use_port_gemv()
    rng = np.random.default_rng(123)
    for t in range(4):
        x = rng.standard_normal((1, CFG["E"])).astype(np.float32)
        y, sel, _ = eng.forward(x, 0, 3)
        cur, ok = x, True
        for L in range(3):
            r = orc.layer_forward(CFG, layers[L], cur, 0)
            ok = ok and bool(np.array_equal(r["sel"], sel[L]))
            cur = r["y"]
        parity["ids_exact"] = parity["ids_exact"] and ok
        parity["bit_identical"] = parity["bit_identical"] and bool(np.array_equal(cur.view(np.uint32), y.view(np.uint32)))
        parity["max_abs"] = max(parity["max_abs"], float(np.abs(cur - y).max()))
    cpu_time_tokens(layers, 1, threads)
    n_tok = 192
    secs, kind = cpu_time_tokens(layers, n_tok, threads, seed=1)
    base = {"value": n_tok / secs, "unit": "tokens/s", "cores": threads, "kind": kind,
            "sample": f"{n_tok} tokens x 30 layers, layer pool of 3 cycled (cold weights), {secs:.1f} s"}
    return base, parity


def ref_gpu_leg(local_rank, torch):
    """The reference's own decode kernels (tools/moe_cpu_bench/moe_cpu_bench.cu, compiled for this GPU into
    oracle/_ref by `make -C oracle ref_gpu`): one token's routed branch of one layer = 8 experts x 5 launches, cold
    weights (a pool of 512 experts = 1.7 GB walked round-robin), timed with CUDA events."""
    so = os.path.join(ROOT, "oracle", "_ref", "libsp_ref_gpu.so")
    if not os.path.exists(so):
        return {"unavailable": "oracle/_ref/libsp_ref_gpu.so was not built (the reference tree was not mounted at build time)"}
    R = C.CDLL(so)
    R.sp_ref_gpu_experts.argtypes = [C.c_void_p] * 8 + [C.c_int] + [C.c_void_p] * 6
    e, f = C.c_int(), C.c_int()
    R.sp_ref_gpu_geometry(C.byref(e), C.byref(f))
    E, FFE, NU, POOL = e.value, f.value, 8, 512
    dev = f"cuda:{local_rank}"
    g = torch.Generator(device=dev).manual_seed(5)
    gub, gusb, dwb, dwsb = 2 * FFE * (E // 2), 2 * FFE * (E // 32), E * (FFE // 2), E * (FFE // 32)
    gu_c = torch.randint(0, 256, (POOL * gub,), dtype=torch.uint8, device=dev, generator=g)
    dn_c = torch.randint(0, 256, (POOL * dwb,), dtype=torch.uint8, device=dev, generator=g)
    gu_s = (torch.rand(POOL * gusb, device=dev, generator=g) * 0.004 + 0.004).to(torch.float16).view(torch.int16)
    dn_s = (torch.rand(POOL * dwsb, device=dev, generator=g) * 0.004 + 0.004).to(torch.float16).view(torch.int16)
    ro_g = (torch.arange(2 * FFE, device=dev, dtype=torch.int64) * (E // 2)).contiguous()
    ro_d = (torch.arange(E, device=dev, dtype=torch.int64) * (FFE // 2)).contiguous()
    x = torch.randn(E, device=dev, generator=g)
    qx = torch.empty(E, dtype=torch.int8, device=dev); sx = torch.empty(E // 16, device=dev)
    gu = torch.empty(2 * FFE, device=dev); h = torch.empty(FFE, device=dev); out = torch.empty(NU * E, device=dev)
    layers = 60
    ids = [(C.c_int * NU)(*[(L * NU + k) % POOL for k in range(NU)]) for L in range(layers)]

    def one_pass():
        st = torch.cuda.current_stream().cuda_stream
        for L in range(layers):
            rc = R.sp_ref_gpu_experts(x.data_ptr(), gu_c.data_ptr(), gu_s.data_ptr(), dn_c.data_ptr(), dn_s.data_ptr(), ro_g.data_ptr(), ro_d.data_ptr(),
                                      C.cast(ids[L], C.c_void_p), NU, qx.data_ptr(), sx.data_ptr(), gu.data_ptr(), h.data_ptr(), out.data_ptr(), st)
            if rc:
                raise RuntimeError(f"reference kernel launch failed: cuda error {rc}")
    for _ in range(2):
        one_pass()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(); one_pass(); e1.record(); torch.cuda.synchronize()
    us_layer = e0.elapsed_time(e1) * 1e3 / layers
    bytes_layer = NU * (gub + dwb + 2 * (gusb + dwsb))
    # the same launches replayed from a CUDA graph: the kernels' own time, without the host's launch pace
    us_graph = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            one_pass()
        graph.replay(); torch.cuda.synchronize()
        e0.record(); graph.replay(); e1.record(); torch.cuda.synchronize()
        us_graph = e0.elapsed_time(e1) * 1e3 / layers
    except Exception:
        pass
    return {"what": "the reference's k_quant_act_int8 + k_gemv_q4b_dp4a_v2 + k_moe_gelu_split_batch as its served decode launches them, built for sm_100a",
            "us_per_layer_routed_branch": us_layer, "us_per_expert": us_layer / NU, "launches_per_layer": 5 * NU,
            "gbs": bytes_layer / (us_layer * 1e-6) / 1e9, "bytes_per_layer": bytes_layer,
            "graph_replay_us_per_layer_routed_branch": us_graph, "graph_replay_gbs": (bytes_layer / (us_graph * 1e-6) / 1e9) if us_graph else None,
            "note": "routed experts only (no router, shared expert, norms or combine), launched from the host like the reference's decode loop"}


# ---------------------------------------------------------------- batched decode / draft-verify shapes
def small_batch_leg(eng, NL, local_rank, rank, peak_gbs):
    """M in {4, 8, 16, 64} tokens per step through the stack in the single-token decode arithmetic
    (what M sequential decode steps compute), unbiased router: the union of active experts grows with M.
    roofline: algorithmic bytes with the MEASURED number of distinct experts per layer."""
    import torch
    from kairos_engine_b200 import FLAVOUR_DECODE, synth
    out = {}
    for M in (4, 8, 16, 64):
        if M > eng.max_tokens:
            continue
        x = synth.make_inputs(CFG, M, seed=300 + M + rank, device=f"cuda:{local_rank}")
        y = torch.empty_like(x)
        sel = torch.empty((NL, M, CFG["NU"]), dtype=torch.int32, device=x.device)
        eng.forward_dev(x, y, 0, NL, FLAVOUR_DECODE, sel=sel)
        eng.status()
        U = [int(torch.unique(sel[L]).numel()) for L in range(NL)]
        for _ in range(3):
            eng.forward_dev(x, y, 0, NL, FLAVOUR_DECODE)
        eng.status()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 5
        e0.record()
        for _ in range(reps):
            eng.forward_dev(x, y, 0, NL, FLAVOUR_DECODE)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / reps
        nbytes = sum(synth.algorithmic_bytes_per_layer(CFG, M=M, U=u) for u in U)
        gbs = nbytes / (ms / 1e3) / 1e9
        # second path: row 0 of the batch equals the single-token kernels' result for that token, bit for bit
        y1 = torch.empty_like(x[0])
        eng.forward_dev(x[0], y1, 0, NL, FLAVOUR_DECODE)
        eng.status()
        out[f"M={M}"] = {"tokens_per_s": M / (ms / 1e3), "ms_per_step": ms, "distinct_experts_per_layer_mean": sum(U) / len(U),
                         "roofline": {"bound": "hbm", "achieved": gbs, "peak": peak_gbs, "unit": "GB/s", "frac": gbs / peak_gbs, "algorithmic_bytes": nbytes},
                         "route": "token by token through the single-token graph" if M <= int(os.environ.get("SP_MOE_SEQ_TOKENS", "5")) else "batched kernels (mma.sync row dots)",
                         "row0_equals_single_token_step": bool(torch.equal(y1.view(torch.int32), y[0].view(torch.int32)))}
    return out


# ---------------------------------------------------------------- where an expert-parallel layer's time goes
def ep_stage_timing_leg(NL, PT, rank, local_rank, world, dist):
    """CUDA-event stage times of one expert-parallel layer (the library loop, padded exchange, run eagerly: events
    cannot be timed inside a graph replay). A second handle opened with SP_MOE_TIMING=1 carries the events, so the
    headline handle stays untimed. Reported: rank 0's last layer, and the slowest rank's whole layer."""
    import torch
    from kairos_engine_b200 import FLAVOUR_PREFILL, MoeEngine, ep, synth
    dev = f"cuda:{local_rank}"
    Ml = PT // world
    NLt = min(NL, 4)
    os.environ["SP_MOE_TIMING"] = "1"
    try:
        eng = MoeEngine(n_layers=NLt, max_tokens=Ml, device=local_rank, max_expert_rows=PT * CFG["NU"], **CFG)
    finally:
        del os.environ["SP_MOE_TIMING"]
    for L in range(NLt):
        layer = synth.make_layer(CFG, 1000 * L, device=dev)
        eng.upload_layer(L, layer, on_device=True)
        del layer
    x = synth.make_inputs(CFG, Ml, seed=99 + rank, device=dev)
    cap = -(-13 * Ml * CFG["NU"] // (10 * world) // 8) * 8
    epm = ep.NcclExpertParallel(eng, CFG, capacity_rows=cap, slices=1)
    for _ in range(3):
        epm.forward(x, 0, NLt, FLAVOUR_PREFILL)
    torch.cuda.synchronize()
    eng.status()
    tm = epm.timing()
    t = torch.tensor([tm["layer"]], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    epm.close()
    eng.close()
    torch.cuda.empty_cache()
    out = {k + "_ms": round(v, 4) for k, v in tm.items()}
    out["layer_ms_slowest_rank"] = round(float(t.item()), 4)
    out["exchanges_share_of_layer"] = round((tm["gather_dispatch"] + tm["combine"]) / tm["layer"], 3) if tm["layer"] > 0 else None
    out["note"] = ("last of %d layers, run eagerly (the timed pass above is a graph replay); gather_dispatch runs on the communication "
                   "stream with the shared expert under it, so experts_after_dispatch is what the compute stream still had to do" % NLt)
    return out


# ---------------------------------------------------------------- prefill with fewer MMA terms per k-step
def prefill_terms_leg(NL, PT, local_rank):
    """The same prefill pass with the weight rounded to fp16 (2 MMAs per k-step) and with the activation
    rounded too (1 MMA: the reference's SP_G4_GEMM_F16 mode), beside the exact 3-term default. The error is
    taken over ONE layer against the 3-term result (deeper stacks diverge through top-k flips of near-tied
    experts, which says nothing about the arithmetic)."""
    import torch
    from kairos_engine_b200 import FLAVOUR_PREFILL, MoeEngine, synth
    dev = f"cuda:{local_rank}"
    x = synth.make_inputs(CFG, PT, seed=90, device=dev)
    out, ref1 = {}, None
    for terms in (3, 2, 1):
        os.environ["SP_MOE_PREFILL_TERMS"] = str(terms)
        try:
            eng = MoeEngine(n_layers=NL, max_tokens=PT, device=local_rank, **CFG)
        finally:
            del os.environ["SP_MOE_PREFILL_TERMS"]
        for L in range(NL):
            layer = synth.make_layer(CFG, 1000 * L, device=dev)
            eng.upload_layer(L, layer, on_device=True)
            del layer
        y = torch.empty_like(x)
        y1 = torch.empty_like(x)
        eng.forward_dev(x, y1, 0, 1, FLAVOUR_PREFILL)
        for _ in range(2):
            eng.forward_dev(x, y, 0, NL, FLAVOUR_PREFILL)
        eng.status()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(3):
            eng.forward_dev(x, y, 0, NL, FLAVOUR_PREFILL)
        e1.record()
        torch.cuda.synchronize()
        eng.status()
        ms = e0.elapsed_time(e1) / 3
        rec = {"tokens_per_s": PT / (ms / 1e3), "ms_per_pass": ms}
        if ref1 is None:
            ref1 = y1.double()
        else:
            d = y1.double() - ref1
            rec["one_layer_rel_l2_vs_3_terms"] = float(d.norm() / ref1.norm())
            rec["one_layer_max_abs_vs_3_terms"] = float(d.abs().max())
        out[f"terms={terms}"] = rec
        eng.close()
        del eng, y, y1
        torch.cuda.empty_cache()
    out["switch"] = "SP_MOE_PREFILL_TERMS (read when a handle opens); 3 is the default and the headline"
    return out


# ---------------------------------------------------------------- the quantised (int8 x int8 -> f16) GEMM
def int_gemm_leg(local_rank):
    import torch
    from kairos_engine_b200.engine import int_gemm_scaled
    M = N = K = 8192
    dev = f"cuda:{local_rank}"
    g = torch.Generator(device=dev).manual_seed(11)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, device=dev, generator=g)
    B = torch.randint(-128, 128, (N, K), dtype=torch.int8, device=dev, generator=g)
    sa = torch.rand(M, device=dev, generator=g) * 1e-3
    sb = torch.rand(N, device=dev, generator=g) * 1e-3
    for _ in range(3):
        int_gemm_scaled(A, B, sa, sb)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = 10
    e0.record()
    for _ in range(reps):
        int_gemm_scaled(A, B, sa, sb)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / reps
    return {"shape": [M, N, K], "ms": ms, "tops": 2.0 * M * N * K / (ms / 1e3) / 1e12,
            "note": "tcgen05 kind::i8, int32 accumulate in TMEM, f16 out with per-row x per-column scales"}


# ---------------------------------------------------------------- prefill (reported beside the decode metric)
def prefill_leg(args, eng, NL, PT, rank, local_rank, world, dist, barrier, zipf=False):
    """PT tokens through the stack in the prefill arithmetic: one GPU runs them all; N GPUs run
    PT/N tokens each with the routed experts partitioned NE/N per GPU (all-to-all each way).
    zipf: the load-imbalance stress (the engine's routers carry a Zipf bias; exact exchange)."""
    import torch
    from kairos_engine_b200 import FLAVOUR_PREFILL, SpMoeError, ep, synth
    Ml = PT // world
    xp = synth.make_inputs(CFG, Ml, seed=99 + rank, device=f"cuda:{local_rank}")
    yp = torch.empty_like(xp)
    # N > 1: padded exchange (no host read per layer) with room for 1.3x the average rows per destination
    # (unbiased routing spreads within a few percent; an overflow on any rank sends all ranks to the exact
    # exchange); the load-imbalance stress uses the exact exchange
    cap = 0 if (world < 2 or zipf) else -(-13 * Ml * CFG["NU"] // (10 * world) // 8) * 8
    if world < 2:
        epm = None
    elif args.ep_impl == "torch":                      # the loop in Python over torch.distributed, stage by stage
        epm = ep.ExpertParallelMoe(eng, CFG, capacity_rows=cap)
    else:                                              # the loop inside the library: NCCL from C++, token slices pipelined
        epm = ep.NcclExpertParallel(eng, CFG, capacity_rows=cap, slices=args.ep_slices)

    def one_pass():
        if epm is None:
            eng.forward_dev(xp, yp, 0, NL, FLAVOUR_PREFILL)
            return yp
        return epm.forward(xp, 0, NL, FLAVOUR_PREFILL)

    def warm():
        for _ in range(2):
            one_pass()
        try:
            eng.status()
            return 1
        except SpMoeError:
            return 0

    ok = warm()
    if dist is not None:
        t = torch.tensor([ok], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = int(t.item())
    if not ok:
        if epm is None or epm.capacity == 0:
            raise RuntimeError("prefill warm-up reported a kernel error")
        epm.capacity = cap = 0                         # some destination overflowed its block on some rank: all ranks go exact
        if not warm():
            raise RuntimeError("prefill warm-up reported a kernel error")
    # ---- parity, outside the timed region: the expert-parallel result against this rank's own single-GPU pass
    # over the same tokens (every rank holds the whole arena), bit for bit; one GPU: a sub-batch against the full batch
    if epm is not None:
        got = one_pass().clone()
        want = torch.empty_like(xp)
        eng.forward_dev(xp, want, 0, NL, FLAVOUR_PREFILL)
        eng.status()
        same = bool(torch.equal(got.view(torch.int32), want.view(torch.int32)))
        what = "expert-parallel pass == this rank's single-GPU pass over its own tokens"
    else:
        full = one_pass().clone()
        sub = torch.empty_like(xp[: Ml // 8])
        eng.forward_dev(xp[: Ml // 8], sub, 0, NL, FLAVOUR_PREFILL)
        eng.status()
        same = bool(torch.equal(sub.view(torch.int32), full[: Ml // 8].view(torch.int32)))
        what = "rows of a one-eighth sub-batch == the same rows of the full batch (other tiles, other offsets)"
    finite = bool(torch.isfinite(yp if epm is None else got).all())
    if dist is not None:
        t = torch.tensor([int(same), int(finite)], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        same, finite = bool(t[0].item()), bool(t[1].item())
    barrier()
    passes = 3
    l0 = eng.kernel_launches
    one_pass()
    per_pass_launches = eng.kernel_launches - l0
    run, replayed = one_pass, False
    if epm is not None and epm.capacity > 0 and not args.no_ep_graph:
        # the padded exchange has no host read, so a whole pass (kernels + collectives) can be replayed from one
        # CUDA graph and the CPU stops pacing the ranks
        try:
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                epm.forward(xp, 0, NL, FLAVOUR_PREFILL)
            graph.replay()
            torch.cuda.synchronize()
            run, replayed = graph.replay, True
        except Exception as e:
            raise RuntimeError(f"CUDA-graph capture of the expert-parallel pass failed ({type(e).__name__}: {e}); rerun with --no-ep-graph")
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(passes):
        run()
    e1.record()
    barrier()
    eng.status()
    ms = e0.elapsed_time(e1)
    rows = float(epm.last_rows) if epm is not None else float(Ml * CFG["NU"])
    if dist is not None:
        t = torch.tensor([ms, rows, -rows], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, rows_max, rows_min = float(t[0]), float(t[1]), -float(t[2])
    else:
        rows_max = rows_min = rows
    flops = synth.flops_per_token_layer(CFG) * PT * NL * passes
    tf = flops / (ms / 1e3) / 1e12 / world
    peak_tf = measured_peaks()[1]
    return {"metric": "MoE-FFN prefill tokens/s (30-layer stack)", "value": PT * passes / (ms / 1e3), "unit": "tokens/s", "tokens": PT,
            "ms_per_pass": ms / passes, "passes": passes, "dtype": "f16 x f16 split operands (3 MMAs per k-step), f32 accumulate in TMEM",
            "parallelism": "single GPU" if world == 1 else f"expert-parallel: {PT // world} tokens and {CFG['NE'] // world} experts per GPU, all-to-all each way",
            "exchange": "none" if world == 1 else (f"padded: {cap} rows per destination, no host read per layer" if cap else "exact: split sizes read on the host once per layer"),
            "driver": "none" if world == 1 else ("torch.distributed loop over the stage entries" if args.ep_impl == "torch" else f"sp_moe_ep_forward_dev (NCCL called from the library, {args.ep_slices if cap else 1} token slice(s) in flight)"),
            "expert_rows_last_layer": {"max_per_gpu": rows_max, "min_per_gpu": rows_min, "mean_per_gpu": float(PT * CFG["NU"]) / world,
                                       "max_over_mean": rows_max * world / float(PT * CFG["NU"]) if not cap else None},
            "parity": {"checked": what, "bit_identical": same, "finite": finite},
            "gpu_launches": int(per_pass_launches * passes), "replayed_from_cuda_graph": replayed,
            "tensor": {"algorithmic_tflops_per_gpu": tf, "peak": peak_tf, "frac": (tf / peak_tf) if peak_tf else None,
                       "note": "algorithmic FLOPs (2*M*N*K once) over the whole pass, all kernels included; the MMAs issued are 3x that"}}


# ---------------------------------------------------------------- our arm
def run_ours(args, rank, local_rank, world):
    import torch
    from kairos_engine_b200 import FLAVOUR_DECODE, MoeEngine, synth
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(seconds=300))
    NL = args.layers
    PT = 0 if args.no_prefill else max(world, args.prefill_tokens // world * world)      # prefill tokens of the whole job
    ZT = 512 if (world > 1 and PT) else 0                                                 # load-imbalance stress tokens (whole job)
    max_tok = max(64 if (PT and world == 1) else 1, PT // world)
    eng = MoeEngine(n_layers=NL, max_tokens=max_tok, device=local_rank, max_expert_rows=PT * CFG["NU"] if world > 1 else 0, **CFG)
    bias = synth.zipf_bias(CFG["NE"], s=args.zipf, seed=3, device=f"cuda:{local_rank}") if args.zipf > 0 else None
    for L in range(NL):
        layer = synth.make_layer(CFG, 1000 * L, device=f"cuda:{local_rank}", bias=bias)
        eng.upload_layer(L, layer, on_device=True)
        del layer
    torch.cuda.empty_cache()
    E = CFG["E"]
    T = args.tokens_per_step
    xs = synth.make_inputs(CFG, T, seed=7 + rank, device=f"cuda:{local_rank}")      # resident inputs
    ys = torch.empty_like(xs)
    stream = torch.cuda.current_stream()

    def step():
        for t in range(T):
            eng.forward_dev(xs[t], ys[t], flavour=FLAVOUR_DECODE, stream=stream)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    eng.status()
    barrier()
    l0 = eng.kernel_launches
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank) as clk:
        ev0.record(stream)
        for _ in range(args.steps):
            step()
        ev1.record(stream)
        barrier()
    eng.status()
    ms = ev0.elapsed_time(ev1)
    launches = eng.kernel_launches - l0
    if dist is not None:
        tms = torch.tensor([ms], device=f"cuda:{local_rank}")
        dist.all_reduce(tms, op=dist.ReduceOp.MAX)
        ms = float(tms.item())
    tokens = T * args.steps * world
    value = tokens / (ms / 1e3)

    # ---- e2e: the host-pointer C-ABI call, pinned host buffers, copies inside the timed region
    xh = xs.cpu().pin_memory().numpy()
    yh = torch.empty((1, E), dtype=torch.float32).pin_memory().numpy()      # page-locked result buffer, as a serving loop would hold
    e2e_steps = max(1, min(args.steps, 4))
    for t in range(min(8, T)):
        eng.forward(xh[t:t + 1], want_routing=False, out=yh)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        for t in range(T):
            eng.forward(xh[t:t + 1], want_routing=False, out=yh)
    barrier()
    e2e_s = time.perf_counter() - t0
    if dist is not None:
        ts = torch.tensor([e2e_s], device=f"cuda:{local_rank}")
        dist.all_reduce(ts, op=dist.ReduceOp.MAX)
        e2e_s = float(ts.item())
    e2e_v = T * e2e_steps * world / e2e_s
    # the host entry and the device entry are the same kernels: the last token's result must agree bit for bit
    e2e_same = bool((torch.from_numpy(yh[0]).view(torch.int32) == ys[T - 1].cpu().view(torch.int32)).all())

    def extra(fn, *a, **kw):                          # the legs beside the headline must not take the headline down
        try:
            return fn(*a, **kw)
        except Exception as e:  # reported in the line instead
            return {"error": f"{type(e).__name__}: {e}"[:300]}

    peak, peak_tf, peak_kind = measured_peaks()
    prefill = extra(prefill_leg, args, eng, NL, PT, rank, local_rank, world, dist, barrier) if PT else None
    zipf = None
    if ZT:
        # the load-imbalance configuration: 512 tokens per step, a Zipf(1.2) bias on every router, exact exchange
        zb = synth.zipf_bias(CFG["NE"], s=1.2, seed=3, device=f"cuda:{local_rank}")
        for L in range(NL):
            eng.set_router_bias(L, zb)
        zipf = extra(prefill_leg, args, eng, NL, ZT, rank, local_rank, world, dist, barrier, zipf=True)
        if isinstance(zipf, dict) and "error" not in zipf:
            zipf["router_bias"] = "zipf s=1.2 per-expert logit bias on every layer (seeded expert permutation)"
        for L in range(NL):
            eng.set_router_bias(L, bias)
    stages = extra(ep_stage_timing_leg, NL, PT, rank, local_rank, world, dist) if (PT and world > 1 and args.ep_impl == "library") else None
    small = extra(small_batch_leg, eng, NL, local_rank, rank, peak) if (PT and world == 1) else None
    igemm = extra(int_gemm_leg, local_rank) if (PT and world == 1) else None
    terms = extra(prefill_terms_leg, NL, PT, local_rank) if (PT and world == 1) else None

    if rank == 0:
        bytes_per_launch = NL * synth.algorithmic_bytes_per_layer(CFG, M=1, U=CFG["NU"])
        launch_ms = ms / (T * args.steps)                 # one launch = one token through 30 layers
        achieved = bytes_per_launch / (launch_ms / 1e3) / 1e9
        line = {"metric": "MoE-FFN decode tokens/s (30-layer stack, M=1)", "value": value, "unit": "tokens/s", "n_gpus": world,
                "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "int8 activations x int4 weights, f32 accumulate", "data": "synthetic",
                "config": {"workload": "configs[1]: 30-layer MoE FFN stack (Gemma-4-26B-A4B geometry), decode M=1, sequential tokens, "
                                       "all experts resident", "layers": NL, "tokens_per_step": T, "parallelism": "replicas" if world > 1 else "single GPU",
                           "l2": "weights 13.2 GB per pass, far larger than L2: no flush needed", "router_bias": f"zipf s={args.zipf}" if args.zipf > 0 else "none"},
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                             "traffic": NL * NCU_TRAFFIC_BYTES_PER_LAYER if NCU_TRAFFIC_BYTES_PER_LAYER else None,
                             "algorithmic_bytes_per_launch": bytes_per_launch,
                             "kernel": "decode graph: per layer k_ds_router_shared + k_ds_experts_up + k_ds_experts_down (one graph launch = one token through the stack)",
                             "launch_ms": launch_ms},
                "e2e": {"value": e2e_v, "unit": "tokens/s", "h2d_bytes_per_step": T * E * 4, "d2h_bytes_per_step": T * E * 4},
                "gpu_launches": int(launches), "clocks": clk.summary(),
                "parity": {"e2e_equals_device_entry_bitwise": e2e_same}}
        if prefill:
            line["prefill"] = prefill
        if zipf:
            line["zipf"] = zipf
        if stages:
            line["ep_stage_times"] = stages
        if small:
            line["small_batch"] = small
        if igemm:
            line["int_gemm"] = igemm
        if terms:
            line["prefill_terms"] = terms
        if world == 1 and not args.no_cpu:
            try:
                line["cpu_baseline"], line["parity"]["decode_vs_checker"] = cpu_baseline_leg(eng, torch)
            except Exception as e:  # the checker is optional equipment for the bench
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"unavailable: {e}"}
            line["ref_gpu_kernels"] = extra(ref_gpu_leg, local_rank, torch)
            if isinstance(line["ref_gpu_kernels"], dict) and "us_per_layer_routed_branch" in line["ref_gpu_kernels"]:
                line["ref_gpu_kernels"]["ours_us_per_layer_whole_layer"] = launch_ms * 1e3 / NL
        print(json.dumps(line), flush=True)
    eng.close()
    if dist is not None:
        dist.barrier(); dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the cpu_baseline leg")
    ap.add_argument("--tokens-per-step", type=int, default=TOKENS_PER_STEP, help="profiling aid: fewer sequential tokens per step than the workload's 256")
    ap.add_argument("--prefill-tokens", type=int, default=4096, help="tokens of the prefill leg (whole job)")
    ap.add_argument("--no-prefill", action="store_true", help="skip the prefill leg")
    ap.add_argument("--no-ep-graph", action="store_true", help="run the expert-parallel prefill pass eagerly instead of from a CUDA graph")
    ap.add_argument("--ep-impl", default="library", choices=["library", "torch"], help="who drives the expert-parallel layers: the library's own NCCL loop, or the Python loop over torch.distributed")
    ap.add_argument("--ep-slices", type=int, default=1, help="token slices the library's expert-parallel loop keeps in flight (1..4)")
    ap.add_argument("--zipf", type=float, default=0.0, help="add a Zipf(s) per-expert bias to every router for the WHOLE run (0 = unbiased; the default N>1 line already carries a `zipf` object)")
    ap.add_argument("--layers", type=int, default=N_LAYERS, help="profiling aid: a shorter stack than the workload's 30 layers (not a bench result)")
    args = ap.parse_args()
    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
