#!/usr/bin/env python
"""bench.py — MoE-FFN decode throughput of the 30-layer Gemma-4-26B-A4B-geometry stack on B200.

Workload (N=1 default): the full 30-layer MoE FFN stack, decode M=1, all 30*128 experts resident
in HBM, random-init Q4B weights (router N(0,0.02) f32; expert/shared weights N(0,0.02) then Q4B),
seeded N(0,1) hidden states. One bench STEP = 256 sequential single-token decode steps through
all 30 layers. `value` = tokens/s with inputs resident in HBM, timed with CUDA events on the
launching stream; `e2e` = the same through the host-pointer C-ABI call (H2D of the token's hidden
state and D2H of the result inside the timed region, every token). N>1 runs N independent
replicas (decode does not shard; expert-parallel prefill is reported separately).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

--impl reference times the reference's own CPU expert code (oracle/_ref: moe_cpu_expert.c compiled
in place, with the restated layer glue around it) on this host's cores on a bounded sample.
"""
import argparse
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
# dram__bytes_read.sum + dram__bytes_write.sum of one decode graph launch (one token, 30 layers), from the ncu
# launch list summarised in profiles/decode_graph_m1.md (caches kept between kernels, as in a real run)
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1164866112


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


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
def cpu_layers(n_pool, torch):
    """n_pool seeded layers generated on the GPU (same recipe as the bench's own), copied to host."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import orc
    from kairos_engine_b200 import synth
    out = []
    for L in range(n_pool):
        layer = synth.make_layer(CFG, 1000 * L)
        out.append(orc.LayerWeights(**synth.layer_to_host(layer)))
        del layer
    torch.cuda.empty_cache()
    return out


def cpu_time_tokens(layers, n_tokens, threads, seed=0):
    """Runs n_tokens single-token passes of the 30-layer stack on the CPU, cycling the layer pool
    (weights stay cold: the pool is far larger than the last-level cache). Returns (seconds, kind)."""
    import numpy as np
    import orc
    kind = orc.use_reference_gemv(threads)
    rng = np.random.default_rng(seed)
    t0 = time.perf_counter()
    for t in range(n_tokens):
        x = rng.standard_normal((1, CFG["E"])).astype(np.float32)
        for L in range(N_LAYERS):
            x = orc.layer_forward(CFG, layers[L % len(layers)], x, 0)["y"]
    return time.perf_counter() - t0, kind


def run_reference(args, rank, world):
    import torch
    if rank != 0:                                      # rank 0 alone runs the CPU arm; the others leave without work
        return
    threads = min(os.cpu_count() or 1, 16)            # the reference pool's cap (moe_cpu_expert.c:225)
    layers = cpu_layers(4, torch)
    tok = 1                                            # one step = one token through 30 layers
    for _ in range(args.warmup):
        cpu_time_tokens(layers, tok, threads)
    secs, kind = cpu_time_tokens(layers, tok * args.steps, threads, seed=1)
    v = tok * args.steps / secs
    sample = f"{tok} token x 30 layers per step, {args.steps} steps, layer pool of 4 cycled (cold weights)"
    line = {"impl": "reference", "metric": "MoE-FFN decode tokens/s (30-layer stack, M=1)", "value": v, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "int8 activations x int4 weights, f32 accumulate",
            "data": "synthetic", "config": {"workload": "configs[1]: 30-layer MoE FFN stack, decode M=1", "cpu_sample": sample},
            "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": threads, "kind": kind, "sample": sample},
            "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ---------------------------------------------------------------- batched decode / draft-verify shapes
def small_batch_leg(eng, NL, local_rank, rank):
    """M in {4, 8, 16, 64} tokens per step through the stack in the single-token decode arithmetic
    (what M sequential decode steps compute), unbiased router: the union of active experts grows with M."""
    import torch
    from kairos_engine_b200 import FLAVOUR_DECODE, synth
    out = {}
    for M in (4, 8, 16, 64):
        if M > eng.max_tokens:
            continue
        x = synth.make_inputs(CFG, M, seed=300 + M + rank, device=f"cuda:{local_rank}")
        y = torch.empty_like(x)
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
        out[f"M={M}"] = {"tokens_per_s": M / (ms / 1e3), "ms_per_step": ms}
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
def prefill_leg(args, eng, NL, PT, rank, local_rank, world, dist, barrier):
    """PT tokens through the stack in the prefill arithmetic: one GPU runs them all; N GPUs run
    PT/N tokens each with the routed experts partitioned NE/N per GPU (all-to-all each way)."""
    import torch
    from kairos_engine_b200 import FLAVOUR_PREFILL, SpMoeError, ep, synth
    Ml = PT // world
    xp = synth.make_inputs(CFG, Ml, seed=99 + rank, device=f"cuda:{local_rank}")
    yp = torch.empty_like(xp)
    # N > 1: padded exchange (no host read per layer) with room for 1.25x the average rows per destination
    # (unbiased routing spreads within a few percent; an overflow on any rank sends all ranks to the exact
    # exchange); the load-imbalance stress uses the exact exchange
    cap = 0 if (world < 2 or args.zipf > 0) else -(-5 * Ml * CFG["NU"] // (4 * world) // 8) * 8
    epm = ep.ExpertParallelMoe(eng, CFG, capacity_rows=cap) if world > 1 else None

    def one_pass():
        if epm is None:
            eng.forward_dev(xp, yp, 0, NL, FLAVOUR_PREFILL)
        else:
            epm.forward(xp, 0, NL, FLAVOUR_PREFILL)

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
    peak_tf = None
    try:
        peak_tf = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
    except Exception:
        pass
    return {"metric": "MoE-FFN prefill tokens/s (30-layer stack)", "value": PT * passes / (ms / 1e3), "unit": "tokens/s", "tokens": PT,
            "ms_per_pass": ms / passes, "passes": passes, "dtype": "f16 x f16 split operands (3 MMAs per k-step), f32 accumulate in TMEM",
            "parallelism": "single GPU" if world == 1 else f"expert-parallel: {PT // world} tokens and {CFG['NE'] // world} experts per GPU, all-to-all each way",
            "exchange": "none" if world == 1 else (f"padded: {cap} rows per destination, no host read per layer" if cap else "exact: split sizes read on the host once per layer"),
            "expert_rows_last_layer": {"max_per_gpu": rows_max, "min_per_gpu": rows_min},
            "gpu_launches": int(per_pass_launches * passes), "replayed_from_cuda_graph": replayed,
            "tensor": {"algorithmic_tflops_per_gpu": tf, "peak": peak_tf, "frac": (tf / peak_tf) if peak_tf else None,
                       "note": "algorithmic FLOPs (2*M*N*K once) over the whole pass, all kernels included; the MMAs issued are 3x that"}}


# ---------------------------------------------------------------- our arm
def run_ours(args, rank, local_rank, world):
    import numpy as np
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
    eng = MoeEngine(n_layers=NL, max_tokens=max(1, PT // world), device=local_rank, max_expert_rows=PT * CFG["NU"] if world > 1 else 0, **CFG)
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

    def extra(fn, *a):                                # the legs beside the headline must not take the headline down
        try:
            return fn(*a)
        except Exception as e:  # reported in the line instead
            return {"error": f"{type(e).__name__}: {e}"[:300]}

    prefill = extra(prefill_leg, args, eng, NL, PT, rank, local_rank, world, dist, barrier) if PT else None
    small = extra(small_batch_leg, eng, NL, local_rank, rank) if (PT and world == 1) else None
    igemm = extra(int_gemm_leg, local_rank) if (PT and world == 1) else None

    if rank == 0:
        peak, peak_kind = measured_peak()
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
                             "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if NL == N_LAYERS else None, "algorithmic_bytes_per_launch": bytes_per_launch, "kernel": "decode graph: per layer k_dg_router_shared + k_dg_experts_up + k_dg_experts_down (one graph launch = one token through the stack)",
                             "launch_ms": launch_ms},
                "e2e": {"value": e2e_v, "unit": "tokens/s", "h2d_bytes_per_step": T * E * 4, "d2h_bytes_per_step": T * E * 4},
                "gpu_launches": int(launches), "clocks": clk.summary()}
        if prefill:
            line["prefill"] = prefill
        if small:
            line["small_batch"] = small
        if igemm:
            line["int_gemm"] = igemm
        if world == 1 and not args.no_cpu:
            try:
                threads = min(os.cpu_count() or 1, 16)
                layers = cpu_layers(3, torch)
                cpu_time_tokens(layers, 1, threads)
                n_tok = 192
                secs, kind = cpu_time_tokens(layers, n_tok, threads, seed=1)
                line["cpu_baseline"] = {"value": n_tok / secs, "unit": "tokens/s", "cores": threads, "kind": kind,
                                        "sample": f"{n_tok} tokens x 30 layers, layer pool of 3 cycled (cold weights), {secs:.1f} s"}
            except Exception as e:  # the checker is optional equipment for the bench
                line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port", "sample": f"unavailable: {e}"}
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
    ap.add_argument("--zipf", type=float, default=0.0, help="load-imbalance stress: add a Zipf(s) per-expert bias to every router (0 = unbiased)")
    ap.add_argument("--layers", type=int, default=N_LAYERS, help="profiling aid: a shorter stack than the workload's 30 layers (not a bench result)")
    args = ap.parse_args()
    rank, local_rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
