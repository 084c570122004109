"""Expert-parallel stages on the GPU: the three-stage cut of a layer is bit-identical to the
one-call path, on one GPU (stages chained by hand) and on two GPUs over NCCL (when present)."""
import os
import socket
import sys

import numpy as np
import pytest

import orc
from gpu_common import make_stack

pytestmark = pytest.mark.gpu
A, B = 0, 1


def _chain_stages(eng, cfg, x, n_layers, flavour):
    import torch
    NE = cfg["NE"]
    for L in range(n_layers):
        sel_asc, cw, rows, counts, pair_index = eng.ep_route(L, x, flavour, defer_shared=bool(L & 1))
        if L & 1:
            eng.ep_shared(L, x.shape[0], flavour)
        off = torch.zeros(NE + 1, dtype=torch.int32, device=x.device)
        off[1:] = torch.cumsum(counts, 0).to(torch.int32)
        out = eng.ep_experts(L, rows, off, flavour)                  # the send buffer is already sorted by expert
        x = eng.ep_finish(L, x, out, pair_index=pair_index)
    return x


@pytest.mark.parametrize("cfg,n_layers,M,flavour", [(orc.TINY, 2, 5, A), (orc.SMALL, 2, 33, B), (orc.SMALL, 1, 16, A),
                                                    (orc.GEMMA, 1, 12, B), (orc.GEMMA, 1, 6, A)])
def test_stages_equal_one_call(cfg, n_layers, M, flavour):
    import torch
    eng, _ = make_stack(cfg, n_layers, seed=31, rand_norms=True, max_tokens=M)
    x = torch.from_numpy(np.random.default_rng(M).standard_normal((M, cfg["E"])).astype(np.float32)).cuda()
    y = torch.empty_like(x)
    eng.forward_dev(x, y, 0, n_layers, flavour)
    eng.status()
    y2 = _chain_stages(eng, cfg, x, n_layers, flavour)
    eng.status()
    assert torch.equal(y.view(torch.int32), y2.view(torch.int32))
    eng.close()


def test_experts_stage_accepts_a_subset_and_empty_input():
    import torch
    from kairos_engine_b200 import ep
    cfg = orc.SMALL
    eng, _ = make_stack(cfg, 1, seed=32, max_tokens=8)
    rows = torch.randn(5, cfg["E"], device="cuda")
    ids = torch.tensor([2, 2, 9, 9, 9], dtype=torch.int32, device="cuda")
    out = eng.ep_experts(0, rows, ep.expert_offsets(ids, cfg["NE"]), B)
    # the same rows one expert at a time give the same bytes
    one = eng.ep_experts(0, rows[:2].contiguous(), ep.expert_offsets(ids[:2], cfg["NE"]), B)
    eng.status()
    assert torch.equal(out[:2].view(torch.int32), one.view(torch.int32))
    empty = eng.ep_experts(0, rows[:0].contiguous(), ep.expert_offsets(ids[:0], cfg["NE"]), B)
    assert empty.shape[0] == 0
    eng.close()


@pytest.mark.parametrize("flavour", [A, B])
def test_experts_stage_with_row_index_equals_sorted_rows(flavour):
    import torch
    from kairos_engine_b200 import ep
    cfg = orc.SMALL
    eng, _ = make_stack(cfg, 1, seed=33, max_tokens=16)
    g = torch.Generator(device="cuda").manual_seed(5)
    R = 40
    rows = torch.randn(R, cfg["E"], device="cuda", generator=g)
    ids = torch.randint(0, cfg["NE"], (R,), device="cuda", generator=g).to(torch.int32)      # arrival order: unsorted
    order = torch.argsort(ids.to(torch.int64), stable=True).to(torch.int32)
    off = ep.expert_offsets(ids, cfg["NE"])
    out_idx = eng.ep_experts(0, rows, off, flavour, row_index=order)                        # rows stay where they are
    out_sorted = eng.ep_experts(0, rows[order.long()].contiguous(), off, flavour)
    eng.status()
    assert torch.equal(out_idx[order.long()].view(torch.int32), out_sorted.view(torch.int32))
    eng.close()


@pytest.mark.parametrize("flavour", [A, B])
def test_padded_route_and_receive_layout_equal_one_call(flavour):
    import torch
    cfg, M = orc.SMALL, 20
    eng, _ = make_stack(cfg, 1, seed=34, rand_norms=True, max_tokens=M, max_expert_rows=M * orc.SMALL["NU"] + 16)
    x = torch.from_numpy(np.random.default_rng(8).standard_normal((M, cfg["E"])).astype(np.float32)).cuda()
    y = torch.empty_like(x)
    eng.forward_dev(x, y, 0, 1, flavour)
    C = M * cfg["NU"] + 16                                           # one "rank", padded beyond what exists
    sel_asc, cw, rows, counts, pair_index = eng.ep_route(0, x, flavour, n_ranks=1, capacity=C)
    assert rows.shape[0] == C
    off, row_index = eng.ep_recv_layout(counts.view(1, -1), 0, C)
    assert off.tolist() == [0] + torch.cumsum(counts, 0).tolist()
    assert row_index[:M * cfg["NU"]].tolist() == list(range(M * cfg["NU"])) and int(row_index[M * cfg["NU"]:].abs().sum()) == 0
    rows[M * cfg["NU"]:] = float("nan")                              # the padding must never be read into a result
    out = eng.ep_experts(0, rows, off, flavour, row_index=row_index)
    y2 = eng.ep_finish(0, x, out, pair_index=pair_index)
    eng.status()
    assert torch.equal(y.view(torch.int32), y2.view(torch.int32))
    eng.close()


def test_receive_layout_kernel_matches_host_arithmetic():
    import torch
    from kairos_engine_b200 import ep
    cfg = orc.SMALL                                                  # 16 experts
    eng, _ = make_stack(cfg, 1, seed=35, max_tokens=64)             # 256 expert rows: room for 4 x 40
    world, C = 4, 40
    g = torch.Generator().manual_seed(3)
    counts_all = torch.randint(0, 10, (world, cfg["NE"]), generator=g, dtype=torch.int32)
    epr = cfg["NE"] // world
    for rank in range(world):
        c = counts_all[:, rank * epr:(rank + 1) * epr].to(torch.int64)
        total = int(c.sum())
        off, idx = eng.ep_recv_layout(counts_all.cuda(), rank, C)
        roff, ridx = ep.recv_layout(counts_all, rank, total)         # dense arrival numbering
        dense_start = (torch.cumsum(c.sum(1), 0) - c.sum(1))
        src = torch.bucketize(ridx.to(torch.int64), dense_start, right=True) - 1
        want = ridx.to(torch.int64) - dense_start[src] + src * C      # the same rows in the padded blocks
        assert off.cpu().tolist() == roff.tolist()
        assert idx.cpu()[:total].tolist() == want.tolist() and int(idx.cpu()[total:].abs().sum()) == 0
    eng.close()


def test_receive_layout_stays_inside_the_buffer_when_a_source_overflows():
    """A source whose block for this rank overflowed reports its full counts but delivered only
    `capacity` rows (the first ones, in expert order). The layout must follow what was delivered:
    no arrival row outside the receive buffer, no more sorted rows than the buffer holds, and the
    experts stage must run on it without touching anything else."""
    import torch
    cfg = orc.SMALL                                                  # 16 experts
    world, C = 4, 12
    eng, _ = make_stack(cfg, 1, seed=37, max_tokens=64, max_expert_rows=world * C)
    epr = cfg["NE"] // world
    counts_all = torch.full((world, cfg["NE"]), 2, dtype=torch.int32)      # 8 rows per source and rank: fits
    counts_all[world - 1, :] = 7                                           # the LAST source sends 28 > 12 to every rank
    counts_all[1, 0] = 30                                                  # and one expert alone exceeds the capacity
    for rank in range(world):
        off, idx = eng.ep_recv_layout(counts_all.cuda(), rank, C)
        off, idx = off.cpu(), idx.cpu()
        kept = torch.zeros(world, epr, dtype=torch.int64)
        for s in range(world):
            room = C
            for e in range(epr):
                kept[s, e] = min(int(counts_all[s, rank * epr + e]), room); room -= int(kept[s, e])
        total = int(kept.sum())
        assert int(off[cfg["NE"]]) == total <= world * C
        assert off[rank * epr:(rank + 1) * epr + 1].tolist() == [0] + torch.cumsum(kept.sum(0), 0).tolist()
        assert int(idx.min()) >= 0 and int(idx.max()) < world * C
        want = []
        for e in range(epr):
            for s in range(world):
                start = s * C + int(kept[s, :e].sum())
                want += list(range(start, start + int(kept[s, e])))
        assert idx[:total].tolist() == want
        rows = torch.randn(world * C, cfg["E"], device="cuda")
        out = eng.ep_experts(0, rows, off.cuda(), flavour=B, row_index=idx.cuda())
        eng.status()
        assert torch.isfinite(out[idx[:total].long().cuda()]).all()
    eng.close()


def test_padded_route_reports_a_block_that_does_not_fit():
    import torch
    from kairos_engine_b200 import SpMoeError
    cfg, M = orc.SMALL, 16
    eng, _ = make_stack(cfg, 1, seed=36, max_tokens=M)
    x = torch.randn(M, cfg["E"], device="cuda")
    eng.ep_route(0, x, B, n_ranks=2, capacity=8)                     # 64 pairs over two ranks cannot fit 8 rows each
    with pytest.raises(SpMoeError):
        eng.status()
    eng.close()


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _nccl_rank(rank, world, port, cases, q, env=None):
    """cases: list of (impl, flavour, capacity, slices). One process pair, one NCCL start-up, every case.
    env: switches the library reads when the handle's expert-parallel state is first built."""
    os.environ.update(env or {})
    import torch
    import torch.distributed as dist
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from kairos_engine_b200 import MoeEngine, ep, synth
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        cfg, n_layers, M = orc.SMALL, 2, 24 + 8 * rank
        os.environ["SP_MOE_TIMING"] = "1"          # stage events carry time (sp_moe_ep_timing); nothing else changes
        try:
            eng = MoeEngine(n_layers=n_layers, max_tokens=64, device=rank, max_expert_rows=512, **cfg)
        finally:
            del os.environ["SP_MOE_TIMING"]
        for L in range(n_layers):
            eng.upload_layer(L, synth.make_layer(cfg, 77 + 1000 * L, rand_norms=True, device=f"cuda:{rank}"), on_device=True)
        x = torch.from_numpy(np.random.default_rng(rank).standard_normal((M, cfg["E"])).astype(np.float32)).cuda()
        results = []
        for impl, flavour, capacity, slices in cases:
            want = torch.empty_like(x)
            eng.forward_dev(x, want, 0, n_layers, flavour)
            if impl == "library":                  # the loop inside the library: NCCL called from C++, token slices pipelined
                drv = ep.NcclExpertParallel(eng, cfg, capacity_rows=capacity, slices=slices)
                got = drv.forward(x, 0, n_layers, flavour)
                again = drv.forward(x, 0, n_layers, flavour)      # buffers and events are reused across calls
                eng.status()
                torch.cuda.synchronize()
                ok = bool(torch.equal(got.view(torch.int32), want.view(torch.int32))) and bool(torch.equal(again.view(torch.int32), want.view(torch.int32)))
                ok = ok and drv.last_rows > 0
                if slices == 1:                    # the stage times of the last layer: positive, and they fit inside the layer
                    tm = drv.timing()
                    ok = ok and tm["layer"] > 0 and all(v >= 0 for v in tm.values()) and tm["route"] + tm["finish"] <= tm["layer"] * 1.001
                drv.close()
            else:
                got = ep.ExpertParallelMoe(eng, cfg, capacity_rows=capacity).forward(x, 0, n_layers, flavour)
                eng.status()
                torch.cuda.synchronize()
                ok = bool(torch.equal(got.view(torch.int32), want.view(torch.int32)))
            results.append(ok)
        q.put((rank, results))
        eng.close()
    finally:
        dist.destroy_process_group()


def _run_pair(cases, env=None):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_nccl_rank, args=(r, 2, port, cases, q, env)) for r in range(2)]
    for p in ps: p.start()
    got = [q.get(timeout=600) for _ in ps]
    for p in ps:
        p.join(120); assert p.exitcode == 0
    for rank, results in got:
        bad = [c for c, ok in zip(cases, results) if not ok]
        assert not bad, f"rank {rank}: not bit-identical to the single-GPU pass: {bad}"


def test_two_gpus_nccl_equal_single_gpu():
    """ExpertParallelMoe over torch.distributed (NCCL) == the single-GPU pass, bit for bit: both arithmetic
    flavours, exact and padded exchange."""
    _run_pair([("torch", A, 0, 1), ("torch", B, 0, 1), ("torch", A, 160, 1), ("torch", B, 160, 1)])


LIBRARY_CASES = [("library", B, 0, 1), ("library", A, 0, 1), ("library", B, 160, 1), ("library", B, 160, 2), ("library", A, 160, 3), ("library", B, 200, 4)]


def test_two_gpus_library_loop_equals_single_gpu():
    """sp_moe_ep_forward_dev (the whole loop behind the C ABI, its own NCCL communicator) == the single-GPU pass,
    bit for bit: exact and padded exchange, one to four token slices in flight. In a world of up to four ranks the rows move
    by device-to-device copies into the peer's buffers, and the padded exchange sends token rows."""
    _run_pair(LIBRARY_CASES)


@pytest.mark.parametrize("env", [{"SP_MOE_EP_EXCHANGE": "nccl"}, {"SP_MOE_EP_EXCHANGE": "nccl", "SP_MOE_EP_DISPATCH": "rows"},
                                 {"SP_MOE_EP_EXCHANGE": "copy", "SP_MOE_EP_DISPATCH": "rows"}])
def test_two_gpus_library_loop_other_exchanges(env):
    """The same cases with the rows moved by NCCL send/recv pairs (what a world of more than four ranks uses), and with
    one row per (token, expert) pair instead of token rows."""
    _run_pair(LIBRARY_CASES, env)
