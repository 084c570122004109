"""Host logic of the expert-parallel run on CPU: 2, 4 and 8 gloo ranks, a stand-in for the stage
calls whose arithmetic is simple enough to restate in one process."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kairos_engine_b200 import ep  # noqa: E402

CFG = dict(E=32, NE=8, NU=3)


class FakeStages:
    """route: scores = x @ Wr, top-NU ascending; experts: out = row * (e + 1) + e; finish: x + sum cw*pair."""

    def __init__(self, cfg, owned=None):
        g = torch.Generator().manual_seed(7)
        self.wr = torch.randn(cfg["E"], cfg["NE"], generator=g)
        self.cfg, self.owned, self.seen = cfg, owned, []

    def _route(self, L, x):
        s = x @ self.wr + L
        idx = torch.topk(s, self.cfg["NU"], dim=1).indices
        sel_asc = torch.sort(idx, dim=1).values.to(torch.int32)
        cw = torch.softmax(torch.gather(s, 1, sel_asc.to(torch.int64)), dim=1)
        return sel_asc, cw

    def ep_shared(self, L, M, flavour):
        self.shared_calls = getattr(self, "shared_calls", 0) + 1

    def ep_route(self, L, x, flavour, defer_shared=False, n_ranks=0, capacity=0):
        assert defer_shared
        sel_asc, cw = self._route(L, x)
        NU, NE = self.cfg["NU"], self.cfg["NE"]
        order, _ = ep.plan_dispatch(sel_asc, NE, 1)
        rows = (x * 2.0)[torch.div(order, NU, rounding_mode="floor")]
        counts = torch.bincount(sel_asc.reshape(-1).to(torch.int64), minlength=NE).to(torch.int32)
        pair_index = torch.empty(order.numel(), dtype=torch.int32)
        pair_index[order] = torch.arange(order.numel(), dtype=torch.int32)
        if capacity:                                    # padded send buffer: rank r's rows start at r * capacity
            epr = NE // n_ranks
            per_rank = counts.view(n_ranks, epr).sum(1)
            assert int(per_rank.max()) <= capacity, "test capacity too small"
            start = torch.cumsum(per_rank, 0) - per_rank
            e_sorted = sel_asc.reshape(-1)[order].to(torch.int64)
            owner = e_sorted // epr
            padded_pos = owner * capacity + (torch.arange(order.numel()) - start[owner])
            padded = torch.full((n_ranks * capacity, x.shape[1]), float("nan"))
            padded[padded_pos] = rows
            pair_index = padded_pos[pair_index.to(torch.int64)].to(torch.int32)
            rows = padded
        return sel_asc, cw, rows, counts, pair_index

    def ep_recv_layout(self, counts_all, rank, capacity):
        world, NE = counts_all.shape
        epr = NE // world
        c = counts_all[:, rank * epr:(rank + 1) * epr].to(torch.int64)
        total = int(c.sum())
        off, idx = ep.recv_layout(counts_all, rank, total)          # dense arrival numbering ...
        arr = c.reshape(-1); dense_start = (torch.cumsum(arr, 0) - arr).view(world, epr)[:, 0]
        src = torch.bucketize(idx.to(torch.int64), dense_start, right=True) - 1
        padded = (idx.to(torch.int64) - dense_start[src] + src * capacity).to(torch.int32)   # ... moved to the padded blocks
        out = torch.zeros(world * capacity, dtype=torch.int32)
        out[:total] = padded
        off = off.clone(); off[(rank + 1) * epr + 1:] = total
        return off, out

    def ep_experts(self, L, rows, offsets, flavour, row_index=None):
        out = torch.empty_like(rows)
        off = offsets.tolist()
        assert off[0] == 0 and off[-1] <= rows.shape[0]
        idx = torch.arange(rows.shape[0]) if row_index is None else row_index.to(torch.int64)
        for e in range(self.cfg["NE"]):
            if off[e + 1] > off[e]:
                if self.owned is not None:
                    assert e in self.owned, f"expert {e} reached a rank that does not own it"
                self.seen.append(e)
                sel = idx[off[e]:off[e + 1]]
                out[sel] = rows[sel] * (e + 1) + e
        return out

    def ep_finish(self, L, x, pair_rows, pair_index=None):
        sel_asc, cw = self._route(L, x)
        M, NU = cw.shape
        pr = pair_rows.reshape(pair_rows.shape[0] if pair_index is not None else M * NU, -1)
        if pair_index is not None:
            pr = pr[pair_index.to(torch.int64)]
        return x + (cw.unsqueeze(-1) * pr.view(M, NU, -1)).sum(1)


def single_process(x, n_layers):
    f = FakeStages(CFG)
    for L in range(n_layers):
        sel_asc, cw = f._route(L, x)
        e = sel_asc.to(torch.float32).unsqueeze(-1)
        pair = (x * 2.0).unsqueeze(1) * (e + 1) + e
        x = x + (cw.unsqueeze(-1) * pair).sum(1)
    return x


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _rank_main(rank, world, port, tokens, n_layers, out_q, capacity=0):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(100 + rank)
        x = torch.randn(tokens[rank], CFG["E"], generator=g)
        per = CFG["NE"] // world
        eng = FakeStages(CFG, owned=set(range(rank * per, (rank + 1) * per)))
        run = ep.ExpertParallelMoe(eng, CFG, capacity_rows=capacity)
        y = run.forward(x, 0, n_layers, 0)
        out_q.put((rank, x.numpy(), y.numpy(), sorted(set(eng.seen))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("tokens", [(5, 9), (1, 16), (7, 7), (3, 6, 2, 9), (4, 4, 4, 4, 1, 7, 2, 5)])
def test_ranks_match_single_process(tokens):
    world, n_layers = len(tokens), 3            # 2, 4 and 8 ranks over the 8 experts
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    ps = [ctx.Process(target=_rank_main, args=(r, world, port, tokens, n_layers, q)) for r in range(world)]
    for p in ps: p.start()
    got = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(60); assert p.exitcode == 0
    for rank, x, y, seen in got:
        want = single_process(torch.from_numpy(x), n_layers).numpy()
        np.testing.assert_array_equal(y, want)


@pytest.mark.parametrize("tokens", [(6, 6), (5, 5, 5, 5)])
def test_padded_exchange_matches_single_process(tokens):
    world, n_layers = len(tokens), 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    cap = tokens[0] * CFG["NU"]                      # worst case: every pair of a rank goes to one rank
    ps = [ctx.Process(target=_rank_main, args=(r, world, port, tokens, n_layers, q, cap)) for r in range(world)]
    for p in ps: p.start()
    got = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(60); assert p.exitcode == 0
    for rank, x, y, seen in got:
        np.testing.assert_array_equal(y, single_process(torch.from_numpy(x), n_layers).numpy())


def test_plan_dispatch_orders_pairs_by_owner():
    sel = torch.tensor([[1, 4, 6], [0, 2, 7], [3, 4, 5]], dtype=torch.int32)
    order, counts = ep.plan_dispatch(sel, 8, 2)
    e = sel.reshape(-1)[order]
    assert torch.all(e[1:] >= e[:-1])
    assert counts.tolist() == [4, 5]
    off = ep.expert_offsets(e, 8)
    assert off.tolist() == [0, 1, 2, 3, 4, 6, 7, 8, 9]


def test_recv_layout_merges_source_blocks_by_expert():
    # 2 ranks, 4 experts (2 each); rank 1 owns experts 2, 3
    counts_all = torch.tensor([[1, 0, 2, 1], [3, 1, 0, 2]], dtype=torch.int32)
    off, idx = ep.recv_layout(counts_all, 1, 5)
    # arrival on rank 1: from rank 0: e2, e2, e3 (rows 0-2); from rank 1: e3, e3 (rows 3-4)
    assert off.tolist() == [0, 0, 0, 2, 5]
    assert idx.tolist() == [0, 1, 2, 3, 4]
    off0, idx0 = ep.recv_layout(counts_all, 0, 5)
    # arrival on rank 0: from rank 0: e0 (row 0); from rank 1: e0, e0, e0, e1 (rows 1-4) -> already sorted
    assert off0.tolist() == [0, 4, 5, 5, 5] and idx0.tolist() == [0, 1, 2, 3, 4]
    counts_all = torch.tensor([[1, 2, 0, 0], [1, 1, 0, 0]], dtype=torch.int32)
    off, idx = ep.recv_layout(counts_all, 0, 5)
    # arrival: r0: e0, e1, e1 (rows 0-2); r1: e0, e1 (rows 3-4) -> sorted: e0: rows 0, 3; e1: rows 1, 2, 4
    assert off.tolist() == [0, 2, 5, 5, 5] and idx.tolist() == [0, 3, 1, 2, 4]


def test_world_must_divide_experts():
    class G:  # minimal stand-in so no process group is needed
        pass
    with pytest.raises(Exception):
        ep.ExpertParallelMoe(FakeStages(CFG), dict(CFG, NE=7))


def test_token_dispatch_protocol():
    """The padded exchange's token dispatch, restated on the host (what k_b_tok_scan / k_b_tok_rows / k_b_tok_idx do on
    the sender and k_b_in_index on the receiver): a token's row travels once per destination rank, every pair carries
    the slot of its token, and the receiver's gather index picks, for every pair, exactly the row a one-row-per-pair
    exchange would have delivered."""
    cfg = dict(E=8, NE=16, NU=4)
    world, M = 4, 23
    epr, NU = cfg["NE"] // world, cfg["NU"]
    cap, cap_t = 48, 24                                       # pairs / token rows per destination block
    g = torch.Generator().manual_seed(5)
    fakes = [FakeStages(cfg) for _ in range(world)]
    xs = [torch.randn(M, cfg["E"], generator=g) for _ in range(world)]
    sent = []
    for s in range(world):
        sel_asc, _, pair_rows, counts, pair_index = fakes[s].ep_route(0, xs[s], 0, defer_shared=True, n_ranks=world, capacity=cap)
        owner = (sel_asc.to(torch.int64) // epr)              # [M][NU]
        flag = torch.zeros(M, world, dtype=torch.bool)
        flag.scatter_(1, owner, True)
        slot = torch.cumsum(flag.to(torch.int64), 0) - 1      # rank of the token among the destination's tokens
        slot[~flag] = -1
        assert int(flag.sum(0).max()) <= cap_t
        tokrows = torch.full((world * cap_t, cfg["E"]), float("nan"))
        for t in range(M):
            for r in range(world):
                if flag[t, r]:
                    tokrows[r * cap_t + slot[t, r]] = (xs[s] * 2.0)[t]       # the fake's routed-input row of token t
        tokidx = torch.zeros(world * cap, dtype=torch.int64)
        pi = pair_index.to(torch.int64).view(M, NU)
        for t in range(M):
            for k in range(NU):
                tokidx[pi[t, k]] = slot[t, owner[t, k]]
        sent.append((pair_rows, counts, tokrows, tokidx))
        assert (flag.sum(0) < NU * M // world + M).all() and int(flag.sum()) < M * NU      # fewer rows than pairs
    counts_all = torch.stack([c for _, c, _, _ in sent])
    for r in range(world):
        pair_recv = torch.cat([sent[s][0][r * cap:(r + 1) * cap] for s in range(world)])     # what pair rows would deliver
        tok_recv = torch.cat([sent[s][2][r * cap_t:(r + 1) * cap_t] for s in range(world)])
        idx_recv = torch.cat([sent[s][3][r * cap:(r + 1) * cap] for s in range(world)])
        off, row_index = fakes[r].ep_recv_layout(counts_all, r, cap)
        total = int(off[(r + 1) * epr])
        a = row_index[:total].to(torch.int64)                 # arrival slot of every sorted position
        in_index = (a // cap) * cap_t + idx_recv[a]
        assert torch.equal(tok_recv[in_index], pair_recv[a])
        assert not torch.isnan(tok_recv[in_index]).any()
