"""Expert-parallel run of the MoE feed-forward layers over one process per GPU.

The reference is single-GPU: its batched branch walks every expert on the one device
(src/backends/cuda/cuda_forward.cu:8925-8965). Here tokens are data-parallel (each rank owns the
residual of its own tokens, the router, the shared expert and the norms) and the routed experts
are partitioned contiguously, `NE / world` per rank. Per layer there is one exchange each way:

  route (local) -> dispatch all-to-all of (expert id, input row) per (token, expert) pair
  -> experts (on the owner) -> combine all-to-all of the output rows back -> finish (local).

The per-token combine still walks the experts in ascending id on the home rank, so the result is
bit-identical to the single-GPU path. torch.distributed is plumbing only (NCCL on GPUs; the same
code runs on gloo/CPU in the tests with a stand-in for the three stage calls).
"""
import torch
import torch.distributed as dist


def plan_dispatch(sel_asc, n_experts, world):
    """sel_asc: int [M][NU] expert ids. Returns (order, send_counts): `order` lists the pair
    indices (t*NU + k) sorted by expert id, stably; because ownership is contiguous that is also
    sorted by destination rank; send_counts[r] = pairs going to rank r."""
    per = n_experts // world
    e = sel_asc.reshape(-1).to(torch.int64)
    order = torch.argsort(e, stable=True)
    send_counts = torch.bincount(e // per, minlength=world)
    return order, send_counts


def expert_offsets(expert_ids, n_experts):
    """int32 [NE+1] start offsets of each expert's rows in a list sorted by expert id."""
    cnt = torch.bincount(expert_ids.to(torch.int64), minlength=n_experts)
    off = torch.zeros(n_experts + 1, dtype=torch.int32, device=expert_ids.device)
    off[1:] = torch.cumsum(cnt, 0).to(torch.int32)
    return off


class ExpertParallelMoe:
    """engine: an object with ep_route / ep_experts / ep_finish (kairos_engine_b200.MoeEngine);
    cfg: its geometry dict. group: a torch.distributed process group (None = the default)."""

    def __init__(self, engine, cfg, group=None):
        self.engine, self.cfg, self.group = engine, cfg, group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if cfg["NE"] % self.world:
            raise ValueError(f"NE={cfg['NE']} is not divisible by the world size {self.world}")
        self.last_rows = 0          # rows this rank's experts processed in the last layer

    def _a2a(self, out, inp, out_splits, in_splits):
        dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.group)

    def layer(self, L, x, flavour):
        NE, NU, E = self.cfg["NE"], self.cfg["NU"], self.cfg["E"]
        M = x.shape[0]
        sel_asc, cw, rows = self.engine.ep_route(L, x, flavour)
        order, send_counts = plan_dispatch(sel_asc, NE, self.world)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=self.group)
        # one host read of 2*world integers per layer: the split sizes of the two exchanges
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        R = sum(rc)
        send_e = sel_asc.reshape(-1)[order].contiguous()
        send_rows = rows[torch.div(order, NU, rounding_mode="floor")].contiguous()
        recv_e = torch.empty(R, dtype=send_e.dtype, device=x.device)
        recv_rows = torch.empty((R, E), dtype=rows.dtype, device=x.device)
        self._a2a(recv_e, send_e, rc, sc)
        self._a2a(recv_rows, send_rows, rc, sc)
        # rows arrive grouped by source rank, each group sorted by expert: the expert stage walks them
        # through one stable sort by expert (an index list; the rows themselves stay where they landed)
        order2 = torch.argsort(recv_e.to(torch.int64), stable=True).to(torch.int32)
        off = expert_offsets(recv_e, NE)
        self.last_rows = R
        out_recv = self.engine.ep_experts(L, recv_rows, off, flavour, row_index=order2)
        back = torch.empty((M * NU, E), dtype=rows.dtype, device=x.device)
        self._a2a(back, out_recv, sc, rc)
        # back[i] is pair order[i]: the finish stage reads pair p at row inv[p]
        inv = torch.empty(M * NU, dtype=torch.int32, device=x.device)
        inv[order] = torch.arange(M * NU, dtype=torch.int32, device=x.device)
        return self.engine.ep_finish(L, x, back, pair_index=inv)

    def forward(self, x, layer_first=0, n_layers=1, flavour=1):
        for L in range(layer_first, layer_first + n_layers):
            x = self.layer(L, x, flavour)
        return x
