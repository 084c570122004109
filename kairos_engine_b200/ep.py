"""Expert-parallel run of the MoE feed-forward layers over one process per GPU.

The reference is single-GPU: its batched branch walks every expert on the one device
(src/backends/cuda/cuda_forward.cu:8925-8965). Here tokens are data-parallel (each rank owns the
residual of its own tokens, the router, the shared expert and the norms) and the routed experts
are partitioned contiguously, `NE / world` per rank. Per layer there is one exchange each way:

  route (local) -> all-gather of the per-expert pair counts -> dispatch all-to-all of the input rows
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
    sorted by destination rank; send_counts[r] = pairs going to rank r. (Reference form of what the
    route stage does on the device; used by tests.)"""
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


def recv_layout(counts_all, rank, n_rows):
    """counts_all: int [world][NE], pairs per expert on every rank. The rows this rank receives arrive
    source-major (each source's block sorted by expert). Returns (offsets int32 [NE+1], row_index int32
    [n_rows]): expert e owns sorted positions [offsets[e], offsets[e+1]) and sorted position p is arrival
    row row_index[p]. No host synchronisation: n_rows is already known from the split sizes."""
    world, NE = counts_all.shape
    epr = NE // world
    dev = counts_all.device
    c = counts_all[:, rank * epr:(rank + 1) * epr].to(torch.int64)          # [source][my expert]
    arr = c.reshape(-1)
    arr_start = (torch.cumsum(arr, 0) - arr).view(world, epr)               # arrival start of block (source, expert)
    ct = c.t().contiguous().reshape(-1)                                     # block sizes in sorted order (expert, source)
    sorted_start = torch.cumsum(ct, 0) - ct
    block = torch.repeat_interleave(torch.arange(world * epr, device=dev), ct, output_size=n_rows)
    start_of_block = arr_start.t().contiguous().reshape(-1)
    row_index = (start_of_block[block] + (torch.arange(n_rows, device=dev) - sorted_start[block])).to(torch.int32)
    offsets = torch.zeros(NE + 1, dtype=torch.int32, device=dev)
    offsets[rank * epr + 1:(rank + 1) * epr + 1] = torch.cumsum(c.sum(0), 0).to(torch.int32)
    offsets[(rank + 1) * epr + 1:] = n_rows
    return offsets, row_index


class ExpertParallelMoe:
    """engine: an object with ep_route / ep_experts / ep_finish (kairos_engine_b200.MoeEngine);
    cfg: its geometry dict. group: a torch.distributed process group (None = the default)."""

    def __init__(self, engine, cfg, group=None, capacity_rows=0):
        """capacity_rows > 0: padded exchange - every rank sends exactly capacity_rows rows to every rank (the
        same number on all ranks), so a layer needs no host read and the CPU can enqueue the whole stack ahead of
        the GPU; a destination that would get more rows than that from one rank is reported by the engine's
        status(). 0: exact exchange with split sizes read on the host once per layer."""
        self.engine, self.cfg, self.group = engine, cfg, group
        self.capacity = int(capacity_rows)
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if cfg["NE"] % self.world:
            raise ValueError(f"NE={cfg['NE']} is not divisible by the world size {self.world}")
        self.last_rows = 0          # rows this rank's experts processed in the last layer

    def _a2a(self, out, inp, out_splits, in_splits):
        dist.all_to_all_single(out, inp, output_split_sizes=out_splits, input_split_sizes=in_splits, group=self.group)

    def _layer_padded(self, L, x, flavour):
        NU, E, world, C = self.cfg["NU"], self.cfg["E"], self.world, self.capacity
        sel_asc, cw, rows, counts, pair_index = self.engine.ep_route(L, x, flavour, defer_shared=True, n_ranks=world, capacity=C)
        gathered = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts, group=self.group)
        counts_all = torch.stack(gathered)
        recv_rows = torch.empty_like(rows)
        work = dist.all_to_all_single(recv_rows, rows, group=self.group, async_op=True)      # equal splits: no sizes needed
        self.engine.ep_shared(L, x.shape[0], flavour)
        offsets, row_index = self.engine.ep_recv_layout(counts_all, self.rank, C)
        work.wait()
        self.last_rows = world * C
        out_recv = self.engine.ep_experts(L, recv_rows, offsets, flavour, row_index=row_index)
        back = torch.empty_like(rows)
        dist.all_to_all_single(back, out_recv, group=self.group)
        return self.engine.ep_finish(L, x, back, pair_index=pair_index)

    def layer(self, L, x, flavour):
        if self.capacity > 0:
            return self._layer_padded(L, x, flavour)
        NE, NU, E = self.cfg["NE"], self.cfg["NU"], self.cfg["E"]
        M, world, epr = x.shape[0], self.world, self.cfg["NE"] // self.world
        # route: the send buffer comes back already sorted by expert (= by owner)
        sel_asc, cw, rows, counts, pair_index = self.engine.ep_route(L, x, flavour, defer_shared=True)
        gathered = [torch.empty_like(counts) for _ in range(world)]
        dist.all_gather(gathered, counts, group=self.group)
        counts_all = torch.stack(gathered)                                   # [world][NE]
        send_counts = counts.view(world, epr).sum(1)
        recv_counts = counts_all[:, self.rank * epr:(self.rank + 1) * epr].sum(1)
        # the one host read of the layer: the split sizes of the two exchanges
        sc, rc = torch.stack([send_counts, recv_counts]).tolist()
        R = sum(rc)
        recv_rows = torch.empty((R, E), dtype=rows.dtype, device=x.device)
        work = dist.all_to_all_single(recv_rows, rows, output_split_sizes=rc, input_split_sizes=sc, group=self.group, async_op=True)
        self.engine.ep_shared(L, M, flavour)                                 # the shared expert runs under the dispatch
        offsets, row_index = recv_layout(counts_all, self.rank, R)
        work.wait()
        self.last_rows = R
        out_recv = self.engine.ep_experts(L, recv_rows, offsets, flavour, row_index=row_index)
        back = torch.empty((M * NU, E), dtype=rows.dtype, device=x.device)
        self._a2a(back, out_recv, sc, rc)
        return self.engine.ep_finish(L, x, back, pair_index=pair_index)

    def forward(self, x, layer_first=0, n_layers=1, flavour=1):
        for L in range(layer_first, layer_first + n_layers):
            x = self.layer(L, x, flavour)
        return x


class NcclExpertParallel:
    """The same loop run inside the library (sp_moe_ep_forward_dev): NCCL called from C++, the exchanges on an internal
    stream beside the GEMMs (the shared expert's two halves run under the dispatch and the combine; with a padded
    exchange a token's row travels once per destination rank; in a world of up to four ranks the rows move by device-to-device
    copies into IPC-mapped peer buffers). torch.distributed is used once, to hand rank 0's NCCL id to the other
    ranks; the communicator is the library's own. Every rank must open its engine with the same configuration."""

    def __init__(self, engine, cfg, group=None, capacity_rows=0, slices=1):
        import ctypes as C
        from . import _lib
        self.engine, self.cfg = engine, cfg
        self.capacity, self.slices = int(capacity_rows), int(slices)
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if cfg["NE"] % self.world:
            raise ValueError(f"NE={cfg['NE']} is not divisible by the world size {self.world}")
        L = _lib.lib()
        ident = (C.c_ubyte * 128)()
        if self.rank == 0:
            _lib.check(L.sp_moe_ep_unique_id(ident))
        box = [bytes(ident)]
        dist.broadcast_object_list(box, src=0, group=group)
        ident = (C.c_ubyte * 128).from_buffer_copy(box[0])
        self._comm = C.c_void_p()
        _lib.check(L.sp_moe_ep_comm_create(ident, self.world, self.rank, C.byref(self._comm)))

    @property
    def last_rows(self):
        from . import _lib
        return int(_lib.lib().sp_moe_ep_last_rows(self.engine._h))

    def timing(self):
        """Stage times (ms) of the last layer of the most recent forward(): needs SP_MOE_TIMING=1 when the engine was
        opened, one slice and a call outside a stream capture."""
        import ctypes as C
        from . import _lib
        ms = (C.c_float * 6)()
        _lib.check(_lib.lib().sp_moe_ep_timing(self.engine._h, ms))
        keys = ("route", "gather_dispatch", "experts_after_dispatch", "combine", "finish", "layer")
        return {k: float(v) for k, v in zip(keys, ms)}

    def forward(self, x, layer_first=0, n_layers=1, flavour=1, out=None):
        from . import _lib
        y = torch.empty_like(x) if out is None else out
        st = torch.cuda.current_stream(x.device).cuda_stream
        _lib.check(_lib.lib().sp_moe_ep_forward_dev(self.engine._h, self._comm, self.world, self.rank, layer_first, n_layers, flavour, x.shape[0],
                                                   x.data_ptr(), y.data_ptr(), self.capacity, self.slices, st))
        return y

    def close(self):
        from . import _lib
        if getattr(self, "_comm", None) is not None and self._comm.value:
            _lib.lib().sp_moe_ep_comm_destroy(self._comm)
            self._comm = None
