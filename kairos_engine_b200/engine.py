"""Host-side mirror of the reference's MoE feed-forward seam, over the C ABI.

`MoeEngine.forward` is g4_ffn_block -> g4_ffn_apply(moe_on=1) of the reference
(src/backends/cuda/cuda_forward.cu:9101-9114, 8314-9050): x [M][E] in, updated residual out,
for a run of consecutive layers. Weights are passed per layer in the reference's own layouts
(include/sp_engine/sp_model.h:50-53). torch is used only to own device buffers and streams.
"""
import ctypes as C

import numpy as np

from . import _lib
from ._lib import SpMoeConfig, SpMoeLayerWeights, check
from .trace import RouteTrace

FLAVOUR_DECODE = 0     # int8 activation quant + exact integer dots (reference decode arithmetic)
FLAVOUR_PREFILL = 1    # exact Q4B dequant + floating-point GEMM (reference prefill arithmetic)

GEMMA4_26B_A4B = dict(E=2816, NE=128, NU=8, FFE=704, FFS=2112, eps=1e-6)

WEIGHT_FIELDS = _lib._PTR_FIELDS


def _ptr(a):
    """Address of a numpy array (host) or torch tensor (device)."""
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        if not a.flags["C_CONTIGUOUS"]:
            raise ValueError("weight arrays must be C-contiguous")
        return a.ctypes.data
    return a.data_ptr()


class MoeEngine:
    """Owns one sp_moe handle: the resident arena of every layer's experts plus scratch."""

    def __init__(self, E, NE, NU, FFE, FFS, n_layers, max_tokens=1, eps=1e-6, device=0, max_expert_rows=0):
        self.cfg = dict(E=E, NE=NE, NU=NU, FFE=FFE, FFS=FFS, eps=eps)
        self.n_layers, self.max_tokens, self.device = n_layers, max_tokens, device
        c = SpMoeConfig(E=E, NE=NE, NU=NU, FFE=FFE, FFS=FFS, n_layers=n_layers,
                        max_tokens=max_tokens, device=device, eps=eps, max_expert_rows=max_expert_rows)
        self._h = C.c_void_p()
        check(_lib.lib().sp_moe_open(C.byref(c), C.byref(self._h)))
        self._trace = RouteTrace()

    # -- lifecycle
    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().sp_moe_close(self._h)
            self._h = C.c_void_p()

    __del__ = close

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    @property
    def device_bytes(self):
        return _lib.lib().sp_moe_device_bytes(self._h)

    @property
    def kernel_launches(self):
        return _lib.lib().sp_moe_kernel_launches(self._h)

    # -- weights
    def upload_layer(self, layer, weights, on_device=False):
        """weights: mapping or object with the fields of sp_moe_layer_weights (numpy arrays, or
        torch CUDA tensors when on_device)."""
        get = weights.get if isinstance(weights, dict) else (lambda k: getattr(weights, k, None))
        keep = [get(f) for f in WEIGHT_FIELDS]
        w = SpMoeLayerWeights(*[_ptr(a) for a in keep])
        fn = _lib.lib().sp_moe_upload_layer_dev if on_device else _lib.lib().sp_moe_upload_layer
        check(fn(self._h, layer, C.byref(w)))

    def load_sp_model(self, path, names=None):
        """Fills every layer from a `.sp-model` file through the library's own loader (sp_moe_load_sp_model).
        names: None, or 18 printf-style templates (see the header)."""
        arr = None
        if names is not None:
            if len(names) != 18:
                raise ValueError("names must hold 18 templates")
            arr = (C.c_char_p * 18)(*[n.encode() for n in names])
        check(_lib.lib().sp_moe_load_sp_model(self._h, str(path).encode(), arr))

    def set_router_bias(self, layer, bias):
        """Replaces the router's per-expert logit bias of one layer (torch CUDA f32 [NE], or None for no bias)."""
        check(_lib.lib().sp_moe_set_router_bias_dev(self._h, layer, _ptr(bias)))

    # -- forward
    def forward(self, x, layer_first=0, n_layers=None, flavour=FLAVOUR_DECODE, want_routing=True, out=None):
        """Host entry: x numpy [M][E] f32 -> (y, sel, wts); sel/wts are [n_layers][M][NU]. `out`: a caller-owned
        [M][E] f32 array for y (page-locked memory makes the copy back asynchronous)."""
        n_layers = self.n_layers - layer_first if n_layers is None else n_layers
        x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, self.cfg["E"])
        M = x.shape[0]
        y = np.empty_like(x) if out is None else out
        if y.shape != x.shape or y.dtype != np.float32 or not y.flags["C_CONTIGUOUS"]:
            raise ValueError("out must be a C-contiguous float32 array of x's shape")
        sel = np.empty((n_layers, M, self.cfg["NU"]), np.int32) if want_routing else None
        wts = np.empty((n_layers, M, self.cfg["NU"]), np.float32) if want_routing else None
        if self._trace.on and sel is None:           # the trace needs the routing even if the caller does not
            tsel = np.empty((n_layers, M, self.cfg["NU"]), np.int32); twts = np.empty((n_layers, M, self.cfg["NU"]), np.float32)
        else:
            tsel, twts = sel, wts
        check(_lib.lib().sp_moe_forward(self._h, layer_first, n_layers, flavour, M, _ptr(x), _ptr(y),
                                        _ptr(tsel), _ptr(twts)))
        self._trace.record(tsel, twts, layer_first)
        return y, sel, wts

    def decode_batch(self, x, layer_first=0, n_layers=None, want_routing=False):
        """B tokens through the layers in ONE call with one synchronisation, each in the single-token
        decode arithmetic: the MoE share of the reference's gemma4_kv_decode_batch
        (src/backends/cuda/cuda_forward.cu:11729-11757), which runs the B tokens as B sequential
        steps. Row t of the result is bit-identical to forward(x[t:t+1])."""
        return self.forward(x, layer_first, n_layers, FLAVOUR_DECODE, want_routing)

    def forward_dev(self, x, y, layer_first=0, n_layers=None, flavour=FLAVOUR_DECODE, sel=None, wts=None, stream=None):
        """Device entry: x, y torch CUDA f32 [M][E]; enqueues on `stream` (a torch stream; default
        the current one) and returns at once. Call status() to collect kernel-side errors."""
        import torch
        n_layers = self.n_layers - layer_first if n_layers is None else n_layers
        M = x.numel() // self.cfg["E"]
        st = (stream or torch.cuda.current_stream(x.device)).cuda_stream
        check(_lib.lib().sp_moe_forward_dev(self._h, layer_first, n_layers, flavour, M, x.data_ptr(), y.data_ptr(),
                                            _ptr(sel), _ptr(wts), st))

    def status(self):
        check(_lib.lib().sp_moe_status(self._h))

    def decode_timing(self):
        """Phase times (microseconds, device clock, CTA 0) of the last layer of the most recent single-token
        decode call; needs SP_MOE_TIMING=1 in the environment when the engine was created (the reference's
        switch for its `[g4-moe] TIMING` line, src/backends/cuda/cuda_forward.cu:7186-7201)."""
        t = _lib.SpMoeTiming()
        check(_lib.lib().sp_moe_decode_timing(self._h, C.byref(t)))
        names = ("router+shared", "topk+gate|up", "down+combine")
        return dict(layer_us=t.layer_us, raw_us=[[round(v, 3) for v in row] for row in t.raw_us], kernels={n: dict(wait_us=t.wait_us[k], prologue_us=t.prologue_us[k], rows_us=t.rows_us[k])
                                                   for k, n in enumerate(names)})

    def debug_wait_timeout(self, polls=4096):
        """Failure-path probe: a one-CTA kernel waits (at most `polls` polls) on a copy nobody starts; the
        wait gives up and the next status() raises the library's timeout error. Nothing hangs."""
        import torch
        check(_lib.lib().sp_moe_debug_wait_timeout(self._h, polls, torch.cuda.current_stream().cuda_stream))

    # -- one layer in three stages (expert-parallel runs move rows between them; see ep.py)
    def ep_route(self, layer, x, flavour=FLAVOUR_PREFILL, sel=None, wts=None, defer_shared=False, n_ranks=0, capacity=0):
        """x torch CUDA f32 [M][E] -> (sel_asc int32 [M][NU], cw f32 [M][NU], rows f32 sorted by expert,
        counts int32 [NE], pair_index int32 [M*NU]). rows is [M*NU][E], or with a capacity the padded send
        buffer [n_ranks*capacity][E] (rank r's rows start at r*capacity; unused rows are not initialised)."""
        import torch
        M, NU, NE = x.shape[0], self.cfg["NU"], self.cfg["NE"]
        sel_asc = torch.empty((M, NU), dtype=torch.int32, device=x.device)
        cw = torch.empty((M, NU), dtype=torch.float32, device=x.device)
        rows = torch.empty((n_ranks * capacity if capacity else M * NU, x.shape[1]), dtype=torch.float32, device=x.device)
        counts = torch.empty(NE, dtype=torch.int32, device=x.device)
        pair_index = torch.empty(M * NU, dtype=torch.int32, device=x.device)
        st = torch.cuda.current_stream(x.device).cuda_stream
        check(_lib.lib().sp_moe_ep_route_dev(self._h, layer, flavour, M, x.data_ptr(), sel_asc.data_ptr(), cw.data_ptr(),
                                             rows.data_ptr(), counts.data_ptr(), pair_index.data_ptr(), _ptr(sel), _ptr(wts),
                                             1 if defer_shared else 0, n_ranks, capacity, st))
        return sel_asc, cw, rows, counts, pair_index

    def ep_recv_layout(self, counts_all, rank, capacity):
        """counts_all torch CUDA int32 [n_ranks][NE] -> (offsets int32 [NE+1], row_index int32 [n_ranks*capacity])
        for the rows a padded exchange delivered to `rank`."""
        import torch
        n_ranks = counts_all.shape[0]
        offsets = torch.empty(self.cfg["NE"] + 1, dtype=torch.int32, device=counts_all.device)
        row_index = torch.empty(n_ranks * capacity, dtype=torch.int32, device=counts_all.device)
        check(_lib.lib().sp_moe_ep_recv_layout_dev(self._h, counts_all.contiguous().data_ptr(), n_ranks, rank, capacity, offsets.data_ptr(),
                                                   row_index.data_ptr(), torch.cuda.current_stream(counts_all.device).cuda_stream))
        return offsets, row_index

    def ep_shared(self, layer, M, flavour=FLAVOUR_PREFILL):
        """The shared expert of the tokens the last ep_route(defer_shared=True) call prepared."""
        import torch
        check(_lib.lib().sp_moe_ep_shared_dev(self._h, layer, flavour, M, torch.cuda.current_stream().cuda_stream))

    def ep_experts(self, layer, rows, offsets, flavour=FLAVOUR_PREFILL, row_index=None):
        """rows torch CUDA f32 [R][E], offsets int32 [NE+1]; sorted position p is row row_index[p]
        (int32; None = rows already sorted by expert) -> the experts' outputs, same row order as `rows`."""
        import torch
        out = torch.empty_like(rows)
        st = torch.cuda.current_stream(rows.device).cuda_stream
        check(_lib.lib().sp_moe_ep_experts_dev(self._h, layer, flavour, rows.shape[0], rows.data_ptr(), _ptr(row_index),
                                               offsets.data_ptr(), out.data_ptr(), st))
        return out

    def ep_finish(self, layer, x, pair_rows, pair_index=None):
        """x [M][E]; token t's k-th expert output (ascending expert id) is row pair_index[t*NU+k] of
        pair_rows (int32; None = row t*NU+k) -> y [M][E]."""
        import torch
        y = torch.empty_like(x)
        st = torch.cuda.current_stream(x.device).cuda_stream
        check(_lib.lib().sp_moe_ep_finish_dev(self._h, layer, x.shape[0], x.data_ptr(), pair_rows.data_ptr(), _ptr(pair_index),
                                              y.data_ptr(), st))
        return y


class MoeExt:
    """The reference's MoE plugin hook (SwiGLU experts, separate gate/up/down tensors, host router):
    sp_q36gpu_upload_experts / sp_q36gpu_moe of src/backends/cuda/cuda_forward.cu:16203-16289."""

    def __init__(self, device=0):
        self._h = C.c_void_p()
        if _lib.lib().sp_moe_ext_open(device, C.byref(self._h)) != 0:
            raise _lib.SpMoeError(1, (_lib.lib().sp_last_error() or b"").decode())

    def upload_experts(self, tag, gate, gate_bs, up, up_bs, down, down_bs, NE, FF, E):
        """numpy arrays in the reference's layouts (codes uint8, scales uint16 holding f16 bits)."""
        arrs = [np.ascontiguousarray(a) for a in (gate, gate_bs, up, up_bs, down, down_bs)]
        if _lib.lib().sp_moe_ext_upload_experts(self._h, tag.encode(), *[a.ctypes.data for a in arrs], NE, FF, E) != 0:
            raise _lib.SpMoeError(1, (_lib.lib().sp_last_error() or b"").decode())

    def moe(self, tag, idx, wt, x, FF):
        """Returns y [E], or None when the hook answers "not mine"."""
        idx = np.ascontiguousarray(idx, np.int32); wt = np.ascontiguousarray(wt, np.float32); x = np.ascontiguousarray(x, np.float32)
        y = np.empty_like(x)
        rc = _lib.lib().sp_moe_ext_moe(self._h, tag.encode(), idx.ctypes.data, wt.ctypes.data, idx.size, x.ctypes.data, x.size, FF, y.ctypes.data)
        return y if rc == 0 else None

    def close(self):
        if getattr(self, "_h", None) is not None and self._h.value:
            _lib.lib().sp_moe_ext_close(self._h)
            self._h = C.c_void_p()

    __del__ = close


def q4b_quantize(w):
    """torch CUDA f32 [rows][cols] -> (codes uint8 [rows][cols/2], scales int16-view f16 [rows][cols/32])."""
    import torch
    rows, cols = w.shape
    w = w.contiguous()
    codes = torch.empty((rows, cols // 2), dtype=torch.uint8, device=w.device)
    bs = torch.empty((rows, cols // 32), dtype=torch.int16, device=w.device)
    check(_lib.lib().sp_moe_q4b_quantize_dev(w.data_ptr(), rows, cols, codes.data_ptr(), bs.data_ptr(),
                                             torch.cuda.current_stream(w.device).cuda_stream))
    return codes, bs


def q4b_dequantize(codes, bs):
    import torch
    rows, cols = codes.shape[0], codes.shape[1] * 2
    w = torch.empty((rows, cols), dtype=torch.float32, device=codes.device)
    check(_lib.lib().sp_moe_q4b_dequantize_dev(codes.data_ptr(), bs.data_ptr(), rows, cols, w.data_ptr(),
                                               torch.cuda.current_stream(codes.device).cuda_stream))
    return w


def gelu_mul(g, up):
    """torch CUDA f32 tensors -> gelu_tanh(g) * up (k_gelu_mul of the reference)."""
    import torch
    g, up = g.contiguous(), up.contiguous()
    out = torch.empty_like(g)
    check(_lib.lib().sp_moe_gelu_mul_dev(g.data_ptr(), up.data_ptr(), g.numel(), out.data_ptr(),
                                         torch.cuda.current_stream(g.device).cuda_stream))
    return out


def gemv_q4b(codes, bs, x):
    """torch CUDA tensors: codes uint8 [rows][in/2], bs int16 [rows][in/32], x f32 [in] -> y f32 [rows]
    (gemv_w_packed of the reference: int8 activation quant + Q4B x int8 GEMV)."""
    import torch
    rows, cols = codes.shape[0], codes.shape[1] * 2
    y = torch.empty(rows, dtype=torch.float32, device=codes.device)
    check(_lib.lib().sp_moe_gemv_q4b_dev(codes.data_ptr(), bs.data_ptr(), cols, rows, x.contiguous().data_ptr(), y.data_ptr(),
                                         torch.cuda.current_stream(codes.device).cuda_stream))
    return y


def int_gemm_scaled(A, B, scale_a, scale_b, packed_int4=False):
    """The reference's quantised GEMM (ptx_mma.cuh): torch CUDA tensors A [M][K], B [N][K] int8 (or uint8
    [.][K/2] packed signed int4), scales f32 [M], [N] -> C f16 [M][N] = f16(float(A.B^T) * sa[m] * sb[n])."""
    import torch
    A, B = A.contiguous(), B.contiguous()
    M, N = A.shape[0], B.shape[0]
    K = A.shape[1] * (2 if packed_int4 else 1)
    Cc = torch.empty((M, N), dtype=torch.float16, device=A.device)
    fn = _lib.lib().sp_frob_matmul_q4_dev if packed_int4 else _lib.lib().sp_frob_matmul_q8_dev
    check(fn(A.data_ptr(), B.data_ptr(), scale_a.contiguous().data_ptr(), scale_b.contiguous().data_ptr(), Cc.data_ptr(), M, K, N,
             torch.cuda.current_stream(A.device).cuda_stream))
    return Cc
