/* ep_nccl.cu — the expert-parallel prefill loop behind the C ABI: one call runs a range of layers over
 * n_ranks GPUs (one process each), NCCL doing the two exchanges of every layer.
 *
 * The reference is single-GPU: its batched branch walks every expert on the one device (CF:8925-8965 of
 * src/backends/cuda/cuda_forward.cu). Here tokens are data-parallel (each rank owns the residual of its own
 * tokens, the router, the shared expert and the norms) and the routed experts are partitioned contiguously,
 * NE / n_ranks per rank. Per layer and token slice:
 *
 *   route (local) -> all-gather of the per-expert pair counts -> dispatch (all-to-all of the input rows)
 *   -> experts (on the owner) -> combine (all-to-all of the output rows back) -> finish (local)
 *
 * Every NCCL call runs on an internal communication stream, every kernel on the caller's stream, and events
 * order them, so with two or more token slices the dispatch of one slice and the combine of another run under
 * the experts stage of a third, and the last combine of a layer runs under the first route of the next.
 * The per-token combine still walks the experts in ascending id on the home rank: the result is bit-identical
 * to sp_moe_forward_dev on one GPU.
 *
 * Two exchanges. Padded (capacity_rows > 0): every rank sends the same number of rows to every rank, the
 * receive layout is built on the device, nothing waits for the host, and the whole call can be captured into a
 * CUDA graph; a block that does not fit is reported by sp_moe_status. Exact (capacity_rows == 0): the split
 * sizes are read on the host once per layer (one slice, no overlap).
 *
 * How the rows travel. NCCL send/recv pairs in a world of more than four ranks. Up to four (or with SP_MOE_EP_EXCHANGE=copy)
 * every rank maps the other ranks' exchange buffers through CUDA IPC once, pushes its blocks with plain
 * device-to-device copies (copy engines: no SM is taken from the GEMMs that run beside them) and a one-int
 * all-reduce tells each rank that its blocks have landed. A buffer is only overwritten after its reader is
 * done: a rank's dispatch of layer L+1 follows its finish of layer L, which needed every peer's combine of
 * layer L, which followed that peer's experts stage - the last reader of the buffer the dispatch writes; the
 * combine's buffer is protected the same way by the dispatch of the same layer.
 * With one token slice the shared expert is split around the experts stage: its gate/up GEMM runs under the
 * dispatch, its down GEMM under the combine.
 *
 * What the dispatch carries. In the padded exchange a token's input row goes to a destination rank once, however
 * many of its NU experts live there (blocks of min(capacity, max_tokens) token rows, which cannot overflow), with
 * a 4-byte slot per pair in the padded pair order; the receiver turns the slots into a gather index for its GEMMs'
 * input rows and still writes one output row per pair (SP_MOE_EP_DISPATCH=rows sends one row per pair instead).
 * The exact exchange sends one row per pair.
 *
 * NCCL is not linked: its entry points are looked up at run time (the copy the process already holds - e.g. the
 * one a framework loaded - or libnccl.so.2 from the loader's path), so a daemon that never runs
 * expert-parallel needs no NCCL at all. No load uses cluster multicast; a peer's memory is only ever the
 * destination of a device-to-device copy.
 */
#include "handle.cuh"
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <dlfcn.h>
#include <mutex>
#include <new>
#include <vector>

namespace {

/* the handful of NCCL declarations this file needs (nccl.h: opaque communicator, 128-byte unique id) */
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclInt8 = 0, ncclInt32 = 2, ncclFloat32 = 7 };
enum { ncclSum = 0, ncclMin = 3 };

struct Nccl {
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t);      /* optional: only the peer-copy exchange needs it */
    ncclResult_t (*Send)(const void *, size_t, int, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*Recv)(void *, size_t, int, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*GroupStart)();
    ncclResult_t (*GroupEnd)();
    const char *(*GetErrorString)(ncclResult_t);
    bool ok = false;
};
Nccl g_nccl;
std::once_flag g_nccl_once;

const Nccl *nccl() {
    std::call_once(g_nccl_once, [] {
        void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);      /* an already-loaded copy with this name is reused */
        if (!lib) lib = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!lib) return;
        auto sym = [&](const char *n) { return dlsym(lib, n); };
        g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))sym("ncclGetUniqueId");
        g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))sym("ncclCommInitRank");
        g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))sym("ncclCommDestroy");
        g_nccl.AllGather = (decltype(g_nccl.AllGather))sym("ncclAllGather");
        g_nccl.AllReduce = (decltype(g_nccl.AllReduce))sym("ncclAllReduce");
        g_nccl.Send = (decltype(g_nccl.Send))sym("ncclSend");
        g_nccl.Recv = (decltype(g_nccl.Recv))sym("ncclRecv");
        g_nccl.GroupStart = (decltype(g_nccl.GroupStart))sym("ncclGroupStart");
        g_nccl.GroupEnd = (decltype(g_nccl.GroupEnd))sym("ncclGroupEnd");
        g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))sym("ncclGetErrorString");
        g_nccl.ok = g_nccl.GetUniqueId && g_nccl.CommInitRank && g_nccl.CommDestroy && g_nccl.AllGather && g_nccl.Send && g_nccl.Recv &&
                    g_nccl.GroupStart && g_nccl.GroupEnd && g_nccl.GetErrorString;
    });
    return g_nccl.ok ? &g_nccl : nullptr;
}

int fail(int code, const char *fmt, ...) {
    char msg[512];
    va_list ap; va_start(ap, fmt); vsnprintf(msg, sizeof msg, fmt, ap); va_end(ap);
    sp_set_error(msg);
    return code;
}
#define CK(call, where) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail(e_ == cudaErrorMemoryAllocation ? SP_MOE_EBACKEND_OOM : SP_MOE_ECUDA, "sp_moe_ep_forward_dev: %s: %s", where, cudaGetErrorString(e_)); } while (0)
int fail_nccl(const char *where, const char *what) {
    char msg[512];
    snprintf(msg, sizeof msg, "sp_moe_ep_forward_dev: %s: NCCL: %s", where, what ? what : "?");
    sp_set_error(msg);
    return SP_MOE_ECUDA;
}
#define NK(call, where) do { ncclResult_t r_ = (call); if (r_ != 0) return fail_nccl(where, N->GetErrorString(r_)); } while (0)

constexpr int kMaxSlices = SP_BATCHED_MAX_SLICES;

struct Slice {                      /* everything one token slice keeps between its stages */
    int32_t *sel_asc, *counts, *pair_index, *counts_all, *offsets, *row_index;
    float *cw, *send, *recv, *out, *back;
    int32_t *ti_send, *ti_recv, *slot, *in_index;   /* token dispatch: per-pair token slots (sent / received), scan scratch, the receiver's input index */
    cudaEvent_t routed, gathered, dispatched, computed, combined;
};
struct EpState {
    int device, n_ranks, max_tokens, rows_cap;      /* rows_cap: rows each of send / recv / out / back holds */
    unsigned char *base; size_t bytes;
    float *xa, *xb;                                 /* residual between layers */
    Slice sl[kMaxSlices];
    int32_t *counts_host;                           /* page-locked, exact exchange */
    cudaStream_t comm;                              /* every NCCL call */
    cudaStream_t local;                             /* peer-copy exchange: this rank's own block, beside the copies to the peers */
    cudaEvent_t fork, joined;
    long long last_rows;
    /* peer-copy exchange: every rank maps every other rank's arena (CUDA IPC) and pushes its blocks with device-to-device
     * copies; NCCL then only carries the counts and a one-int all-reduce that tells a rank its blocks have landed */
    int p2p;                                        /* 0 = not tried yet, 1 = in use, -1 = unavailable (NCCL send/recv instead) */
    unsigned char *peer_base[64];
    size_t o_recv, o_back, o_tir;                   /* where recv / back / ti_recv sit in every rank's arena (same layout everywhere) */
    int token_dispatch;                             /* padded exchange: each token's row travels once per destination (SP_MOE_EP_DISPATCH=rows switches it off) */
    int32_t *sync_dev;                              /* [4] ints for the landing all-reduce + 64 bytes per rank of IPC handles */
    bool timed;                                     /* SP_MOE_TIMING=1 at open: events carry time, begin/end bracket every layer */
    cudaEvent_t begin, end;
    bool timing_valid;                              /* the last call ran outside a stream capture with one slice */
};

void ep_free(void *p) {
    EpState *s = (EpState *)p;
    if (!s) return;
    cudaSetDevice(s->device);
    if (s->comm) { cudaStreamSynchronize(s->comm); cudaStreamDestroy(s->comm); }
    for (auto &x : s->sl) for (cudaEvent_t e : {x.routed, x.gathered, x.dispatched, x.computed, x.combined}) if (e) cudaEventDestroy(e);
    for (int r = 0; r < 64; r++) if (s->peer_base[r]) cudaIpcCloseMemHandle(s->peer_base[r]);
    if (s->sync_dev) cudaFree(s->sync_dev);
    if (s->fork) cudaEventDestroy(s->fork);
    if (s->joined) cudaEventDestroy(s->joined);
    if (s->local) cudaStreamDestroy(s->local);
    if (s->begin) cudaEventDestroy(s->begin);
    if (s->end) cudaEventDestroy(s->end);
    if (s->base) cudaFree(s->base);
    if (s->counts_host) cudaFreeHost(s->counts_host);
    delete s;
}

/* rows the exchange buffers hold: the handle's max_expert_rows covers both the worst exact exchange and
 * n_ranks * capacity of a padded one (sp_moe_ep_recv_layout_dev checks the same bound) */
int ep_ensure(sp_moe *h, int n_ranks, EpState **out) {
    EpState *s = (EpState *)h->ep_state;
    if (s && s->n_ranks == n_ranks) { *out = s; return SP_MOE_OK; }
    if (s) { ep_free(s); h->ep_state = nullptr; }
    s = new (std::nothrow) EpState();
    if (!s) return fail(SP_MOE_ENOMEM, "sp_moe_ep_forward_dev: host OOM");
    memset(s, 0, sizeof *s);
    s->device = h->device; s->n_ranks = n_ranks; s->max_tokens = h->cfg.max_tokens; s->rows_cap = h->bs.max_rows;
    s->timed = h->stamps != nullptr;                    /* the handle was opened with SP_MOE_TIMING=1 */
    const size_t E = h->cfg.E, NE = h->cfg.NE, NU = h->cfg.NU, MT = (size_t)s->max_tokens, R = (size_t)s->rows_cap;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    /* the slices share the token range and the row buffers: slice k of n uses its own part of each */
    size_t o = 0;
    auto take = [&](size_t bytes) { const size_t at = o; o = up(o + bytes); return at; };
    const size_t o_xa = take(4 * MT * E), o_xb = take(4 * MT * E), o_sel = take(4 * MT * NU), o_cw = take(4 * MT * NU), o_pi = take(4 * MT * NU);
    const size_t o_cnt = take(4 * NE * kMaxSlices), o_call = take(4 * NE * (size_t)n_ranks * kMaxSlices), o_off = take(4 * (NE + 1) * kMaxSlices), o_ri = take(4 * R);
    const size_t o_send = take(4 * R * E), o_recv = take(4 * R * E), o_out = take(4 * R * E), o_back = take(4 * R * E);
    const size_t o_tis = take(4 * R), o_tir = take(4 * R), o_slot = take(4 * MT * (size_t)n_ranks), o_ii = take(4 * R);
    s->bytes = o; s->o_recv = o_recv; s->o_back = o_back; s->o_tir = o_tir;
    { const char *dv = getenv("SP_MOE_EP_DISPATCH"); s->token_dispatch = !(dv && dv[0] == 'r'); }
    cudaError_t e = cudaMalloc(&s->base, s->bytes);
    if (e != cudaSuccess) { delete s; return fail(SP_MOE_EBACKEND_OOM, "sp_moe_ep_forward_dev: exchange buffers (%lld MB): cuda error %lld", (long long)(o >> 20), (long long)e); }
    unsigned char *b = s->base;
    s->xa = (float *)(b + o_xa); s->xb = (float *)(b + o_xb);
    for (int k = 0; k < kMaxSlices; k++) {
        Slice &x = s->sl[k];
        x.sel_asc = (int32_t *)(b + o_sel); x.cw = (float *)(b + o_cw); x.pair_index = (int32_t *)(b + o_pi);          /* + token offset at use */
        x.counts = (int32_t *)(b + o_cnt) + (size_t)k * NE; x.counts_all = (int32_t *)(b + o_call) + (size_t)k * NE * n_ranks;
        x.offsets = (int32_t *)(b + o_off) + (size_t)k * (NE + 1); x.row_index = (int32_t *)(b + o_ri);                  /* + row offset at use */
        x.send = (float *)(b + o_send); x.recv = (float *)(b + o_recv); x.out = (float *)(b + o_out); x.back = (float *)(b + o_back);
        x.ti_send = (int32_t *)(b + o_tis); x.ti_recv = (int32_t *)(b + o_tir); x.slot = (int32_t *)(b + o_slot); x.in_index = (int32_t *)(b + o_ii);   /* + row / token offset at use */
        for (cudaEvent_t *ev : {&x.routed, &x.gathered, &x.dispatched, &x.computed, &x.combined})
            if (cudaEventCreateWithFlags(ev, s->timed ? cudaEventDefault : cudaEventDisableTiming) != cudaSuccess) { ep_free(s); return fail(SP_MOE_ECUDA, "sp_moe_ep_forward_dev: event creation failed"); }
    }
    if (s->timed && (cudaEventCreate(&s->begin) != cudaSuccess || cudaEventCreate(&s->end) != cudaSuccess)) { ep_free(s); return fail(SP_MOE_ECUDA, "sp_moe_ep_forward_dev: event creation failed"); }
    if (cudaMallocHost((void **)&s->counts_host, 4 * NE * (size_t)n_ranks) != cudaSuccess || cudaStreamCreateWithFlags(&s->comm, cudaStreamNonBlocking) != cudaSuccess ||
        cudaStreamCreateWithFlags(&s->local, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreateWithFlags(&s->fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s->joined, cudaEventDisableTiming) != cudaSuccess) {
        ep_free(s); return fail(SP_MOE_ECUDA, "sp_moe_ep_forward_dev: stream / pinned buffer creation failed");
    }
    h->ep_state = s; h->ep_state_free = ep_free;
    h->scratch_bytes += s->bytes;
    *out = s;
    return SP_MOE_OK;
}

/* Maps every peer's exchange arena into this process (once per handle and world size, outside any stream capture).
 * All ranks must end up in the same mode, so the outcome is agreed on with a min all-reduce. */
int ep_p2p_setup(EpState *s, const Nccl *N, ncclComm_t comm, int n_ranks, int rank) {
    s->p2p = -1;
    if (!N->AllReduce || n_ranks > 64) return SP_MOE_OK;
    /* measured on B200 / NVSwitch, 4096 tokens: a copy engine moves a block at ~750 GB/s against ~310 GB/s for an NCCL
     * send/recv pair, but the copies of one rank are queued one after the other (destinations staggered so that every rank
     * receives one copy at a time) and a one-int all-reduce follows them. 2 GPUs: 69.8 K -> 80.3 K tokens/s with copies;
     * 4 GPUs: 0.865 against 0.972 ms per layer; 8 GPUs: 0.704 against 0.594 ms per layer (seven small copies and the
     * all-reduce cost more than NCCL's concurrent pairs). So: copies up to four ranks, NCCL beyond;
     * SP_MOE_EP_EXCHANGE=copy|nccl overrides. */
    const char *ev = getenv("SP_MOE_EP_EXCHANGE");
    int ok = ev && ev[0] == 'c' ? 1 : (ev && ev[0] == 'n' ? 0 : (n_ranks <= 4 ? 1 : 0));
    if (cudaMalloc((void **)&s->sync_dev, 16 + 64 * (size_t)n_ranks) != cudaSuccess) { cudaGetLastError(); s->sync_dev = nullptr; return SP_MOE_OK; }
    unsigned char *hd = reinterpret_cast<unsigned char *>(s->sync_dev) + 16;
    cudaIpcMemHandle_t mine;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (cudaIpcGetMemHandle(&mine, s->base) != cudaSuccess) { cudaGetLastError(); ok = 0; memset(&mine, 0, sizeof mine); }
    std::vector<cudaIpcMemHandle_t> all((size_t)n_ranks);
    CK(cudaMemcpyAsync(hd + 64 * (size_t)rank, &mine, 64, cudaMemcpyHostToDevice, s->comm), "handle H2D");
    NK(N->AllGather(hd + 64 * (size_t)rank, hd, 64, ncclInt8, comm, s->comm), "all-gather of the IPC handles");
    CK(cudaMemcpyAsync(all.data(), hd, 64 * (size_t)n_ranks, cudaMemcpyDeviceToHost, s->comm), "handles D2H");
    CK(cudaStreamSynchronize(s->comm), "stream synchronize");
    for (int r = 0; r < n_ranks && ok; r++) {
        if (r == rank) continue;
        void *p = nullptr;
        if (cudaIpcOpenMemHandle(&p, all[r], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); ok = 0; break; }
        s->peer_base[r] = (unsigned char *)p;
    }
    int agreed = 0;
    CK(cudaMemcpyAsync(s->sync_dev, &ok, 4, cudaMemcpyHostToDevice, s->comm), "flag H2D");
    NK(N->AllReduce(s->sync_dev, s->sync_dev + 1, 1, ncclInt32, ncclMin, comm, s->comm), "all-reduce of the mode");
    CK(cudaMemcpyAsync(&agreed, s->sync_dev + 1, 4, cudaMemcpyDeviceToHost, s->comm), "flag D2H");
    CK(cudaStreamSynchronize(s->comm), "stream synchronize");
    CK(cudaMemsetAsync(s->sync_dev, 0, 16, s->comm), "memset");
    if (agreed == 1) s->p2p = 1;
    else for (int r = 0; r < 64; r++) if (s->peer_base[r]) { cudaIpcCloseMemHandle(s->peer_base[r]); s->peer_base[r] = nullptr; }
    return SP_MOE_OK;
}

}  // namespace

/* ---------------------------------------------------------------- communicator helpers */
extern "C" int sp_moe_ep_unique_id(void *id128) {
    const Nccl *N = nccl();
    if (!N) return fail(SP_MOE_EUNSUPPORTED, "sp_moe_ep_unique_id: libnccl.so.2 is not available to this process");
    if (!id128) return fail(SP_MOE_EBADARG, "sp_moe_ep_unique_id: NULL argument");
    ncclUniqueId id;
    const ncclResult_t r = N->GetUniqueId(&id);
    if (r != 0) return fail(SP_MOE_ECUDA, "sp_moe_ep_unique_id: NCCL: %s", N->GetErrorString(r));
    memcpy(id128, &id, sizeof id);
    return SP_MOE_OK;
}
extern "C" int sp_moe_ep_comm_create(const void *id128, int n_ranks, int rank, void **comm_out) {
    const Nccl *N = nccl();
    if (!N) return fail(SP_MOE_EUNSUPPORTED, "sp_moe_ep_comm_create: libnccl.so.2 is not available to this process");
    if (!id128 || !comm_out || n_ranks <= 0 || rank < 0 || rank >= n_ranks) return fail(SP_MOE_EBADARG, "sp_moe_ep_comm_create: bad argument");
    ncclUniqueId id; memcpy(&id, id128, sizeof id);
    ncclComm_t c = nullptr;
    const ncclResult_t r = N->CommInitRank(&c, n_ranks, id, rank);      /* on the CUDA device current in this thread */
    if (r != 0) return fail(SP_MOE_ECUDA, "sp_moe_ep_comm_create: NCCL: %s", N->GetErrorString(r));
    *comm_out = c;
    return SP_MOE_OK;
}
extern "C" int sp_moe_ep_comm_destroy(void *comm) {
    const Nccl *N = nccl();
    if (!comm) return SP_MOE_OK;
    if (!N) return fail(SP_MOE_EUNSUPPORTED, "sp_moe_ep_comm_destroy: libnccl.so.2 is not available to this process");
    const ncclResult_t r = N->CommDestroy((ncclComm_t)comm);
    return r == 0 ? SP_MOE_OK : fail(SP_MOE_ECUDA, "sp_moe_ep_comm_destroy: NCCL: %s", N->GetErrorString(r));
}
extern "C" long long sp_moe_ep_last_rows(const sp_moe *h) { return (h && h->ep_state) ? ((const EpState *)h->ep_state)->last_rows : 0; }

/* ---------------------------------------------------------------- the layer loop */
extern "C" int sp_moe_ep_forward_dev(sp_moe *h, void *nccl_comm, int n_ranks, int rank, int lf, int nl, int flavour, int M,
                                     const float *x_dev, float *y_dev, int capacity_rows, int slices, void *stream) {
    const Nccl *N = nccl();
    if (!N) return fail(SP_MOE_EUNSUPPORTED, "sp_moe_ep_forward_dev: libnccl.so.2 is not available to this process");
    if (!h || !nccl_comm || !x_dev || !y_dev) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: NULL argument");
    const sp_moe_config &c = h->cfg;
    if (n_ranks <= 0 || c.NE % n_ranks || rank < 0 || rank >= n_ranks) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: need 0 <= rank < n_ranks and n_ranks dividing NE");
    if (lf < 0 || nl <= 0 || lf + nl > c.n_layers) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: layers out of range");
    if (M <= 0 || M > c.max_tokens) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: M=%d outside (0, max_tokens=%d]", M, c.max_tokens);
    if (flavour != SP_MOE_FLAVOUR_DECODE && flavour != SP_MOE_FLAVOUR_PREFILL) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: unknown flavour");
    for (int L = lf; L < lf + nl; L++) if (!h->uploaded[L]) return fail(SP_MOE_EBADSTATE, "sp_moe_ep_forward_dev: layer %d has no weights uploaded", L);
    if (capacity_rows < 0) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: capacity_rows must not be negative");
    const bool padded = capacity_rows > 0;
    int ns = padded ? (slices < 1 ? 1 : (slices > kMaxSlices ? kMaxSlices : slices)) : 1;
    if (ns > M) ns = M;
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    EpState *s = nullptr;
    { const int rc = ep_ensure(h, n_ranks, &s); if (rc) return rc; }
    const int E = c.E, NE = c.NE, NU = c.NU, epr = NE / n_ranks;
    /* per-slice capacity: the per-destination room of the whole call split over the slices, in multiples of 8 rows */
    const int cap = padded ? ((capacity_rows + ns - 1) / ns + 7) / 8 * 8 : 0;
    if (padded && (long long)n_ranks * cap * ns > s->rows_cap)
        return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: %d slices x n_ranks x %d rows = %lld rows exceed max_expert_rows = %d", ns, cap, (long long)n_ranks * cap * ns, s->rows_cap);
    if (!padded && (long long)M * NU > s->rows_cap) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: M * NU exceeds max_expert_rows");
    cudaStream_t st = (cudaStream_t)stream, cs = s->comm;
    ncclComm_t comm = (ncclComm_t)nccl_comm;
    h->last_stream = st;
    int nlaunch = 0, nlk = 0;
    const SpDims &d = h->d;
    /* token range and row range of every slice */
    int t0[kMaxSlices], tm[kMaxSlices]; size_t r0[kMaxSlices];
    for (int k = 0; k < ns; k++) { t0[k] = (int)((long long)M * k / ns); tm[k] = (int)((long long)M * (k + 1) / ns) - t0[k]; r0[k] = padded ? (size_t)k * n_ranks * cap : 0; }

    if (s->p2p == 0) {                                    /* first call for this world: map the peers' buffers (not possible inside a capture) */
        cudaStreamCaptureStatus cst = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(st, &cst) == cudaSuccess && cst == cudaStreamCaptureStatusNone) {
            const int rc = ep_p2p_setup(s, N, comm, n_ranks, rank);
            if (rc) return rc;
        }
    }
    const bool p2p = s->p2p == 1;
    /* token dispatch (padded exchange): a destination never gets more distinct tokens than this rank may hold, so blocks
     * of min(capacity, max_tokens) token rows cannot overflow; every rank derives the same size from the shared config */
    const bool tokd = padded && s->token_dispatch;
    const int capT = tokd ? (cap < (c.max_tokens + 7) / 8 * 8 ? cap : (c.max_tokens + 7) / 8 * 8) : 0;
    /* this rank's own block: a copy on a stream of its own, forked from the communication stream before the copies to
     * the peers are queued there and joined back after them, so that it runs beside them */
    auto own_fork = [&](void *dstp, const void *srcp, size_t bytes, void *dst2 = nullptr, const void *src2 = nullptr, size_t bytes2 = 0) -> cudaError_t {
        cudaError_t e2 = cudaEventRecord(s->fork, s->comm);
        if (e2 == cudaSuccess) e2 = cudaStreamWaitEvent(s->local, s->fork, 0);
        if (e2 == cudaSuccess && bytes) e2 = cudaMemcpyAsync(dstp, srcp, bytes, cudaMemcpyDeviceToDevice, s->local);
        if (e2 == cudaSuccess && bytes2) e2 = cudaMemcpyAsync(dst2, src2, bytes2, cudaMemcpyDeviceToDevice, s->local);
        if (e2 == cudaSuccess) e2 = cudaEventRecord(s->joined, s->local);
        return e2;
    };
    auto own_join = [&]() -> cudaError_t { return cudaStreamWaitEvent(s->comm, s->joined, 0); };
    bool timing = false;
    if (s->timed && ns == 1) {
        cudaStreamCaptureStatus cst = cudaStreamCaptureStatusNone;
        timing = cudaStreamIsCapturing(st, &cst) == cudaSuccess && cst == cudaStreamCaptureStatusNone;
    }
    const float *cur = x_dev;
    for (int li = 0; li < nl; li++) {
        const int L = lf + li;
        const SpLayerDev &W = h->layers_host[L];
        float *dst = (li == nl - 1) ? y_dev : ((li & 1) ? s->xb : s->xa);
        if (timing && li == nl - 1) CK(cudaEventRecord(s->begin, st), "event record");
        if (padded) {
            /* ---- route every slice; its count gather and its dispatch follow on the communication stream */
            for (int k = 0; k < ns; k++) {
                Slice &x = s->sl[k];
                cudaError_t e = sp_batched_ep_route(d, W, flavour, tm[k], cur + (size_t)t0[k] * E, x.sel_asc + (size_t)t0[k] * NU, x.cw + (size_t)t0[k] * NU,
                                                    tokd ? nullptr : x.send + r0[k] * E, x.counts, x.pair_index + (size_t)t0[k] * NU, nullptr, nullptr, 1, n_ranks, cap,
                                                    &h->bs, h->status, st, &nlk, t0[k], k);
                nlaunch += nlk;
                CK(e, "route");
                if (tokd) {                                   /* token rows per destination + every pair's token slot, instead of one row per pair */
                    e = sp_batched_ep_tokens(d, tm[k], n_ranks, cap, capT, x.sel_asc + (size_t)t0[k] * NU, x.pair_index + (size_t)t0[k] * NU, x.send + r0[k] * E,
                                             x.ti_send + r0[k], x.slot + (size_t)t0[k] * n_ranks, &h->bs, h->status, st, &nlk, t0[k], k);
                    nlaunch += nlk;
                    CK(e, "token dispatch");
                }
                CK(cudaEventRecord(x.routed, st), "event record");
                CK(cudaStreamWaitEvent(cs, x.routed, 0), "event wait");
                NK(N->AllGather(x.counts, x.counts_all, (size_t)NE, ncclInt32, comm, cs), "all-gather of the counts");
                CK(cudaEventRecord(x.gathered, cs), "event record");
                const size_t drows = tokd ? (size_t)capT : (size_t)cap;      /* rows per destination block of the dispatch */
                if (p2p) {                                    /* push block r into rank r's receive buffer, slot `rank`; then learn that every block has landed */
                    CK(own_fork(x.recv + (r0[k] + rank * drows) * E, x.send + (r0[k] + rank * drows) * E, drows * E * 4,
                                x.ti_recv + r0[k] + (size_t)rank * cap, x.ti_send + r0[k] + (size_t)rank * cap, tokd ? (size_t)cap * 4 : 0), "own block");
                    for (int i = 1; i < n_ranks; i++) {           /* rank + 1, rank + 2, ...: at every step each rank is the destination of exactly one copy */
                        const int r = (rank + i) % n_ranks;
                        float *dstb = reinterpret_cast<float *>(s->peer_base[r] + s->o_recv);
                        CK(cudaMemcpyAsync(dstb + (r0[k] + rank * drows) * E, x.send + (r0[k] + r * drows) * E, drows * E * 4, cudaMemcpyDeviceToDevice, cs), "dispatch copy");
                        if (tokd) CK(cudaMemcpyAsync(reinterpret_cast<int32_t *>(s->peer_base[r] + s->o_tir) + r0[k] + (size_t)rank * cap, x.ti_send + r0[k] + (size_t)r * cap,
                                                     (size_t)cap * 4, cudaMemcpyDeviceToDevice, cs), "dispatch copy (slots)");
                    }
                    CK(own_join(), "own block");
                    if (n_ranks > 1) NK(N->AllReduce(s->sync_dev, s->sync_dev + 1, 1, ncclInt32, ncclSum, comm, cs), "landing all-reduce");
                } else {
                    NK(N->GroupStart(), "group start");
                    for (int r = 0; r < n_ranks; r++) {
                        NK(N->Send(x.send + (r0[k] + r * drows) * E, drows * E, ncclFloat32, r, comm, cs), "dispatch send");
                        NK(N->Recv(x.recv + (r0[k] + r * drows) * E, drows * E, ncclFloat32, r, comm, cs), "dispatch recv");
                        if (tokd) {
                            NK(N->Send(x.ti_send + r0[k] + (size_t)r * cap, (size_t)cap, ncclInt32, r, comm, cs), "dispatch send (slots)");
                            NK(N->Recv(x.ti_recv + r0[k] + (size_t)r * cap, (size_t)cap, ncclInt32, r, comm, cs), "dispatch recv (slots)");
                        }
                    }
                    NK(N->GroupEnd(), "group end");
                }
                CK(cudaEventRecord(x.dispatched, cs), "event record");
            }
            /* ---- per slice: the shared expert and the receive layout (under the dispatch), the experts, the combine */
            for (int k = 0; k < ns; k++) {
                Slice &x = s->sl[k];
                /* the counts first (a tiny collective that must not queue behind a GEMM that fills every SM), then the
                 * shared expert under the dispatch. With one slice only its gate/up half goes here and its down half
                 * runs under the combine; with more slices the halves would share one hidden-vector scratch. */
                CK(cudaStreamWaitEvent(st, x.gathered, 0), "event wait");
                cudaError_t e = sp_batched_ep_shared(d, W, flavour, tm[k], &h->bs, h->status, st, &nlk, t0[k], k, ns == 1 ? 1 : 0);
                nlaunch += nlk;
                CK(e, "shared expert");
                e = sp_batched_ep_recv_layout(d, x.counts_all, n_ranks, rank, cap, x.offsets, x.row_index + r0[k], st, &nlk);
                nlaunch += nlk;
                CK(e, "receive layout");
                CK(cudaStreamWaitEvent(st, x.dispatched, 0), "event wait");
                if (tokd) {
                    e = sp_batched_ep_in_index(x.row_index + r0[k], x.ti_recv + r0[k], n_ranks, cap, capT, x.in_index + r0[k], st, &nlk);
                    nlaunch += nlk;
                    CK(e, "input index");
                }
                e = sp_batched_ep_experts(d, W, flavour, n_ranks * cap, x.recv + r0[k] * E, x.row_index + r0[k], x.offsets, x.out + r0[k] * E, &h->bs, h->status, st, &nlk,
                                          tokd ? x.in_index + r0[k] : nullptr, tokd ? n_ranks * capT : 0);
                nlaunch += nlk;
                CK(e, "experts");
                CK(cudaEventRecord(x.computed, st), "event record");
                if (ns == 1) {                                /* the shared expert's down rows, under the combine */
                    e = sp_batched_ep_shared(d, W, flavour, tm[k], &h->bs, h->status, st, &nlk, t0[k], k, 2);
                    nlaunch += nlk;
                    CK(e, "shared expert (down)");
                }
                CK(cudaStreamWaitEvent(cs, x.computed, 0), "event wait");
                if (p2p) {
                    CK(own_fork(x.back + (r0[k] + (size_t)rank * cap) * E, x.out + (r0[k] + (size_t)rank * cap) * E, (size_t)cap * E * 4), "own block");
                    for (int i = 1; i < n_ranks; i++) {
                        const int r = (rank + i) % n_ranks;
                        float *dstb = reinterpret_cast<float *>(s->peer_base[r] + s->o_back);
                        CK(cudaMemcpyAsync(dstb + (r0[k] + (size_t)rank * cap) * E, x.out + (r0[k] + (size_t)r * cap) * E, (size_t)cap * E * 4, cudaMemcpyDeviceToDevice, cs), "combine copy");
                    }
                    CK(own_join(), "own block");
                    if (n_ranks > 1) NK(N->AllReduce(s->sync_dev, s->sync_dev + 1, 1, ncclInt32, ncclSum, comm, cs), "landing all-reduce");
                } else {
                    NK(N->GroupStart(), "group start");
                    for (int r = 0; r < n_ranks; r++) {
                        NK(N->Send(x.out + (r0[k] + (size_t)r * cap) * E, (size_t)cap * E, ncclFloat32, r, comm, cs), "combine send");
                        NK(N->Recv(x.back + (r0[k] + (size_t)r * cap) * E, (size_t)cap * E, ncclFloat32, r, comm, cs), "combine recv");
                    }
                    NK(N->GroupEnd(), "group end");
                }
                CK(cudaEventRecord(x.combined, cs), "event record");
            }
            /* ---- finish every slice as its rows come back */
            for (int k = 0; k < ns; k++) {
                Slice &x = s->sl[k];
                CK(cudaStreamWaitEvent(st, x.combined, 0), "event wait");
                cudaError_t e = sp_batched_ep_finish(d, W, tm[k], cur + (size_t)t0[k] * E, x.back + r0[k] * E, x.pair_index + (size_t)t0[k] * NU, dst + (size_t)t0[k] * E,
                                                     &h->bs, st, &nlk, t0[k], k);
                nlaunch += nlk;
                CK(e, "finish");
            }
            s->last_rows = (long long)n_ranks * cap * ns;
        } else {
            /* ---- exact exchange: one slice, the split sizes read on the host */
            Slice &x = s->sl[0];
            cudaError_t e = sp_batched_ep_route(d, W, flavour, M, cur, x.sel_asc, x.cw, x.send, x.counts, x.pair_index, nullptr, nullptr, 1, 0, 0, &h->bs, h->status, st, &nlk, 0, 0);
            nlaunch += nlk;
            CK(e, "route");
            CK(cudaEventRecord(x.routed, st), "event record");
            CK(cudaStreamWaitEvent(cs, x.routed, 0), "event wait");
            NK(N->AllGather(x.counts, x.counts_all, (size_t)NE, ncclInt32, comm, cs), "all-gather of the counts");
            CK(cudaMemcpyAsync(s->counts_host, x.counts_all, 4 * (size_t)NE * n_ranks, cudaMemcpyDeviceToHost, cs), "counts D2H");
            CK(cudaStreamSynchronize(cs), "stream synchronize");               /* the one host read of the layer */
            long long send_n[64 * 16], recv_n[64 * 16];
            if (n_ranks > 1024) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: more than 1024 ranks");
            long long R = 0, soff = 0;
            for (int r = 0; r < n_ranks; r++) {
                long long a = 0, b2 = 0;
                for (int q = 0; q < epr; q++) { a += s->counts_host[(size_t)rank * NE + r * epr + q]; b2 += s->counts_host[(size_t)r * NE + rank * epr + q]; }
                send_n[r] = a; recv_n[r] = b2; R += b2;
            }
            if (R > s->rows_cap) return fail(SP_MOE_EBADARG, "sp_moe_ep_forward_dev: this rank would receive %lld rows, max_expert_rows is %d", R, s->rows_cap);
            /* rows rank a sends to rank b, from the gathered counts every rank holds */
            auto rows_ab = [&](int a, int b2) { long long v = 0; for (int q = 0; q < epr; q++) v += s->counts_host[(size_t)a * NE + (size_t)b2 * epr + q]; return v; };
            if (p2p) {                                        /* my block for rank r lands behind the blocks of the ranks before me */
                for (int i = 0; i < n_ranks; i++) {               /* own block first, then rank + 1, rank + 2, ...: one copy per destination at a time */
                    const int r = (rank + i) % n_ranks;
                    long long at = 0, from = 0;
                    for (int a = 0; a < rank; a++) at += rows_ab(a, r);
                    for (int b2 = 0; b2 < r; b2++) from += send_n[b2];
                    float *dstb = reinterpret_cast<float *>((r == rank ? s->base : s->peer_base[r]) + s->o_recv);
                    if (send_n[r]) CK(cudaMemcpyAsync(dstb + (size_t)at * E, x.send + (size_t)from * E, (size_t)send_n[r] * E * 4, cudaMemcpyDeviceToDevice, cs), "dispatch copy");
                }
                if (n_ranks > 1) NK(N->AllReduce(s->sync_dev, s->sync_dev + 1, 1, ncclInt32, ncclSum, comm, cs), "landing all-reduce");
            } else {
                NK(N->GroupStart(), "group start");
                { long long ro = 0; soff = 0;
                  for (int r = 0; r < n_ranks; r++) {
                      if (send_n[r]) NK(N->Send(x.send + (size_t)soff * E, (size_t)send_n[r] * E, ncclFloat32, r, comm, cs), "dispatch send");
                      if (recv_n[r]) NK(N->Recv(x.recv + (size_t)ro * E, (size_t)recv_n[r] * E, ncclFloat32, r, comm, cs), "dispatch recv");
                      soff += send_n[r]; ro += recv_n[r];
                  } }
                NK(N->GroupEnd(), "group end");
            }
            CK(cudaEventRecord(x.dispatched, cs), "event record");
            e = sp_batched_ep_shared(d, W, flavour, M, &h->bs, h->status, st, &nlk, 0, 0, 1);      /* gate/up under the dispatch, down under the combine */
            nlaunch += nlk;
            CK(e, "shared expert");
            /* the rows arrive source-major, each source's block sorted by expert: the layout kernel with a capacity
             * equal to each source's real block would need per-source capacities, so build it here on the host */
            {
                static thread_local std::vector<int32_t> off, idx;
                off.assign((size_t)NE + 1, 0); idx.resize((size_t)R);
                std::vector<long long> arrival((size_t)n_ranks + 1, 0);
                for (int r = 0; r < n_ranks; r++) arrival[r + 1] = arrival[r] + recv_n[r];
                long long p = 0;
                std::vector<long long> within((size_t)n_ranks, 0);
                for (int q = 0; q < epr; q++) {
                    off[(size_t)rank * epr + q] = (int32_t)p;
                    for (int r = 0; r < n_ranks; r++) {
                        const int cnt = s->counts_host[(size_t)r * NE + rank * epr + q];
                        for (int i = 0; i < cnt; i++) idx[(size_t)p++] = (int32_t)(arrival[r] + within[r] + i);
                        within[r] += cnt;
                    }
                }
                for (int eidx = rank * epr + epr; eidx <= NE; eidx++) off[(size_t)eidx] = (int32_t)R;
                CK(cudaMemcpyAsync(x.offsets, off.data(), 4 * ((size_t)NE + 1), cudaMemcpyHostToDevice, st), "offsets H2D");
                if (R) CK(cudaMemcpyAsync(x.row_index, idx.data(), 4 * (size_t)R, cudaMemcpyHostToDevice, st), "row index H2D");
                CK(cudaStreamSynchronize(st), "stream synchronize");             /* the staging vectors are reused by the next layer */
            }
            CK(cudaStreamWaitEvent(st, x.dispatched, 0), "event wait");
            if (R) {
                e = sp_batched_ep_experts(d, W, flavour, (int)R, x.recv, x.row_index, x.offsets, x.out, &h->bs, h->status, st, &nlk);
                nlaunch += nlk;
                CK(e, "experts");
            }
            CK(cudaEventRecord(x.computed, st), "event record");
            e = sp_batched_ep_shared(d, W, flavour, M, &h->bs, h->status, st, &nlk, 0, 0, 2);
            nlaunch += nlk;
            CK(e, "shared expert (down)");
            CK(cudaStreamWaitEvent(cs, x.computed, 0), "event wait");
            if (p2p) {                                        /* what came from rank r goes back to where r keeps the pairs it sent here */
                for (int i = 0; i < n_ranks; i++) {
                    const int r = (rank + i) % n_ranks;
                    long long at = 0, from = 0;
                    for (int b2 = 0; b2 < rank; b2++) at += rows_ab(r, b2);
                    for (int a = 0; a < r; a++) from += recv_n[a];
                    float *dstb = reinterpret_cast<float *>((r == rank ? s->base : s->peer_base[r]) + s->o_back);
                    if (recv_n[r]) CK(cudaMemcpyAsync(dstb + (size_t)at * E, x.out + (size_t)from * E, (size_t)recv_n[r] * E * 4, cudaMemcpyDeviceToDevice, cs), "combine copy");
                }
                if (n_ranks > 1) NK(N->AllReduce(s->sync_dev, s->sync_dev + 1, 1, ncclInt32, ncclSum, comm, cs), "landing all-reduce");
            } else {
                NK(N->GroupStart(), "group start");
                { long long ro = 0; soff = 0;
                  for (int r = 0; r < n_ranks; r++) {
                      if (recv_n[r]) NK(N->Send(x.out + (size_t)ro * E, (size_t)recv_n[r] * E, ncclFloat32, r, comm, cs), "combine send");
                      if (send_n[r]) NK(N->Recv(x.back + (size_t)soff * E, (size_t)send_n[r] * E, ncclFloat32, r, comm, cs), "combine recv");
                      soff += send_n[r]; ro += recv_n[r];
                  } }
                NK(N->GroupEnd(), "group end");
            }
            CK(cudaEventRecord(x.combined, cs), "event record");
            CK(cudaStreamWaitEvent(st, x.combined, 0), "event wait");
            e = sp_batched_ep_finish(d, W, M, cur, x.back, x.pair_index, dst, &h->bs, st, &nlk, 0, 0);
            nlaunch += nlk;
            CK(e, "finish");
            s->last_rows = R;
        }
        if (timing && li == nl - 1) CK(cudaEventRecord(s->end, st), "event record");
        cur = dst;
    }
    s->timing_valid = timing;
    h->launches += (uint64_t)nlaunch;
    return SP_MOE_OK;
}

/* Stage times of the LAST layer of the most recent sp_moe_ep_forward_dev call, from CUDA events (handle opened
 * with SP_MOE_TIMING=1, the call made outside a stream capture, one token slice): ms[0] route (norms, router,
 * top-NU, send buffer), ms[1] count gather + dispatch exchange on the communication stream, ms[2] from the end of
 * the dispatch to the end of the experts stage on the compute stream (the shared expert and the receive layout ran
 * under the dispatch), ms[3] combine exchange, ms[4] finish, ms[5] the whole layer. Synchronises both streams. */
extern "C" int sp_moe_ep_timing(sp_moe *h, float *ms6) {
    if (!h || !ms6) return fail(SP_MOE_EBADARG, "sp_moe_ep_timing: NULL argument");
    EpState *s = (EpState *)h->ep_state;
    if (!s || !s->timed || !s->timing_valid) return fail(SP_MOE_EBADSTATE, "sp_moe_ep_timing: needs SP_MOE_TIMING=1 at open and a one-slice sp_moe_ep_forward_dev call outside a stream capture");
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    CK(cudaEventSynchronize(s->end), "event synchronize");
    const Slice &x = s->sl[0];
    CK(cudaEventElapsedTime(ms6 + 0, s->begin, x.routed), "elapsed");
    CK(cudaEventElapsedTime(ms6 + 1, x.routed, x.dispatched), "elapsed");
    CK(cudaEventElapsedTime(ms6 + 2, x.dispatched, x.computed), "elapsed");
    CK(cudaEventElapsedTime(ms6 + 3, x.computed, x.combined), "elapsed");
    CK(cudaEventElapsedTime(ms6 + 4, x.combined, s->end), "elapsed");
    CK(cudaEventElapsedTime(ms6 + 5, s->begin, s->end), "elapsed");
    return SP_MOE_OK;
}
