/* api.cu — the extern "C" surface of libsp_moe_b200 (include/sp_engine/moe_backend.h).
 *
 * Holds what the reference keeps in process globals (g_w MoE fields CF:1856-1903, the expert
 * cache CF:6773-6951, g4_moe_scratch CF:5547) inside one handle: a single resident arena with
 * every layer's router, norm vectors, shared expert and all NE routed experts, plus scratch.
 * With all experts resident, moe_resident's hit branch (pointer arithmetic, CF:6923-6942) is
 * the only branch left. CF = src/backends/cuda/cuda_forward.cu of nihilistau/kairos-engine.
 */
#include "common.cuh"
#include "decode.cuh"
#include "batched.cuh"
#include "../../include/sp_engine/moe_backend.h"
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <new>
#include <cstdlib>
#include <vector>

/* ---------------------------------------------------------------- error text (sp_status.h:57-59) */
static thread_local char g_err[768];
extern "C" __attribute__((weak)) void sp_set_error(const char *msg) {
    std::snprintf(g_err, sizeof g_err, "%s", msg ? msg : "");
}
extern "C" __attribute__((weak)) const char *sp_last_error(void) { return g_err; }

static int fail(int code, const char *fmt, ...) {
    char b[640];
    va_list ap; va_start(ap, fmt); std::vsnprintf(b, sizeof b, fmt, ap); va_end(ap);
    sp_set_error(b);
    return code;
}
static int fail_cuda(cudaError_t e, const char *where) {       /* CF:189-195 */
    const int code = (e == cudaErrorMemoryAllocation) ? SP_MOE_EBACKEND_OOM : SP_MOE_ECUDA;
    return fail(code, "CUDA: %s: %s (%d)", where, cudaGetErrorString(e), (int)e);
}
#define CK(call, where) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return fail_cuda(e_, where); } while (0)

#include "handle.cuh"

static size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }

static void layout(const sp_moe_config &c, LayerOffsets &o) {
    size_t p = 0;
    auto take = [&](size_t bytes) { size_t at = p; p = up256(p + bytes); return at; };
    const size_t E = c.E, NE = c.NE, FFE = c.FFE, FFS = c.FFS;
    o.router_w = take(4 * NE * E); o.router_scale = take(4 * E); o.router_bias = take(4 * NE);
    o.ffn_norm = take(4 * E); o.post_ffw1 = take(4 * E); o.pre_ffw2 = take(4 * E);
    o.post_ffw2 = take(4 * E); o.post_ffw = take(4 * E); o.dexps_scale = take(4 * NE);
    o.sg_codes = take(FFS * E / 2); o.sg_bs = take(2 * FFS * (E / 32));
    o.su_codes = take(FFS * E / 2); o.su_bs = take(2 * FFS * (E / 32));
    o.sd_codes = take(E * FFS / 2); o.sd_bs = take(2 * E * (FFS / 32));
    o.gu_codes = take(NE * 2 * FFE * E / 2); o.gu_bs = take(2 * NE * 2 * FFE * (E / 32));
    o.dn_codes = take(NE * E * FFE / 2); o.dn_bs = take(2 * NE * E * (FFE / 32));
    o.end = p;
}

static SpLayerDev layer_view(const sp_moe *h, int L, bool bias) {
    unsigned char *b = h->arena + (size_t)L * h->layer_bytes;
    const LayerOffsets &o = h->off;
    SpLayerDev v;
    v.router_w = (const float *)(b + o.router_w); v.router_scale = (const float *)(b + o.router_scale);
    v.router_bias = bias ? (const float *)(b + o.router_bias) : nullptr;
    v.ffn_norm = (const float *)(b + o.ffn_norm); v.post_ffw1 = (const float *)(b + o.post_ffw1);
    v.pre_ffw2 = (const float *)(b + o.pre_ffw2); v.post_ffw2 = (const float *)(b + o.post_ffw2);
    v.post_ffw = (const float *)(b + o.post_ffw); v.dexps_scale = (const float *)(b + o.dexps_scale);
    v.gu_codes = b + o.gu_codes; v.gu_bs = (const uint16_t *)(b + o.gu_bs);
    v.dn_codes = b + o.dn_codes; v.dn_bs = (const uint16_t *)(b + o.dn_bs);
    v.sg_codes = b + o.sg_codes; v.sg_bs = (const uint16_t *)(b + o.sg_bs);
    v.su_codes = b + o.su_codes; v.su_bs = (const uint16_t *)(b + o.su_bs);
    v.sd_codes = b + o.sd_codes; v.sd_bs = (const uint16_t *)(b + o.sd_bs);
    return v;
}

extern "C" int sp_moe_open(const sp_moe_config *cfg, sp_moe **out) {
    if (!cfg || !out) return fail(SP_MOE_EBADARG, "sp_moe_open: NULL argument");
    *out = nullptr;
    const sp_moe_config &c = *cfg;
    if (c.E <= 0 || (c.E & 31) || c.E > 4096 || c.FFE <= 0 || (c.FFE & 31) || c.FFE > 4096 ||
        c.FFS <= 0 || (c.FFS & 31) || c.FFS > 4096)                                  /* CF:13828; moe_cpu_expert.c:243 */
        return fail(SP_MOE_EBADARG, "sp_moe_open: E, FFE, FFS must be multiples of 32 in (0, 4096] (got %d, %d, %d)", c.E, c.FFE, c.FFS);
    if (c.NE <= 0 || c.NE > 1024 || c.NU <= 0 || c.NU > SP_MAX_NU || c.NU > c.NE)
        return fail(SP_MOE_EBADARG, "sp_moe_open: need 0 < NU <= min(NE, %d), NE <= 1024 (got NE=%d NU=%d)", SP_MAX_NU, c.NE, c.NU);
    if (c.n_layers <= 0 || c.max_tokens <= 0) return fail(SP_MOE_EBADARG, "sp_moe_open: n_layers and max_tokens must be positive");
    if (c.max_expert_rows < 0) return fail(SP_MOE_EBADARG, "sp_moe_open: max_expert_rows must not be negative");
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev == 0) { cudaGetLastError(); return fail(SP_MOE_ECUDA, "sp_moe_open: no CUDA device (%s); this library has no CPU path", cudaGetErrorString(e)); }
    if (c.device < 0 || c.device >= ndev) return fail(SP_MOE_EBADARG, "sp_moe_open: device %d out of range (%d present)", c.device, ndev);
    CK(cudaSetDevice(c.device), "cudaSetDevice");
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, c.device), "cudaGetDeviceProperties");
    if (prop.major != 10) return fail(SP_MOE_EUNSUPPORTED, "sp_moe_open: built for sm_100a only; device is sm_%d%d", prop.major, prop.minor);

    sp_moe *h = new (std::nothrow) sp_moe();
    if (!h) return fail(SP_MOE_ENOMEM, "sp_moe_open: host OOM");
    h->cfg = c; h->device = c.device;
    h->d.E = c.E; h->d.NE = c.NE; h->d.NU = c.NU; h->d.FFE = c.FFE; h->d.FFS = c.FFS; h->d.eps = c.eps;
    h->d.inv_sqrt_e = 1.0f / sqrtf((float)c.E);
    layout(c, h->off);
    h->layer_bytes = h->off.end;
    h->arena_bytes = h->layer_bytes * (size_t)c.n_layers;
    h->layers_host.resize(c.n_layers); h->has_bias.assign(c.n_layers, 0); h->uploaded.assign(c.n_layers, 0);
#define OPEN_CK(call, where) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { int rc_ = fail_cuda(e_, where); sp_moe_close(h); return rc_; } } while (0)
    OPEN_CK(cudaMalloc(&h->arena, h->arena_bytes), "arena cudaMalloc");
    OPEN_CK(cudaMalloc(&h->layers_dev, sizeof(SpLayerDev) * c.n_layers), "layer table cudaMalloc");
    for (int L = 0; L < c.n_layers; L++) h->layers_host[L] = layer_view(h, L, false);
    OPEN_CK(cudaMemcpy(h->layers_dev, h->layers_host.data(), sizeof(SpLayerDev) * c.n_layers, cudaMemcpyHostToDevice), "layer table H2D");
    size_t sb = 0;
    auto dalloc = [&](void **p, size_t bytes) { sb += up256(bytes); return cudaMalloc(p, bytes); };
    OPEN_CK(dalloc((void **)&h->status, 256), "scratch");
    OPEN_CK(cudaMemset(h->status, 0, 256), "memset");
    OPEN_CK(cudaMallocHost((void **)&h->status_host, 64), "status word (host)");
    const size_t mt = (size_t)c.max_tokens;
    OPEN_CK(dalloc((void **)&h->x_dev, 4 * mt * c.E), "staging"); OPEN_CK(dalloc((void **)&h->y_dev, 4 * mt * c.E), "staging");
    OPEN_CK(dalloc((void **)&h->sel_dev, 4 * mt * c.NU * c.n_layers), "staging"); OPEN_CK(dalloc((void **)&h->wts_dev, 4 * mt * c.NU * c.n_layers), "staging");
    {   /* scratch of the graph decode path */
        const size_t E = c.E, NE = c.NE, NU = c.NU, FFE = c.FFE, FFS = c.FFS;
        size_t o = 0; auto take = [&](size_t bytes) { size_t at = o; o = up256(o + bytes); return at; };
        const size_t o_lg = take(4 * NE), o_hd = take(4 * FFS), o_dn = take(4 * E), o_h = take(4 * NU * FFE), o_acc = take(4 * E),
                     o_q = take(E), o_s = take(4 * (E / 16)), o_c = take(4 * (E / 16)), o_sel = take(4 * SP_MAX_NU), o_cw = take(4 * SP_MAX_NU),
                     o_x0 = take(4 * E), o_x1 = take(4 * E), o_gx = take(4 * E), o_gy = take(4 * E),
                     o_gsel = take(4 * NU * (size_t)c.n_layers), o_gw = take(4 * NU * (size_t)c.n_layers);
        cudaDeviceGetAttribute(&h->sms, cudaDevAttrMultiProcessorCount, c.device);
        const size_t o_sl = take(48 * (size_t)h->sms);
        OPEN_CK(dalloc((void **)&h->gs_base, o), "scratch");
        unsigned char *b = h->gs_base;
        {
            std::vector<int> sl(12 * (size_t)h->sms);
            sp_staged_slices(h->d, h->sms, sl.data());
            OPEN_CK(cudaMemcpy(b + o_sl, sl.data(), sl.size() * sizeof(int), cudaMemcpyHostToDevice), "slice table H2D");
            h->gs.slices = (const int *)(b + o_sl);
        }
        h->gs.logits = (float *)(b + o_lg); h->gs.hd = (float *)(b + o_hd); h->gs.dn = (float *)(b + o_dn); h->gs.h = (float *)(b + o_h); h->gs.acc = (float *)(b + o_acc);
        h->gs.in_q = (signed char *)(b + o_q); h->gs.in_s = (float *)(b + o_s); h->gs.in_c = (int *)(b + o_c);
        h->gs.sel_asc = (int *)(b + o_sel); h->gs.cw = (float *)(b + o_cw); h->gs.status = h->status;
        h->gs.xbuf[0] = (float *)(b + o_x0); h->gs.xbuf[1] = (float *)(b + o_x1);
        h->gs.prev_post_ffw1 = h->gs.prev_post_ffw2 = h->gs.prev_post_ffw = nullptr;
        h->g_x = (float *)(b + o_gx); h->g_y = (float *)(b + o_gy); h->g_sel = (int32_t *)(b + o_gsel); h->g_wts = (float *)(b + o_gw);
        cudaDeviceGetAttribute(&h->sms, cudaDevAttrMultiProcessorCount, c.device);
        int optin = 0;
        cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, c.device);
        /* house convention: behaviour switches are SP_* variables read once. SP_MOE_DECODE_IMPL=direct keeps the
         * weight rows out of shared memory (the path every geometry can take); the default stages them when they fit. */
        const char *ev = getenv("SP_MOE_DECODE_IMPL");
        h->decode_impl = ((ev && ev[0] == 'd') || !sp_staged_fits(h->d, h->sms, (size_t)optin)) ? 1 : 0;
        const char *fv = getenv("SP_MOE_STAGED_FLAGS");
        h->staged_flags = fv ? (unsigned)strtoul(fv, nullptr, 0) : (unsigned)SP_STAGED_DEFAULT;
        const char *sq = getenv("SP_MOE_SEQ_TOKENS");              /* tuning switch: 1 sends every batch of 2+ tokens to the batched kernels */
        h->seq_tokens = sq ? atoi(sq) : 5;
        if (h->seq_tokens < 1) h->seq_tokens = 1;
        /* the kernels' shared-memory limits are a per-device setting: set them for this handle's device */
        OPEN_CK(sp_graph_prepare(), "decode kernel attributes");
        if (h->decode_impl == 0) OPEN_CK(sp_staged_prepare(h->d, h->sms), "decode kernel attributes");
        const char *tv = getenv("SP_MOE_TIMING");                 /* the reference's switch for its [g4-moe] TIMING line (CF:7186-7201) */
        if (tv && tv[0] == '1') {
            OPEN_CK(dalloc((void **)&h->stamps, 48 * sizeof(long long)), "timing stamps");
            OPEN_CK(cudaMemset(h->stamps, 0, 48 * sizeof(long long)), "memset");
            OPEN_CK(cudaMallocHost((void **)&h->stamps_host, 48 * sizeof(long long)), "timing stamps (host)");
        }
    }
    { size_t bb = 0; cudaError_t be = sp_batched_alloc(h->d, c.max_tokens, c.max_expert_rows, &h->bs, &bb); sb += bb; OPEN_CK(be, "batched scratch"); }
    OPEN_CK(cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking), "cudaStreamCreate");
    h->last_stream = h->stream;
    h->scratch_bytes = sb;
#undef OPEN_CK
    *out = h;
    return SP_MOE_OK;
}

extern "C" int sp_moe_close(sp_moe *h) {
    if (!h) return SP_MOE_OK;
    cudaSetDevice(h->device);
    if (h->stream) { cudaStreamSynchronize(h->stream); cudaStreamDestroy(h->stream); }
    if (h->ep_state && h->ep_state_free) { h->ep_state_free(h->ep_state); h->ep_state = nullptr; }
    sp_batched_free(&h->bs);
    for (auto &g : h->graphs) if (g.exec) cudaGraphExecDestroy(g.exec);
    for (auto &g : h->bgraphs) if (g.exec) cudaGraphExecDestroy(g.exec);
    void *ps[] = {h->gs_base, h->arena, h->layers_dev, h->status, h->x_dev, h->y_dev, h->sel_dev, h->wts_dev, h->stamps};
    for (void *p : ps) if (p) cudaFree(p);
    if (h->status_host) cudaFreeHost(h->status_host);
    if (h->stamps_host) cudaFreeHost(h->stamps_host);
    cudaGetLastError();
    delete h;
    return SP_MOE_OK;
}

const sp_moe_config *sp_moe_config_of(const sp_moe *h) { return &h->cfg; }      /* for the other translation units of the library */
extern "C" size_t sp_moe_device_bytes(const sp_moe *h) { return h ? h->arena_bytes + h->scratch_bytes : 0; }
extern "C" uint64_t sp_moe_kernel_launches(const sp_moe *h) { return h ? h->launches : 0; }

static void drop_graphs_of_layer(sp_moe *h, int L);
static int upload(sp_moe *h, int L, const sp_moe_layer_weights *w, cudaMemcpyKind kind, const char *who) {
    if (!h || !w) return fail(SP_MOE_EBADARG, "%s: NULL argument", who);
    if (L < 0 || L >= h->cfg.n_layers) return fail(SP_MOE_EBADARG, "%s: layer %d out of range [0, %d)", who, L, h->cfg.n_layers);
    const void *req[] = {w->router_w, w->router_scale, w->ffn_norm, w->post_ffw1, w->pre_ffw2, w->post_ffw2, w->post_ffw, w->dexps_scale,
                         w->gu_codes, w->gu_bs, w->dn_codes, w->dn_bs, w->sg_codes, w->sg_bs, w->su_codes, w->su_bs, w->sd_codes, w->sd_bs};
    for (const void *p : req) if (!p) return fail(SP_MOE_EBADARG, "%s: a MoE weight/norm/scale pointer is NULL at L=%d", who, L);   /* CF:8386-8393 */
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    unsigned char *b = h->arena + (size_t)L * h->layer_bytes;
    const LayerOffsets &o = h->off;
    const size_t E = h->cfg.E, NE = h->cfg.NE, FFE = h->cfg.FFE, FFS = h->cfg.FFS;
#define UP(off, src, bytes) CK(cudaMemcpy(b + (off), (src), (bytes), kind), who)
    UP(o.router_w, w->router_w, 4 * NE * E); UP(o.router_scale, w->router_scale, 4 * E);
    if (w->router_bias) UP(o.router_bias, w->router_bias, 4 * NE);
    UP(o.ffn_norm, w->ffn_norm, 4 * E); UP(o.post_ffw1, w->post_ffw1, 4 * E); UP(o.pre_ffw2, w->pre_ffw2, 4 * E);
    UP(o.post_ffw2, w->post_ffw2, 4 * E); UP(o.post_ffw, w->post_ffw, 4 * E); UP(o.dexps_scale, w->dexps_scale, 4 * NE);
    UP(o.sg_codes, w->sg_codes, FFS * E / 2); UP(o.sg_bs, w->sg_bs, 2 * FFS * (E / 32));
    UP(o.su_codes, w->su_codes, FFS * E / 2); UP(o.su_bs, w->su_bs, 2 * FFS * (E / 32));
    UP(o.sd_codes, w->sd_codes, E * FFS / 2); UP(o.sd_bs, w->sd_bs, 2 * E * (FFS / 32));
    UP(o.gu_codes, w->gu_codes, NE * 2 * FFE * E / 2); UP(o.gu_bs, w->gu_bs, 2 * NE * 2 * FFE * (E / 32));
    UP(o.dn_codes, w->dn_codes, NE * E * FFE / 2); UP(o.dn_bs, w->dn_bs, 2 * NE * E * (FFE / 32));
#undef UP
    h->has_bias[L] = w->router_bias != nullptr;
    h->layers_host[L] = layer_view(h, L, h->has_bias[L]);
    drop_graphs_of_layer(h, L);
    CK(cudaMemcpy(h->layers_dev + L, &h->layers_host[L], sizeof(SpLayerDev), cudaMemcpyHostToDevice), who);
    h->uploaded[L] = 1;
    return SP_MOE_OK;
}
static void drop_graphs_of_layer(sp_moe *h, int L) {
    /* captured graphs hold this layer's view by value (the bias pointer may just have appeared or gone) */
    for (size_t i = h->graphs.size(); i-- > 0;)
        if (L >= h->graphs[i].lf && L < h->graphs[i].lf + h->graphs[i].nl) { cudaGraphExecDestroy(h->graphs[i].exec); h->graphs.erase(h->graphs.begin() + (long)i); }
    for (size_t i = h->bgraphs.size(); i-- > 0;)
        if (L >= h->bgraphs[i].lf && L < h->bgraphs[i].lf + h->bgraphs[i].nl) { cudaGraphExecDestroy(h->bgraphs[i].exec); h->bgraphs.erase(h->bgraphs.begin() + (long)i); }
}
extern "C" int sp_moe_set_router_bias_dev(sp_moe *h, int L, const float *bias_dev) {
    if (!h) return fail(SP_MOE_EBADARG, "sp_moe_set_router_bias_dev: NULL handle");
    if (L < 0 || L >= h->cfg.n_layers) return fail(SP_MOE_EBADARG, "sp_moe_set_router_bias_dev: layer %d out of range [0, %d)", L, h->cfg.n_layers);
    if (!h->uploaded[L]) return fail(SP_MOE_EBADSTATE, "sp_moe_set_router_bias_dev: layer %d has no weights uploaded", L);
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    CK(cudaStreamSynchronize(h->last_stream), "stream synchronize");
    if (bias_dev) CK(cudaMemcpy(h->arena + (size_t)L * h->layer_bytes + h->off.router_bias, bias_dev, 4 * (size_t)h->cfg.NE, cudaMemcpyDeviceToDevice), "router bias copy");
    h->has_bias[L] = bias_dev != nullptr;
    h->layers_host[L] = layer_view(h, L, h->has_bias[L]);
    CK(cudaMemcpy(h->layers_dev + L, &h->layers_host[L], sizeof(SpLayerDev), cudaMemcpyHostToDevice), "layer table H2D");
    drop_graphs_of_layer(h, L);
    return SP_MOE_OK;
}
extern "C" int sp_moe_upload_layer(sp_moe *h, int L, const sp_moe_layer_weights *w) { return upload(h, L, w, cudaMemcpyHostToDevice, "sp_moe_upload_layer"); }
extern "C" int sp_moe_upload_layer_dev(sp_moe *h, int L, const sp_moe_layer_weights *w) { return upload(h, L, w, cudaMemcpyDeviceToDevice, "sp_moe_upload_layer_dev"); }

/* ---------------------------------------------------------------- forward */
static int check_forward(sp_moe *h, int lf, int nl, int flavour, int M, const void *x, const void *y, const char *who) {
    if (!h || !x || !y) return fail(SP_MOE_EBADARG, "%s: NULL argument", who);
    if (lf < 0 || nl <= 0 || lf + nl > h->cfg.n_layers) return fail(SP_MOE_EBADARG, "%s: layers [%d, %d) outside [0, %d)", who, lf, lf + nl, h->cfg.n_layers);
    if (M <= 0 || M > h->cfg.max_tokens) return fail(SP_MOE_EBADARG, "%s: M=%d outside (0, max_tokens=%d]", who, M, h->cfg.max_tokens);
    if (flavour != SP_MOE_FLAVOUR_DECODE && flavour != SP_MOE_FLAVOUR_PREFILL) return fail(SP_MOE_EBADARG, "%s: unknown flavour %d", who, flavour);
    for (int L = lf; L < lf + nl; L++) if (!h->uploaded[L]) return fail(SP_MOE_EBADSTATE, "%s: layer %d has no weights uploaded", who, L);
    return SP_MOE_OK;
}

extern "C" int sp_moe_forward_dev(sp_moe *h, int lf, int nl, int flavour, int M,
                                  const float *x_dev, float *y_dev, int32_t *sel_dev, float *wts_dev, void *stream) {
    int rc = check_forward(h, lf, nl, flavour, M, x_dev, y_dev, "sp_moe_forward_dev");
    if (rc) return rc;
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream;
    h->last_stream = st;
    if (M <= h->seq_tokens && flavour == SP_MOE_FLAVOUR_DECODE) {
        /* A handful of tokens goes through the single-token graph one token after the other: below
         * seq_tokens that is faster than the batched kernels, and each row is the single-token result
         * by construction. */
        const bool routing = sel_dev || wts_dev;
        sp_moe::DecodeGraph *dg = nullptr;
        for (auto &g : h->graphs) if (g.lf == lf && g.nl == nl && g.routing == routing) dg = &g;
        if (!dg) {                                                   /* first use: capture the layer run once */
            cudaStream_t cs = h->stream;
            cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr; int nlaunch = 0;
            CK(cudaStreamSynchronize(cs), "stream synchronize");
            CK(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal), "begin capture");
            cudaError_t e = h->decode_impl == 0
                ? sp_staged_decode_enqueue(h->d, h->layers_host.data(), lf, nl, h->g_x, h->g_y, routing ? h->g_sel : nullptr,
                                           routing ? h->g_wts : nullptr, h->gs, h->sms, h->staged_flags, h->stamps, cs, true, &nlaunch)
                : sp_graph_decode_enqueue(h->d, h->layers_host.data(), lf, nl, h->g_x, h->g_y, routing ? h->g_sel : nullptr,
                                          routing ? h->g_wts : nullptr, h->gs, h->sms, cs, true, &nlaunch);
            cudaError_t e2 = cudaStreamEndCapture(cs, &graph);
            if (e != cudaSuccess || e2 != cudaSuccess) { if (graph) cudaGraphDestroy(graph); cudaGetLastError(); return fail_cuda(e != cudaSuccess ? e : e2, "decode graph capture"); }
            e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) return fail_cuda(e, "decode graph instantiate");
            h->graphs.push_back({lf, nl, routing, exec, nlaunch});
            dg = &h->graphs.back();
        }
        const size_t E = (size_t)h->cfg.E, NU = (size_t)h->cfg.NU, nb = E * 4;
        for (int t = 0; t < M; t++) {
            CK(cudaMemcpyAsync(h->g_x, x_dev + t * E, nb, cudaMemcpyDeviceToDevice, st), "x staging");
            CK(cudaGraphLaunch(dg->exec, st), "decode graph launch");
            CK(cudaMemcpyAsync(y_dev + t * E, h->g_y, nb, cudaMemcpyDeviceToDevice, st), "y staging");
            /* routing tables are [layer][token][NU]: one NU-wide strip per layer for this token */
            if (sel_dev) CK(cudaMemcpy2DAsync(sel_dev + t * NU, (size_t)M * NU * 4, h->g_sel, NU * 4, NU * 4, (size_t)nl, cudaMemcpyDeviceToDevice, st), "sel staging");
            if (wts_dev) CK(cudaMemcpy2DAsync(wts_dev + t * NU, (size_t)M * NU * 4, h->g_wts, NU * 4, NU * 4, (size_t)nl, cudaMemcpyDeviceToDevice, st), "wts staging");
            h->launches += (uint64_t)dg->launches;
        }
        return SP_MOE_OK;
    }
    if (M <= 64) {
        const bool routing = sel_dev || wts_dev;
        sp_moe::BatchGraph *bg = nullptr;
        for (auto &g : h->bgraphs) if (g.lf == lf && g.nl == nl && g.M == M && g.flavour == flavour && g.routing == routing) bg = &g;
        if (!bg) {
            if (h->bgraphs.size() >= 32) { cudaGraphExecDestroy(h->bgraphs.front().exec); h->bgraphs.erase(h->bgraphs.begin()); }
            cudaStream_t cs = h->stream;
            cudaGraph_t graph = nullptr; cudaGraphExec_t exec = nullptr; int nlaunch = 0;
            CK(cudaStreamSynchronize(cs), "stream synchronize");
            CK(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal), "begin capture");
            cudaError_t e = sp_batched_forward(h->d, h->layers_host.data(), lf, nl, flavour, M, h->x_dev, h->y_dev, routing ? h->sel_dev : nullptr,
                                               routing ? h->wts_dev : nullptr, &h->bs, h->status, cs, &nlaunch);
            cudaError_t e2 = cudaStreamEndCapture(cs, &graph);
            if (e != cudaSuccess || e2 != cudaSuccess) { if (graph) cudaGraphDestroy(graph); cudaGetLastError(); return fail_cuda(e != cudaSuccess ? e : e2, "batched graph capture"); }
            e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) return fail_cuda(e, "batched graph instantiate");
            h->bgraphs.push_back({lf, nl, M, flavour, routing, exec, nlaunch});
            bg = &h->bgraphs.back();
        }
        const size_t nb = (size_t)M * h->cfg.E * 4, ns = (size_t)nl * M * h->cfg.NU * 4;
        if (x_dev != h->x_dev) CK(cudaMemcpyAsync(h->x_dev, x_dev, nb, cudaMemcpyDeviceToDevice, st), "x staging");
        CK(cudaGraphLaunch(bg->exec, st), "batched graph launch");
        if (y_dev != h->y_dev) CK(cudaMemcpyAsync(y_dev, h->y_dev, nb, cudaMemcpyDeviceToDevice, st), "y staging");
        if (sel_dev && sel_dev != h->sel_dev) CK(cudaMemcpyAsync(sel_dev, h->sel_dev, ns, cudaMemcpyDeviceToDevice, st), "sel staging");
        if (wts_dev && wts_dev != h->wts_dev) CK(cudaMemcpyAsync(wts_dev, h->wts_dev, ns, cudaMemcpyDeviceToDevice, st), "wts staging");
        h->launches += (uint64_t)bg->launches;
        return SP_MOE_OK;
    }
    int nlaunch = 0;
    cudaError_t e = sp_batched_forward(h->d, h->layers_host.data(), lf, nl, flavour, M, x_dev, y_dev, sel_dev, wts_dev, &h->bs, h->status, st, &nlaunch);
    h->launches += (uint64_t)nlaunch;
    if (e != cudaSuccess) return fail_cuda(e, "batched forward launch");
    return SP_MOE_OK;
}

/* ---------------------------------------------------------------- expert-parallel stages (one layer) */
static int check_ep(sp_moe *h, int L, int flavour, const char *who) {
    if (!h) return fail(SP_MOE_EBADARG, "%s: NULL handle", who);
    if (L < 0 || L >= h->cfg.n_layers) return fail(SP_MOE_EBADARG, "%s: layer %d out of range [0, %d)", who, L, h->cfg.n_layers);
    if (flavour != SP_MOE_FLAVOUR_DECODE && flavour != SP_MOE_FLAVOUR_PREFILL) return fail(SP_MOE_EBADARG, "%s: unknown flavour %d", who, flavour);
    if (!h->uploaded[L]) return fail(SP_MOE_EBADSTATE, "%s: layer %d has no weights uploaded", who, L);
    return SP_MOE_OK;
}
extern "C" int sp_moe_ep_route_dev(sp_moe *h, int layer, int flavour, int M, const float *x_dev, int32_t *sel_asc_dev, float *cw_dev,
                                   float *rows_dev, int32_t *counts_dev, int32_t *pair_index_dev, int32_t *sel_dev, float *wts_dev, int defer_shared,
                                   int n_ranks, int capacity, void *stream) {
    int rc = check_ep(h, layer, flavour, "sp_moe_ep_route_dev");
    if (rc) return rc;
    if (!x_dev || !sel_asc_dev || !cw_dev || !rows_dev || !counts_dev || !pair_index_dev) return fail(SP_MOE_EBADARG, "sp_moe_ep_route_dev: NULL argument");
    if (M <= 0 || M > h->cfg.max_tokens) return fail(SP_MOE_EBADARG, "sp_moe_ep_route_dev: M=%d outside (0, max_tokens=%d]", M, h->cfg.max_tokens);
    if (capacity < 0 || (capacity > 0 && (n_ranks <= 0 || h->cfg.NE % n_ranks)))
        return fail(SP_MOE_EBADARG, "sp_moe_ep_route_dev: a capacity needs n_ranks > 0 dividing NE=%d (got n_ranks=%d capacity=%d)", h->cfg.NE, n_ranks, capacity);
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream; h->last_stream = st;
    int nlaunch = 0;
    cudaError_t e = sp_batched_ep_route(h->d, h->layers_host[layer], flavour, M, x_dev, sel_asc_dev, cw_dev, rows_dev, counts_dev, pair_index_dev, sel_dev, wts_dev,
                                        defer_shared, n_ranks, capacity, &h->bs, h->status, st, &nlaunch);
    h->launches += (uint64_t)nlaunch;
    return e == cudaSuccess ? SP_MOE_OK : fail_cuda(e, "expert-parallel route launch");
}
extern "C" int sp_moe_ep_recv_layout_dev(sp_moe *h, const int32_t *counts_all_dev, int n_ranks, int rank, int capacity,
                                         int32_t *offsets_dev, int32_t *row_index_dev, void *stream) {
    if (!h || !counts_all_dev || !offsets_dev || !row_index_dev) return fail(SP_MOE_EBADARG, "sp_moe_ep_recv_layout_dev: NULL argument");
    if (n_ranks <= 0 || h->cfg.NE % n_ranks || rank < 0 || rank >= n_ranks || capacity <= 0)
        return fail(SP_MOE_EBADARG, "sp_moe_ep_recv_layout_dev: need 0 <= rank < n_ranks, n_ranks dividing NE=%d, capacity > 0", h->cfg.NE);
    if ((long long)n_ranks * capacity > h->bs.max_rows)
        return fail(SP_MOE_EBADARG, "sp_moe_ep_recv_layout_dev: n_ranks * capacity = %lld exceeds max_expert_rows=%d", (long long)n_ranks * capacity, h->bs.max_rows);
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream; h->last_stream = st;
    int nlaunch = 0;
    cudaError_t e = sp_batched_ep_recv_layout(h->d, counts_all_dev, n_ranks, rank, capacity, offsets_dev, row_index_dev, st, &nlaunch);
    h->launches += (uint64_t)nlaunch;
    return e == cudaSuccess ? SP_MOE_OK : fail_cuda(e, "expert-parallel receive layout launch");
}
extern "C" int sp_moe_ep_shared_dev(sp_moe *h, int layer, int flavour, int M, void *stream) {
    int rc = check_ep(h, layer, flavour, "sp_moe_ep_shared_dev");
    if (rc) return rc;
    if (M <= 0 || M > h->cfg.max_tokens) return fail(SP_MOE_EBADARG, "sp_moe_ep_shared_dev: M=%d outside (0, max_tokens=%d]", M, h->cfg.max_tokens);
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream; h->last_stream = st;
    int nlaunch = 0;
    cudaError_t e = sp_batched_ep_shared(h->d, h->layers_host[layer], flavour, M, &h->bs, h->status, st, &nlaunch);
    h->launches += (uint64_t)nlaunch;
    return e == cudaSuccess ? SP_MOE_OK : fail_cuda(e, "expert-parallel shared-expert launch");
}
extern "C" int sp_moe_ep_experts_dev(sp_moe *h, int layer, int flavour, int n_rows, const float *rows_in_dev, const int32_t *row_index_dev,
                                     const int32_t *offsets_dev, float *rows_out_dev, void *stream) {
    int rc = check_ep(h, layer, flavour, "sp_moe_ep_experts_dev");
    if (rc) return rc;
    if (n_rows < 0 || n_rows > h->bs.max_rows)
        return fail(SP_MOE_EBADARG, "sp_moe_ep_experts_dev: n_rows=%d outside [0, max_expert_rows=%d] (set sp_moe_config.max_expert_rows for the "
                                    "worst case an expert-parallel rank can receive)", n_rows, h->bs.max_rows);
    if (n_rows == 0) return SP_MOE_OK;
    if (!rows_in_dev || !offsets_dev || !rows_out_dev) return fail(SP_MOE_EBADARG, "sp_moe_ep_experts_dev: NULL argument");
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream; h->last_stream = st;
    int nlaunch = 0;
    cudaError_t e = sp_batched_ep_experts(h->d, h->layers_host[layer], flavour, n_rows, rows_in_dev, row_index_dev, offsets_dev, rows_out_dev, &h->bs, h->status, st, &nlaunch);
    h->launches += (uint64_t)nlaunch;
    return e == cudaSuccess ? SP_MOE_OK : fail_cuda(e, "expert-parallel expert launch");
}
extern "C" int sp_moe_ep_finish_dev(sp_moe *h, int layer, int M, const float *x_dev, const float *pair_rows_dev, const int32_t *pair_index_dev,
                                    float *y_dev, void *stream) {
    int rc = check_ep(h, layer, SP_MOE_FLAVOUR_DECODE, "sp_moe_ep_finish_dev");
    if (rc) return rc;
    if (!x_dev || !pair_rows_dev || !y_dev) return fail(SP_MOE_EBADARG, "sp_moe_ep_finish_dev: NULL argument");
    if (M <= 0 || M > h->cfg.max_tokens) return fail(SP_MOE_EBADARG, "sp_moe_ep_finish_dev: M=%d outside (0, max_tokens=%d]", M, h->cfg.max_tokens);
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream; h->last_stream = st;
    int nlaunch = 0;
    cudaError_t e = sp_batched_ep_finish(h->d, h->layers_host[layer], M, x_dev, pair_rows_dev, pair_index_dev, y_dev, &h->bs, st, &nlaunch);
    h->launches += (uint64_t)nlaunch;
    return e == cudaSuccess ? SP_MOE_OK : fail_cuda(e, "expert-parallel finish launch");
}

extern "C" int sp_moe_status(sp_moe *h) {
    if (!h) return fail(SP_MOE_EBADARG, "sp_moe_status: NULL handle");
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    CK(cudaMemcpyAsync(h->status_host, h->status, sizeof(int), cudaMemcpyDeviceToHost, h->last_stream), "status D2H");
    CK(cudaStreamSynchronize(h->last_stream), "stream synchronize");
    const int st = *h->status_host;
    if (st == SP_KERR_NONE) return SP_MOE_OK;
    cudaMemset(h->status, 0, sizeof(int));
    if (st == SP_KERR_BARRIER_TIMEOUT) {
        return fail(SP_MOE_ECUDA, "gemma4-MoE: a bounded device-side wait ran out; the step's output is invalid");
    }
    if (st == SP_KERR_NAN_ROUTER)                     /* CF:8596-8620 */
        return fail(SP_MOE_EBADSTATE, "gemma4-MoE: router produced no usable expert: a logit row holds NaN, "
                                       "which means the router input upstream is bad, not the top-k");
    return fail(SP_MOE_ECUDA, "gemma4-MoE: kernel error word %d", st);
}

/* ---------------------------------------------------------------- phase timing (SP_MOE_TIMING=1) */
static int read_timing(sp_moe *h, sp_moe_timing *t) {
    CK(cudaMemcpyAsync(h->stamps_host, h->stamps, 48 * sizeof(long long), cudaMemcpyDeviceToHost, h->last_stream), "timing D2H");
    CK(cudaStreamSynchronize(h->last_stream), "stream synchronize");
    const long long *s = h->stamps_host;
    for (int k = 0; k < 3; k++) {
        t->wait_us[k] = (float)((s[k * 16 + 1] - s[k * 16 + 0]) * 1e-3);
        t->prologue_us[k] = (float)((s[k * 16 + 3] - s[k * 16 + 1]) * 1e-3);
        t->rows_us[k] = (float)((s[k * 16 + 4] - s[k * 16 + 3]) * 1e-3);
    }
    t->layer_us = (float)((s[2 * 16 + 4] - s[0]) * 1e-3);
    for (int k = 0; k < 3; k++) for (int i = 0; i < 16; i++) t->raw_us[k][i] = s[k * 16 + i] ? (float)((s[k * 16 + i] - s[0]) * 1e-3) : 0.0f;
    return SP_MOE_OK;
}
extern "C" int sp_moe_decode_timing(sp_moe *h, sp_moe_timing *out) {
    if (!h || !out) return fail(SP_MOE_EBADARG, "sp_moe_decode_timing: NULL argument");
    if (!h->stamps) return fail(SP_MOE_EBADSTATE, "sp_moe_decode_timing: open the handle with SP_MOE_TIMING=1 in the environment");
    if (h->decode_impl != 0) return fail(SP_MOE_EUNSUPPORTED, "sp_moe_decode_timing: only the shared-memory-staged decode path records phases");
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    return read_timing(h, out);
}
/* the reference prints its line every 300 router syncs = 10 tokens x 30 layers (CF:9022); same cadence in decoded layers */
static void timing_accumulate(sp_moe *h, int nl) {
    sp_moe_timing t;
    if (!h->stamps || h->decode_impl != 0 || read_timing(h, &t) != SP_MOE_OK) return;
    for (int k = 0; k < 3; k++) { h->timing_us[k][0] += t.wait_us[k]; h->timing_us[k][1] += t.prologue_us[k]; h->timing_us[k][2] += t.rows_us[k]; h->timing_us[k][3] += 1.0; }
    h->timing_layer_us += t.layer_us;
    const uint64_t before = h->timing_runs; h->timing_runs += (uint64_t)nl;
    if (before / 300 != h->timing_runs / 300) {
        const double n = h->timing_us[0][3] > 0 ? h->timing_us[0][3] : 1.0;
        std::fprintf(stderr, "    [g4-moe] TIMING after %llu decoded layers (last layer of each call sampled, device clock): layer %.1f us | "
                             "router+shared: wait %.1f prologue %.1f rows %.1f | top-k+gate|up: wait %.1f prologue %.1f rows %.1f | "
                             "down+combine: wait %.1f prologue %.1f rows %.1f\n",
                     (unsigned long long)h->timing_runs, h->timing_layer_us / n,
                     h->timing_us[0][0] / n, h->timing_us[0][1] / n, h->timing_us[0][2] / n,
                     h->timing_us[1][0] / n, h->timing_us[1][1] / n, h->timing_us[1][2] / n,
                     h->timing_us[2][0] / n, h->timing_us[2][1] / n, h->timing_us[2][2] / n);
        std::fflush(stderr);
    }
}

/* ---------------------------------------------------------------- failure-path probe */
__global__ void k_wait_timeout_probe(int polls, int *status) {
    __shared__ unsigned long long bar;
    const unsigned addr = (unsigned)__cvta_generic_to_shared(&bar);
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(addr) : "memory");
    /* nothing ever arrives on this barrier: the wait below can only run out */
    for (int i = 0; i < polls; i++) {
        unsigned ok;
        asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0, 1, 0, p; }" : "=r"(ok) : "r"(addr) : "memory");
        if (ok) return;
    }
    atomicExch(status, SP_KERR_BARRIER_TIMEOUT);
}
extern "C" int sp_moe_debug_wait_timeout(sp_moe *h, int polls, void *stream) {
    if (!h) return fail(SP_MOE_EBADARG, "sp_moe_debug_wait_timeout: NULL handle");
    if (polls < 1 || polls > (1 << 20)) return fail(SP_MOE_EBADARG, "sp_moe_debug_wait_timeout: polls=%d outside [1, 1048576]", polls);
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    cudaStream_t st = (cudaStream_t)stream; h->last_stream = st;
    k_wait_timeout_probe<<<1, 1, 0, st>>>(polls, h->status);
    h->launches += 1;
    CK(cudaGetLastError(), "wait-timeout probe launch");
    return SP_MOE_OK;
}

extern "C" int sp_moe_forward(sp_moe *h, int lf, int nl, int flavour, int M,
                              const float *x, float *y, int32_t *sel, float *wts) {
    int rc = check_forward(h, lf, nl, flavour, M, x, y, "sp_moe_forward");
    if (rc) return rc;
    CK(cudaSetDevice(h->device), "cudaSetDevice");
    const size_t nx = (size_t)M * h->cfg.E * 4, ns = (size_t)nl * M * h->cfg.NU * 4;
    CK(cudaMemcpyAsync(h->x_dev, x, nx, cudaMemcpyHostToDevice, h->stream), "x H2D");
    rc = sp_moe_forward_dev(h, lf, nl, flavour, M, h->x_dev, h->y_dev, sel ? h->sel_dev : nullptr, wts ? h->wts_dev : nullptr, h->stream);
    if (rc) return rc;
    CK(cudaMemcpyAsync(y, h->y_dev, nx, cudaMemcpyDeviceToHost, h->stream), "y D2H");
    if (sel) CK(cudaMemcpyAsync(sel, h->sel_dev, ns, cudaMemcpyDeviceToHost, h->stream), "sel D2H");
    if (wts) CK(cudaMemcpyAsync(wts, h->wts_dev, ns, cudaMemcpyDeviceToHost, h->stream), "wts D2H");
    rc = sp_moe_status(h);
    if (rc == SP_MOE_OK && M == 1 && flavour == SP_MOE_FLAVOUR_DECODE) timing_accumulate(h, nl);
    return rc;
}
