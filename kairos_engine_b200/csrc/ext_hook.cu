/* ext_hook.cu — the reference's MoE plugin hook for SwiGLU models with separate gate / up / down
 * expert tensors (its qwen36 service: sp_q36gpu_upload_experts / sp_q36gpu_moe,
 * src/backends/cuda/cuda_forward.cu:16203-16289, registered through q36_boot_moe_ext,
 * CF:16444-16454): a layer's experts are uploaded once under a tag; a call names the tag, the
 * expert ids and weights the HOST router chose, and a host x[E]; the result is
 *     y = sum_k wt[k] * Wd[idx[k]] . ( silu(Wg[idx[k]] . x) * (Wu[idx[k]] . x) )
 * accumulated in the caller's k order (dg_k_axpy, fused multiply-add), every matmul in the decode
 * arithmetic (gemv_w_packed: int8 per-16 activation quant + Q4B x int8 GEMV, CF:13566-13599).
 * Contract of the hook: 0 = handled (y filled), nonzero = not mine (unknown tag or other shape).
 * Same flow as the reference: one H2D of x, NU x (gate, up, silu*mul, down, axpy) enqueued on one
 * stream, one synchronisation, one D2H of y. Only Q4B tensors are served here.
 */
#include "common.cuh"
#include "gemv_common.cuh"
#include "../../include/sp_engine/moe_backend.h"
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

/* k_silu_mul (CF:1377-1383): g = (g / (1 + exp(-g))) * up */
__global__ void k_ext_silu_mul(float *g, const float *up, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { const float x = g[i]; g[i] = __fmul_rn(__fdiv_rn(x, __fadd_rn(1.0f, expf(-x))), up[i]); }
}
__global__ void k_ext_axpy(float *yo, const float *de, float w, int E) {      /* dg_k_axpy */
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < E) yo[i] = __fmaf_rn(w, de[i], yo[i]);
}

struct ExtLayer {
    std::string tag; int NE, FF, E;
    uint8_t *g_codes, *u_codes, *d_codes; uint16_t *g_bs, *u_bs, *d_bs;
};

int ext_fail(const char *msg) { sp_set_error(msg); return 1; }

}  // namespace

struct ExtScratch {
    float *dX, *dG, *dU, *dDe, *dYo;                       /* x[E], gate[FF], up[FF], down[E], accumulator[E] */
    signed char *qx, *qh; float *sx, *sh; int *cx, *ch;    /* int8 activations of x and of silu(g)*u */
};
struct sp_moe_ext {
    int device;
    cudaStream_t st;
    std::vector<ExtLayer> layers;
    ExtScratch s;
    int cap_e, cap_ff;
};

static void ext_free_scratch(ExtScratch &s) {
    void *ps[] = {s.dX, s.dG, s.dU, s.dDe, s.dYo, s.qx, s.qh, s.sx, s.sh, s.cx, s.ch};
    for (void *p : ps) if (p) cudaFree(p);
    s = ExtScratch{};
}
/* all-or-nothing: on failure whatever was allocated is freed and `s` is left empty */
static bool ext_alloc_scratch(ExtScratch &s, int ce, int cf) {
    s = ExtScratch{};
    const bool ok =
        cudaMalloc((void **)&s.dX, 4 * (size_t)ce) == cudaSuccess && cudaMalloc((void **)&s.dG, 4 * (size_t)cf) == cudaSuccess &&
        cudaMalloc((void **)&s.dU, 4 * (size_t)cf) == cudaSuccess && cudaMalloc((void **)&s.dDe, 4 * (size_t)ce) == cudaSuccess &&
        cudaMalloc((void **)&s.dYo, 4 * (size_t)ce) == cudaSuccess &&
        cudaMalloc((void **)&s.qx, (size_t)ce) == cudaSuccess && cudaMalloc((void **)&s.qh, (size_t)cf) == cudaSuccess &&
        cudaMalloc((void **)&s.sx, 4 * (size_t)(ce / 16)) == cudaSuccess && cudaMalloc((void **)&s.sh, 4 * (size_t)(cf / 16)) == cudaSuccess &&
        cudaMalloc((void **)&s.cx, 4 * (size_t)(ce / 16)) == cudaSuccess && cudaMalloc((void **)&s.ch, 4 * (size_t)(cf / 16)) == cudaSuccess;
    if (!ok) { ext_free_scratch(s); cudaGetLastError(); }
    return ok;
}

extern "C" int sp_moe_ext_open(int device, sp_moe_ext **out) {
    if (!out) return ext_fail("sp_moe_ext_open: NULL argument");
    *out = nullptr;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { cudaGetLastError(); return ext_fail("sp_moe_ext_open: no CUDA device; this library has no CPU path"); }
    if (device < 0 || device >= ndev) return ext_fail("sp_moe_ext_open: device out of range");
    if (cudaSetDevice(device) != cudaSuccess) return ext_fail("sp_moe_ext_open: cudaSetDevice failed");
    sp_moe_ext *h = new sp_moe_ext();
    h->device = device; h->s = ExtScratch{}; h->cap_e = h->cap_ff = 0;
    if (cudaStreamCreateWithFlags(&h->st, cudaStreamNonBlocking) != cudaSuccess) { delete h; return ext_fail("sp_moe_ext_open: stream creation failed"); }
    *out = h;
    return 0;
}

extern "C" int sp_moe_ext_close(sp_moe_ext *h) {
    if (!h) return 0;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->st);
    for (auto &l : h->layers) { void *ps[] = {l.g_codes, l.u_codes, l.d_codes, l.g_bs, l.u_bs, l.d_bs}; for (void *p : ps) cudaFree(p); }
    ext_free_scratch(h->s);
    cudaStreamDestroy(h->st);
    delete h;
    return 0;
}

extern "C" int sp_moe_ext_upload_experts(sp_moe_ext *h, const char *tag,
                                         const uint8_t *gate_codes, const uint16_t *gate_bs,
                                         const uint8_t *up_codes, const uint16_t *up_bs,
                                         const uint8_t *down_codes, const uint16_t *down_bs, int NE, int FF, int E) {
    if (!h || !tag || !gate_codes || !gate_bs || !up_codes || !up_bs || !down_codes || !down_bs) return ext_fail("sp_moe_ext_upload_experts: NULL argument");
    if (NE <= 0 || FF <= 0 || E <= 0 || (FF & 31) || (E & 31) || FF > 4096 || E > 4096) return ext_fail("sp_moe_ext_upload_experts: E and FF must be multiples of 32 in (0, 4096]");
    if (cudaSetDevice(h->device) != cudaSuccess) return ext_fail("sp_moe_ext_upload_experts: cudaSetDevice failed");
    ExtLayer l{}; l.tag = tag; l.NE = NE; l.FF = FF; l.E = E;
    const size_t gb = (size_t)NE * FF * E / 2, gs = (size_t)NE * FF * (E / 32) * 2, db = (size_t)NE * E * FF / 2, ds = (size_t)NE * E * (FF / 32) * 2;
    struct { void **p; const void *src; size_t n; } up[] = {{(void **)&l.g_codes, gate_codes, gb}, {(void **)&l.g_bs, gate_bs, gs}, {(void **)&l.u_codes, up_codes, gb},
                                                           {(void **)&l.u_bs, up_bs, gs}, {(void **)&l.d_codes, down_codes, db}, {(void **)&l.d_bs, down_bs, ds}};
    bool ok = true;
    for (auto &u : up) { *u.p = nullptr; if (ok && (cudaMalloc(u.p, u.n) != cudaSuccess || cudaMemcpy(*u.p, u.src, u.n, cudaMemcpyHostToDevice) != cudaSuccess)) ok = false; }
    if (ok && (E > h->cap_e || FF > h->cap_ff)) {          /* scratch for the largest shapes seen so far */
        /* the larger set is allocated first and swapped in only when it is complete: on failure the old
         * scratch, its sizes and the layers uploaded earlier all stay valid */
        const int ce = E > h->cap_e ? E : h->cap_e, cf = FF > h->cap_ff ? FF : h->cap_ff;
        ExtScratch fresh;
        ok = ext_alloc_scratch(fresh, ce, cf);
        if (ok) {
            cudaStreamSynchronize(h->st);
            ext_free_scratch(h->s);
            h->s = fresh; h->cap_e = ce; h->cap_ff = cf;
        }
    }
    if (!ok) {
        for (auto &u : up) if (*u.p) cudaFree(*u.p);
        cudaGetLastError();
        return ext_fail("sp_moe_ext_upload_experts: device allocation or copy failed");
    }
    h->layers.push_back(l);
    return 0;
}

extern "C" int sp_moe_ext_moe(void *vh, const char *tag, const int *idx, const float *wt, int NU,
                              const float *x, int E, int FF, float *y) {
    sp_moe_ext *h = (sp_moe_ext *)vh;
    if (!h || !tag || !idx || !wt || !x || !y || NU <= 0) return -1;
    const ExtLayer *M = nullptr;
    for (const auto &l : h->layers) if (l.tag == tag) { M = &l; break; }
    if (!M || M->FF != FF || M->E != E) return -1;                       /* not mine */
    for (int k = 0; k < NU; k++) if (idx[k] < 0 || idx[k] >= M->NE) { sp_set_error("sp_moe_ext_moe: expert index out of range"); return -1; }
    if (cudaSetDevice(h->device) != cudaSuccess) return -1;
    cudaStream_t st = h->st;
    if (cudaMemcpyAsync(h->s.dX, x, 4 * (size_t)E, cudaMemcpyHostToDevice, st) != cudaSuccess) return -1;
    if (cudaMemsetAsync(h->s.dYo, 0, 4 * (size_t)E, st) != cudaSuccess) return -1;
    const size_t grow = (size_t)FF * (E / 2), gsrow = (size_t)FF * (E / 32), drow = (size_t)E * (FF / 2), dsrow = (size_t)E * (FF / 32);
    k_quant_act<<<(E / 16 + 127) / 128, 128, 0, st>>>(h->s.dX, E, h->s.qx, h->s.sx, h->s.cx);       /* the same x feeds every expert's gate and up */
    for (int k = 0; k < NU; k++) {
        const size_t e = (size_t)idx[k];
        k_gemv_q4b<<<(FF + 7) / 8, 256, 0, st>>>(M->g_codes + e * grow, M->g_bs + e * gsrow, E, FF, h->s.qx, h->s.sx, h->s.cx, h->s.dG);
        k_gemv_q4b<<<(FF + 7) / 8, 256, 0, st>>>(M->u_codes + e * grow, M->u_bs + e * gsrow, E, FF, h->s.qx, h->s.sx, h->s.cx, h->s.dU);
        k_ext_silu_mul<<<(FF + 255) / 256, 256, 0, st>>>(h->s.dG, h->s.dU, FF);
        k_quant_act<<<(FF / 16 + 127) / 128, 128, 0, st>>>(h->s.dG, FF, h->s.qh, h->s.sh, h->s.ch);
        k_gemv_q4b<<<(E + 7) / 8, 256, 0, st>>>(M->d_codes + e * drow, M->d_bs + e * dsrow, FF, E, h->s.qh, h->s.sh, h->s.ch, h->s.dDe);
        k_ext_axpy<<<(E + 255) / 256, 256, 0, st>>>(h->s.dYo, h->s.dDe, wt[k], E);
    }
    if (cudaMemcpyAsync(y, h->s.dYo, 4 * (size_t)E, cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
    return cudaStreamSynchronize(st) == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -1;
}
