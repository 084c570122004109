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
#include "../../include/sp_engine/moe_backend.h"
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

namespace {

__global__ void k_ext_quant(const float *x, int n, signed char *q, float *sx, int *corr) {
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < (n >> 4); b += gridDim.x * blockDim.x) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = x[16 * b + i];
        sx[b] = quant_block16(v, q + 16 * b, corr + b);
    }
}
/* k_gemv_q4b_dp4a_v2 (CF:1688-1713): warp per row, chunk c on lane c % 32, shuffle tree */
__global__ void k_ext_gemv(const uint8_t *codes, const uint16_t *bs, int in, int out,
                           const signed char *q, const float *sx, const int *corr, float *y) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * (blockDim.x >> 5) + warp;
    if (j >= out) return;
    const int n32 = in >> 5;
    const uint8_t *row = codes + (size_t)j * (in >> 1);
    const uint16_t *rbs = bs + (size_t)j * n32;
    const int4 *q4 = reinterpret_cast<const int4 *>(q);
    float facc = 0.0f;
    for (int c = lane; c < n32; c += 32) {
        const int4 w = ld_stream16(row + 16 * (size_t)c);
        int a0, a1;
        q4b_chunk_dot(w, q4[2 * c], q4[2 * c + 1], corr[2 * c], corr[2 * c + 1], a0, a1);
        const float t = __fmaf_rn((float)a0, sx[2 * c], __fmul_rn((float)a1, sx[2 * c + 1]));
        facc = __fmaf_rn(h2f(rbs[c]), t, facc);
    }
    for (int o = 16; o > 0; o >>= 1) facc += __shfl_down_sync(0xffffffffu, facc, o);
    if (lane == 0) y[j] = facc;
}
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

struct sp_moe_ext {
    int device;
    cudaStream_t st;
    std::vector<ExtLayer> layers;
    float *dX, *dG, *dU, *dDe, *dYo;                       /* x[E], gate[FF], up[FF], down[E], accumulator[E] */
    signed char *qx, *qh; float *sx, *sh; int *cx, *ch;    /* int8 activations of x and of silu(g)*u */
    int cap_e, cap_ff;
};

extern "C" int sp_moe_ext_open(int device, sp_moe_ext **out) {
    if (!out) return ext_fail("sp_moe_ext_open: NULL argument");
    *out = nullptr;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { cudaGetLastError(); return ext_fail("sp_moe_ext_open: no CUDA device; this library has no CPU path"); }
    if (device < 0 || device >= ndev) return ext_fail("sp_moe_ext_open: device out of range");
    if (cudaSetDevice(device) != cudaSuccess) return ext_fail("sp_moe_ext_open: cudaSetDevice failed");
    sp_moe_ext *h = new sp_moe_ext();
    h->device = device; h->dX = nullptr; h->cap_e = h->cap_ff = 0;
    if (cudaStreamCreateWithFlags(&h->st, cudaStreamNonBlocking) != cudaSuccess) { delete h; return ext_fail("sp_moe_ext_open: stream creation failed"); }
    *out = h;
    return 0;
}

static void ext_free_scratch(sp_moe_ext *h) {
    void *ps[] = {h->dX, h->dG, h->dU, h->dDe, h->dYo, h->qx, h->qh, h->sx, h->sh, h->cx, h->ch};
    if (h->dX) for (void *p : ps) cudaFree(p);
    h->dX = nullptr;
}

extern "C" int sp_moe_ext_close(sp_moe_ext *h) {
    if (!h) return 0;
    cudaSetDevice(h->device);
    cudaStreamSynchronize(h->st);
    for (auto &l : h->layers) { void *ps[] = {l.g_codes, l.u_codes, l.d_codes, l.g_bs, l.u_bs, l.d_bs}; for (void *p : ps) cudaFree(p); }
    ext_free_scratch(h);
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
        ext_free_scratch(h);
        const int ce = E > h->cap_e ? E : h->cap_e, cf = FF > h->cap_ff ? FF : h->cap_ff;
        ok = cudaMalloc((void **)&h->dX, 4 * (size_t)ce) == cudaSuccess && cudaMalloc((void **)&h->dG, 4 * (size_t)cf) == cudaSuccess &&
             cudaMalloc((void **)&h->dU, 4 * (size_t)cf) == cudaSuccess && cudaMalloc((void **)&h->dDe, 4 * (size_t)ce) == cudaSuccess &&
             cudaMalloc((void **)&h->dYo, 4 * (size_t)ce) == cudaSuccess &&
             cudaMalloc((void **)&h->qx, (size_t)ce) == cudaSuccess && cudaMalloc((void **)&h->qh, (size_t)cf) == cudaSuccess &&
             cudaMalloc((void **)&h->sx, 4 * (size_t)(ce / 16)) == cudaSuccess && cudaMalloc((void **)&h->sh, 4 * (size_t)(cf / 16)) == cudaSuccess &&
             cudaMalloc((void **)&h->cx, 4 * (size_t)(ce / 16)) == cudaSuccess && cudaMalloc((void **)&h->ch, 4 * (size_t)(cf / 16)) == cudaSuccess;
        h->cap_e = ce; h->cap_ff = cf;
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
    if (cudaMemcpyAsync(h->dX, x, 4 * (size_t)E, cudaMemcpyHostToDevice, st) != cudaSuccess) return -1;
    if (cudaMemsetAsync(h->dYo, 0, 4 * (size_t)E, st) != cudaSuccess) return -1;
    const size_t grow = (size_t)FF * (E / 2), gsrow = (size_t)FF * (E / 32), drow = (size_t)E * (FF / 2), dsrow = (size_t)E * (FF / 32);
    k_ext_quant<<<(E / 16 + 127) / 128, 128, 0, st>>>(h->dX, E, h->qx, h->sx, h->cx);       /* the same x feeds every expert's gate and up */
    for (int k = 0; k < NU; k++) {
        const size_t e = (size_t)idx[k];
        k_ext_gemv<<<(FF + 7) / 8, 256, 0, st>>>(M->g_codes + e * grow, M->g_bs + e * gsrow, E, FF, h->qx, h->sx, h->cx, h->dG);
        k_ext_gemv<<<(FF + 7) / 8, 256, 0, st>>>(M->u_codes + e * grow, M->u_bs + e * gsrow, E, FF, h->qx, h->sx, h->cx, h->dU);
        k_ext_silu_mul<<<(FF + 255) / 256, 256, 0, st>>>(h->dG, h->dU, FF);
        k_ext_quant<<<(FF / 16 + 127) / 128, 128, 0, st>>>(h->dG, FF, h->qh, h->sh, h->ch);
        k_ext_gemv<<<(E + 7) / 8, 256, 0, st>>>(M->d_codes + e * drow, M->d_bs + e * dsrow, FF, E, h->qh, h->sh, h->ch, h->dDe);
        k_ext_axpy<<<(E + 255) / 256, 256, 0, st>>>(h->dYo, h->dDe, wt[k], E);
    }
    if (cudaMemcpyAsync(y, h->dYo, 4 * (size_t)E, cudaMemcpyDeviceToHost, st) != cudaSuccess) return -1;
    return cudaStreamSynchronize(st) == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -1;
}
