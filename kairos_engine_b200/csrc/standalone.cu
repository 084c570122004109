/* standalone.cu — gemma4_moe_ffn_q4b_cuda, the reference's self-contained single-token MoE
 * operator (CF:13821-13977 of src/backends/cuda/cuda_forward.cu), same signature and semantics:
 * all pointers are host memory; it allocates, uploads the whole packed expert set, runs and frees.
 *
 * Semantics (they differ from the served layer, decode_graph.cu): ONE weightless rmsnorm with a
 * float sum of squares (dg_k_rmsnorm_vec, CF:13632-13644); experts consume that normed vector;
 * router input = normed * (1/sqrt(E) * scale[i]) (CF:13647-13650); logits by a lane-strided
 * fp32 GEMV (dg_k_gemv_f32, CF:13655-13665); host softmax with float expf and a double sum,
 * greedy top-NU with strict > (ties to the lower id), renormalised without a clamp
 * (CF:13908-13925); per expert in descending-probability order: int8 activation quant + Q4B
 * dp4a GEMV gate|up, GeGLU, quant, down GEMV, yo += w * de (CF:13930-13958).
 */
#include "common.cuh"
#include "gemv_common.cuh"
#include "../../include/sp_engine/moe_backend.h"
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <vector>

namespace {

__global__ void k_sa_rmsnorm_vec(const float *x, int E, float eps, float *out) {
    extern __shared__ float sh[];
    float acc = 0.0f;
    for (int i = threadIdx.x; i < E; i += blockDim.x) acc = __fmaf_rn(x[i], x[i], acc);
    sh[threadIdx.x] = acc; __syncthreads();
    for (int s = blockDim.x >> 1; s > 0; s >>= 1) { if (threadIdx.x < s) sh[threadIdx.x] += sh[threadIdx.x + s]; __syncthreads(); }
    const float inv = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sh[0], (float)E), eps)));
    for (int i = threadIdx.x; i < E; i += blockDim.x) out[i] = __fmul_rn(x[i], inv);
}
__global__ void k_sa_router_in(const float *xn, const float *scale_vec, float rscale, int E, float *tmp) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < E) tmp[i] = __fmul_rn(xn[i], __fmul_rn(rscale, scale_vec[i]));
}
__global__ void k_sa_gemv_f32(const float *W, const float *x, float *y, int in, int out) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = blockIdx.x * (blockDim.x >> 5) + warp;
    if (o >= out) return;
    const float *wr = W + (size_t)o * in;
    float acc = 0.0f;
    for (int i = lane; i < in; i += 32) acc = __fmaf_rn(wr[i], x[i], acc);
    for (int s = 16; s > 0; s >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, s);
    if (lane == 0) y[o] = acc;
}
__global__ void k_sa_geglu(const float *gu, float *h, int FF) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < FF) h[i] = gelu_mul(gu[i], gu[FF + i]);
}
__global__ void k_sa_axpy(float *yo, const float *de, float w, int E) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < E) yo[i] = __fmaf_rn(w, de[i], yo[i]);
}

struct DevBufs {
    std::vector<void *> all;
    template <class T> cudaError_t get(T **p, size_t n) { void *v = nullptr; cudaError_t e = cudaMalloc(&v, n * sizeof(T)); if (e == cudaSuccess) all.push_back(v); *p = (T *)v; return e; }
    ~DevBufs() { for (void *p : all) cudaFree(p); }
};

}  // namespace

extern "C" int gemma4_moe_ffn_q4b_cuda(int E, int NE, int NU, int FF, float eps,
                                       const float *gate_inp, const float *gate_inp_scale,
                                       const unsigned char *gu_codes, const unsigned short *gu_bscale,
                                       const unsigned char *dn_codes, const unsigned short *dn_bscale,
                                       const float *hidden, float *out, int *sel_out) {
    if (E <= 0 || FF <= 0 || (E & 31) || (FF & 31)) { sp_set_error("moe_q4b: E,FF must be %32"); return 1; }     /* CF:13828 */
    if (NE <= 0 || NU <= 0 || NU > NE || !gate_inp || !gate_inp_scale || !gu_codes || !gu_bscale || !dn_codes || !dn_bscale || !hidden || !out) {
        sp_set_error("moe_q4b: bad argument"); return 1; }
    const size_t gu_rows = (size_t)FF * 2, dn_rows = (size_t)E;
    const size_t gu_cb = (size_t)NE * gu_rows * (E / 2), dn_cb = (size_t)NE * dn_rows * (FF / 2);
    const size_t gu_sn = (size_t)NE * gu_rows * (E / 32), dn_sn = (size_t)NE * dn_rows * (FF / 32);
    const int maxin = E > FF ? E : FF;
    DevBufs B;
    float *d_hidden, *d_x, *d_tmp, *d_scale, *d_gi, *d_logits, *d_gu, *d_h, *d_de, *d_yo, *d_sx;
    unsigned char *d_gc, *d_dc; unsigned short *d_gs, *d_ds; signed char *d_q; int *d_corr;
#define SA(call, what) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { char b_[256]; snprintf(b_, sizeof b_, "moe_q4b: %s: %s", what, cudaGetErrorString(e_)); sp_set_error(b_); cudaGetLastError(); return 1; } } while (0)
    SA(B.get(&d_hidden, E), "cudaMalloc"); SA(B.get(&d_x, E), "cudaMalloc"); SA(B.get(&d_tmp, E), "cudaMalloc"); SA(B.get(&d_scale, E), "cudaMalloc");
    SA(B.get(&d_gi, (size_t)NE * E), "cudaMalloc"); SA(B.get(&d_logits, NE), "cudaMalloc"); SA(B.get(&d_gu, 2 * (size_t)FF), "cudaMalloc");
    SA(B.get(&d_h, FF), "cudaMalloc"); SA(B.get(&d_de, E), "cudaMalloc"); SA(B.get(&d_yo, E), "cudaMalloc");
    SA(B.get(&d_gc, gu_cb), "packed cudaMalloc"); SA(B.get(&d_dc, dn_cb), "packed cudaMalloc");
    SA(B.get(&d_gs, gu_sn), "packed cudaMalloc"); SA(B.get(&d_ds, dn_sn), "packed cudaMalloc");
    SA(B.get(&d_q, maxin), "actq cudaMalloc"); SA(B.get(&d_sx, maxin / 16), "actq cudaMalloc"); SA(B.get(&d_corr, maxin / 16), "actq cudaMalloc");
    SA(cudaMemcpy(d_gc, gu_codes, gu_cb, cudaMemcpyHostToDevice), "packed H2D"); SA(cudaMemcpy(d_dc, dn_codes, dn_cb, cudaMemcpyHostToDevice), "packed H2D");
    SA(cudaMemcpy(d_gs, gu_bscale, gu_sn * 2, cudaMemcpyHostToDevice), "packed H2D"); SA(cudaMemcpy(d_ds, dn_bscale, dn_sn * 2, cudaMemcpyHostToDevice), "packed H2D");
    SA(cudaMemcpy(d_hidden, hidden, (size_t)E * 4, cudaMemcpyHostToDevice), "H2D copy");
    SA(cudaMemcpy(d_scale, gate_inp_scale, (size_t)E * 4, cudaMemcpyHostToDevice), "H2D copy");
    SA(cudaMemcpy(d_gi, gate_inp, (size_t)NE * E * 4, cudaMemcpyHostToDevice), "H2D copy");
    cudaStream_t st = 0;
    { int bd = 256; while (bd > E && bd > 32) bd >>= 1;
      k_sa_rmsnorm_vec<<<1, bd, bd * sizeof(float), st>>>(d_hidden, E, eps, d_x);
      k_sa_router_in<<<(E + 255) / 256, 256, 0, st>>>(d_x, d_scale, 1.0f / sqrtf((float)E), E, d_tmp); }
    k_sa_gemv_f32<<<(NE + 7) / 8, 256, 0, st>>>(d_gi, d_tmp, d_logits, E, NE);
    std::vector<float> lg(NE);
    SA(cudaMemcpy(lg.data(), d_logits, (size_t)NE * 4, cudaMemcpyDeviceToHost), "logits D2H");
    std::vector<int> idx(NU); std::vector<float> wt(NU);
    {   /* CF:13908-13925 */
        float mx = lg[0];
        for (int i = 1; i < NE; i++) if (lg[i] > mx) mx = lg[i];
        double se = 0.0;
        for (int i = 0; i < NE; i++) { lg[i] = expf(lg[i] - mx); se += lg[i]; }
        for (int i = 0; i < NE; i++) lg[i] = (float)(lg[i] / se);
        std::vector<char> used(NE, 0);
        float wsum = 0.0f;
        for (int k = 0; k < NU; k++) {
            int best = -1; float bv = -1.0f;
            for (int i = 0; i < NE; i++) if (!used[i] && lg[i] > bv) { bv = lg[i]; best = i; }
            if (best < 0) { sp_set_error("moe_q4b: router produced no usable expert (NaN logits)"); return 1; }
            used[best] = 1; idx[k] = best; wt[k] = bv; wsum += bv;
        }
        for (int k = 0; k < NU; k++) wt[k] = (wt[k] / wsum) * 1.0f;
        if (sel_out) for (int k = 0; k < NU; k++) sel_out[k] = idx[k];
    }
    SA(cudaMemsetAsync(d_yo, 0, (size_t)E * 4, st), "memset");
    for (int k = 0; k < NU; k++) {
        const int e = idx[k];
        k_quant_act<<<1, 256, 0, st>>>(d_x, E, d_q, d_sx, d_corr);
        k_gemv_q4b<<<(unsigned)((gu_rows + 7) / 8), 256, 0, st>>>(d_gc + (size_t)e * gu_rows * (E / 2), d_gs + (size_t)e * gu_rows * (E / 32),
                                                                  E, (int)gu_rows, d_q, d_sx, d_corr, d_gu);
        k_sa_geglu<<<(FF + 255) / 256, 256, 0, st>>>(d_gu, d_h, FF);
        k_quant_act<<<1, 256, 0, st>>>(d_h, FF, d_q, d_sx, d_corr);
        k_gemv_q4b<<<(unsigned)((dn_rows + 7) / 8), 256, 0, st>>>(d_dc + (size_t)e * dn_rows * (FF / 2), d_ds + (size_t)e * dn_rows * (FF / 32),
                                                                  FF, (int)dn_rows, d_q, d_sx, d_corr, d_de);
        k_sa_axpy<<<(E + 255) / 256, 256, 0, st>>>(d_yo, d_de, wt[k], E);
    }
    SA(cudaGetLastError(), "kernel launch");
    SA(cudaMemcpy(out, d_yo, (size_t)E * 4, cudaMemcpyDeviceToHost), "out D2H");
    SA(cudaDeviceSynchronize(), "sync");
#undef SA
    return 0;
}

/* gemv_w_packed for OK_Q4B (CF:13566-13599): y[rows] = Q4B(W)[rows][in] . x[in] in the decode
 * arithmetic: k_quant_act_int8 on x (CF:1564-1585), then k_gemv_q4b_dp4a_v2 (CF:1688-1713).
 * Device pointers. The reference's caller owns the int8 scratch (dqx, dsx); here the call
 * allocates it and frees it again. */
extern "C" int sp_moe_gemv_q4b_dev(const uint8_t *codes_dev, const uint16_t *bs_dev, int in, int rows,
                                   const float *x_dev, float *y_dev, void *stream) {
    if (!codes_dev || !bs_dev || !x_dev || !y_dev || in <= 0 || rows <= 0 || (in & 31) || in > 4096) {     /* gemv_w_packed declines in % 32 != 0, CF:13574 */
        sp_set_error("sp_moe_gemv_q4b_dev: bad argument (in must be a multiple of 32, at most 4096)"); return SP_MOE_EBADARG; }
    cudaStream_t st = (cudaStream_t)stream;
    signed char *q = nullptr; float *sx = nullptr; int *corr = nullptr;
    cudaError_t e = cudaMalloc(&q, (size_t)in);
    if (e == cudaSuccess) e = cudaMalloc(&sx, sizeof(float) * (in / 16));
    if (e == cudaSuccess) e = cudaMalloc(&corr, sizeof(int) * (in / 16));
    if (e == cudaSuccess) {
        k_quant_act<<<1, 256, 0, st>>>(x_dev, in, q, sx, corr);
        k_gemv_q4b<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(codes_dev, bs_dev, in, rows, q, sx, corr, y_dev);
        e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaStreamSynchronize(st);            /* the scratch is freed below */
    }
    cudaFree(q); cudaFree(sx); cudaFree(corr);
    if (e != cudaSuccess) { char b[256]; snprintf(b, sizeof b, "sp_moe_gemv_q4b_dev: %s", cudaGetErrorString(e)); sp_set_error(b); cudaGetLastError();
        return e == cudaErrorMemoryAllocation ? SP_MOE_EBACKEND_OOM : SP_MOE_ECUDA; }
    return SP_MOE_OK;
}

/* ---------------------------------------------------------------- the same GEMV with no allocation
 * Some callers must not allocate device memory when they call: a serving loop that has already
 * committed the whole card to pre-sized arenas (cudaMalloc can then fail, and cudaMalloc/cudaFree
 * stall every stream of the device while they run), or a component that is handed buffers by its
 * host and has no business touching the allocator at all. For them the int8 scratch of the GEMV
 * lives in this fixed array, which every device that loads the library holds until the process
 * exits: SP_MOE_GEMV_STATIC_MAX_IN codes + two 4-byte words per 16 inputs = 6 KB.
 *
 * In host code the array's name is only a stand-in; the device address comes from
 * cudaGetSymbolAddress, asked once per device with that device current. */
#define SP_MOE_GEMV_STATIC_MAX_IN 4096
static __device__ __align__(256) unsigned char g_gemv_static_scratch[SP_MOE_GEMV_STATIC_MAX_IN + 2 * 4 * (SP_MOE_GEMV_STATIC_MAX_IN / 16)];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
unsigned char *g_static_ptr[kMaxDevices];     /* device address of the array, per device; NULL until set up */
}

extern "C" int sp_moe_gemv_q4b_static_dev(const uint8_t *codes_dev, const uint16_t *bs_dev, int in, int rows,
                                          const float *x_dev, float *y_dev, void *stream) {
    if (!codes_dev || !bs_dev || !x_dev || !y_dev || in <= 0 || rows <= 0 || (in & 31)) {
        sp_set_error("sp_moe_gemv_q4b_static_dev: bad argument (in must be a positive multiple of 32)"); return SP_MOE_EBADARG; }
    if (in > SP_MOE_GEMV_STATIC_MAX_IN) {
        char b[192]; snprintf(b, sizeof b, "sp_moe_gemv_q4b_static_dev: in=%d exceeds the fixed scratch (at most %d inputs); use sp_moe_gemv_q4b_dev", in, SP_MOE_GEMV_STATIC_MAX_IN);
        sp_set_error(b); return SP_MOE_EBADARG; }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess && (dev < 0 || dev >= kMaxDevices)) { sp_set_error("sp_moe_gemv_q4b_static_dev: device ordinal out of range"); return SP_MOE_EUNSUPPORTED; }
    unsigned char *base = nullptr;
    if (e == cudaSuccess) {
        std::lock_guard<std::mutex> lk(g_static_mu);
        if (!g_static_ptr[dev]) {                                 /* first call on this device: look the array up */
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_gemv_static_scratch);
            if (e == cudaSuccess) g_static_ptr[dev] = static_cast<unsigned char *>(p);
        }
        base = g_static_ptr[dev];
    }
    if (e == cudaSuccess) {
        cudaStream_t st = (cudaStream_t)stream;
        signed char *q = reinterpret_cast<signed char *>(base);
        float *sx = reinterpret_cast<float *>(base + SP_MOE_GEMV_STATIC_MAX_IN);
        int *corr = reinterpret_cast<int *>(base + SP_MOE_GEMV_STATIC_MAX_IN + 4 * (SP_MOE_GEMV_STATIC_MAX_IN / 16));
        /* nothing in the scratch has to start at zero: the quantiser writes every byte the GEMV reads */
        k_quant_act<<<1, 256, 0, st>>>(x_dev, in, q, sx, corr);
        k_gemv_q4b<<<(unsigned)((rows + 7) / 8), 256, 0, st>>>(codes_dev, bs_dev, in, rows, q, sx, corr, y_dev);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) { char b[256]; snprintf(b, sizeof b, "sp_moe_gemv_q4b_static_dev: %s", cudaGetErrorString(e)); sp_set_error(b); cudaGetLastError(); return SP_MOE_ECUDA; }
    return SP_MOE_OK;
}
