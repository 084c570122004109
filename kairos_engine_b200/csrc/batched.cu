/* batched.cu — the M > 1 paths of the MoE feed-forward layer: a few stream-ordered kernels per
 * layer with routing, bucketing and combine all on the device (no host round trip).
 *
 * Replaces g4_ffn_apply's expert-major batched branch (CF:8430-8965 of
 * src/backends/cuda/cuda_forward.cu): batched router prep + router GEMM, the D2H + host top-k +
 * host bucketing (CF:8483-8625), per-expert gather / GEMM / GELU split / GEMM / scatter-acc
 * (CF:8925-8965), and the recombine (CF:9014-9019).
 *
 * Two arithmetic flavours, the reference's AMMD switch (CF:8322-8324):
 *   decode  (per-token int8 activation quant + exact integer dots; what B sequential decode
 *            steps compute, CF:11737-11757) for small batches;
 *   prefill (w = code * f16 scale exactly, floating-point dot, fp32 accumulate; gemm_w,
 *            CF:13488-13518) for large ones.
 * Every (token, expert) pair is computed independently and the per-token combine walks the
 * experts in ascending id with acc = acc + w*out, so results do not depend on scheduling.
 */
#include "batched.cuh"
#include "prefill_tc.cuh"
#include <cstdlib>
#include "../../include/sp_engine/moe_backend.h"

namespace {

struct BView {                 /* carved scratch */
    float *rin, *nx_f, *in_f, *logits, *cw, *hd, *dn, *h, *eo, *xa, *xb;
    signed char *nx_q, *in_q, *hd_q, *h_q;
    float *nx_s, *in_s, *hd_s, *h_s;
    int *nx_c, *in_c, *hd_c, *h_c;
    int *sel_asc, *count, *list, *pairpos, *ep_off;
    signed char *ep_q; float *ep_s; int *ep_c;      /* expert-parallel stage: quantised received rows, [max_rows] */
};

size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
constexpr int kSlices = SP_BATCHED_MAX_SLICES;     /* token slices of one layer that may be between route and finish at the same time */

template <class F>
size_t blayout(const SpDims &d, int Mx, int Rx, F place) {
    size_t o = 0; int id = 0;
    auto take = [&](size_t bytes) { place(id++, o); o = up256(o + bytes); };
    const size_t M = Mx, R = Rx, E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;    /* R >= M * NU */
    take(4 * M * E); take(4 * M * E); take(4 * M * E); take(4 * M * NE); take(4 * M * NU);            /* rin nx_f in_f logits cw */
    take(4 * M * FFS); take(4 * M * E); take(4 * R * FFE); take(4 * M * NU * E);                     /* hd dn h eo */
    take(4 * M * E); take(4 * M * E);                                                               /* xa xb */
    take(M * E); take(M * E); take(M * FFS); take(R * FFE);                                          /* q */
    take(4 * M * (E / 16)); take(4 * M * (E / 16)); take(4 * M * (FFS / 16)); take(4 * R * (FFE / 16));        /* s */
    take(4 * M * (E / 16)); take(4 * M * (E / 16)); take(4 * M * (FFS / 16)); take(4 * R * (FFE / 16));        /* c */
    take(4 * M * NU); take(4 * NE * kSlices); take(4 * NE * M);                                     /* sel_asc count list */
    take(R * E); take(4 * R * (E / 16)); take(4 * R * (E / 16));                                    /* ep_q ep_s ep_c */
    take(4 * M * NU); take(4 * (NE + 1) * kSlices);                                                 /* pairpos ep_off */
    return o;
}
BView bview(const SpDims &d, const SpBatchedScratch *s) {
    unsigned char *p[31];
    blayout(d, s->max_tokens, s->max_rows, [&](int id, size_t off) { p[id] = (unsigned char *)s->base + off; });
    BView v;
    v.rin = (float *)p[0]; v.nx_f = (float *)p[1]; v.in_f = (float *)p[2]; v.logits = (float *)p[3]; v.cw = (float *)p[4];
    v.hd = (float *)p[5]; v.dn = (float *)p[6]; v.h = (float *)p[7]; v.eo = (float *)p[8]; v.xa = (float *)p[9]; v.xb = (float *)p[10];
    v.nx_q = (signed char *)p[11]; v.in_q = (signed char *)p[12]; v.hd_q = (signed char *)p[13]; v.h_q = (signed char *)p[14];
    v.nx_s = (float *)p[15]; v.in_s = (float *)p[16]; v.hd_s = (float *)p[17]; v.h_s = (float *)p[18];
    v.nx_c = (int *)p[19]; v.in_c = (int *)p[20]; v.hd_c = (int *)p[21]; v.h_c = (int *)p[22];
    v.sel_asc = (int *)p[23]; v.count = (int *)p[24]; v.list = (int *)p[25];
    v.ep_q = (signed char *)p[26]; v.ep_s = (float *)p[27]; v.ep_c = (int *)p[28]; v.pairpos = (int *)p[29]; v.ep_off = (int *)p[30];
    return v;
}
/* The same scratch seen by token slice `slice` of a layer, whose first token is `t0`: everything the route stage
 * leaves for the finish stage (per-token and per-pair rows, the per-expert counters) moves to the slice's own
 * place, so several slices of one layer can be between route and finish at once (an expert-parallel run pipelines
 * them). What only the experts stage uses (h, the received rows' quantised copies) is shared: that stage runs one
 * slice at a time. */
BView bview_slice(const SpDims &d, const SpBatchedScratch *s, int t0, int slice) {
    BView v = bview(d, s);
    const size_t E = d.E, NE = d.NE, NU = d.NU, FFS = d.FFS, t = (size_t)t0;
    v.rin += t * E; v.nx_f += t * E; v.in_f += t * E; v.logits += t * NE; v.cw += t * NU; v.hd += t * FFS; v.dn += t * E; v.eo += t * NU * E;
    v.nx_q += t * E; v.in_q += t * E; v.hd_q += t * FFS;
    v.nx_s += t * (E / 16); v.in_s += t * (E / 16); v.hd_s += t * (FFS / 16);
    v.nx_c += t * (E / 16); v.in_c += t * (E / 16); v.hd_c += t * (FFS / 16);
    v.sel_asc += t * NU; v.pairpos += t * NU; v.list += t * NE;
    v.count += (size_t)slice * NE; v.ep_off += (size_t)slice * (NE + 1);
    return v;
}

/* ---------------------------------------------------------------- device helpers */
/* sum of squares in the reference's order (k_rmsnorm, CF:503-511); blockDim.x == 256 */
__device__ double sumsq256(const float *v, int n, double *sh) {
    const int t = threadIdx.x;
    double s = 0.0;
    for (int i = t; i < n; i += 256) { const double a = v[i]; s += a * a; }
    sh[t] = s;
    __syncthreads();
    for (int o = 128; o >= 32; o >>= 1) { if (t < o) sh[t] += sh[t + o]; __syncthreads(); }
    if (t < 32) {
        double a = sh[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_down_sync(0xffffffffu, a, o);
        if (t == 0) sh[0] = a;
    }
    __syncthreads();
    const double r = sh[0];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float rms_scale_from(double ss, int n, float eps) {
    const float ms = (float)(ss / (double)n);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
}
__device__ __forceinline__ float warp_tree(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}
/* quantise one row with all 256 threads (k_quant_act_int8_batched, CF:1725-1746) */
template <class F>
__device__ __forceinline__ void quant_row(int n, signed char *q, float *sx, int *corr, F get) {
    for (int base = 0; base < n; base += 256) {
        const int i = base + (int)threadIdx.x;
        const bool valid = i < n;
        const float v = valid ? get(i) : 0.0f;
        const int b = i >> 4;
        quant_elem16(v, valid, q + 16 * b, sx + b, corr + b);
    }
}

/* ---------------------------------------------------------------- K1: per-token norms of x (CF:8347, 8402-8404, 8425) */
/* block sum of 256 per-thread doubles in sumsq256's order */
__device__ double block_sum256(double s, double *sh) {
    const int t = threadIdx.x;
    sh[t] = s;
    __syncthreads();
    for (int o = 128; o >= 32; o >>= 1) { if (t < o) sh[t] += sh[t + o]; __syncthreads(); }
    if (t < 32) {
        double a = sh[t];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_down_sync(0xffffffffu, a, o);
        if (t == 0) sh[0] = a;
    }
    __syncthreads();
    const double r = sh[0];
    __syncthreads();
    return r;
}
/* One block per token. Everything a thread needs (its 256-strided elements of x and of the three norm
 * vectors) is fetched before the first dependent step, so a block pays the memory latency once and not
 * once per 256 elements; rows wider than 256 * kPrepK take the plain loops. */
constexpr int kPrepK = 12;
template <bool FA>
__global__ void __launch_bounds__(256) k_b_prep(SpDims d, SpLayerDev L, const float *x, BView v, float *rows_f) {
    __shared__ double sh[256];
    const int t = blockIdx.x, E = d.E, tid = threadIdx.x;
    const float *xt = x + (size_t)t * E;
    if (t == 0) for (int i = tid; i < d.NE; i += 256) v.count[i] = 0;
    if (E <= 256 * kPrepK) {
        float xv[kPrepK], n1[kPrepK], n2[kPrepK], rs[kPrepK];
#pragma unroll
        for (int k = 0; k < kPrepK; k++) {
            const int i = tid + 256 * k; const bool ok = i < E;
            xv[k] = ok ? xt[i] : 0.0f; n1[k] = ok ? __ldg(L.ffn_norm + i) : 0.0f;
            n2[k] = ok ? __ldg(L.pre_ffw2 + i) : 0.0f; rs[k] = ok ? __ldg(L.router_scale + i) : 0.0f;
        }
        double ss = 0.0;
#pragma unroll
        for (int k = 0; k < kPrepK; k++) if (256 * k < E) { const double a = xv[k]; if (tid + 256 * k < E) ss += a * a; }
        const float scale = rms_scale_from(block_sum256(ss, sh), E, d.eps);
        const size_t b16 = (size_t)t * (E / 16), row = (size_t)t * E;
#pragma unroll
        for (int k = 0; k < kPrepK; k++) {
            if (256 * k < E) {                                  /* block-uniform: every lane of a warp reaches the shuffles */
                const int i = tid + 256 * k; const bool ok = i < E;
                const float xs = __fmul_rn(xv[k], scale);
                const float nv = __fmul_rn(xs, n1[k]), iv = __fmul_rn(xs, n2[k]);
                if (FA) {
                    const int b = i >> 4;
                    quant_elem16(nv, ok, v.nx_q + row + 16 * b, v.nx_s + b16 + b, v.nx_c + b16 + b);
                    quant_elem16(iv, ok, v.in_q + row + 16 * b, v.in_s + b16 + b, v.in_c + b16 + b);
                } else if (ok) { v.nx_f[row + i] = nv; v.in_f[row + i] = iv; }
                if (ok) {
                    if (rows_f) rows_f[row + i] = iv;
                    v.rin[row + i] = __fmul_rn(__fmul_rn(xs, d.inv_sqrt_e), rs[k]);
                }
            }
        }
        return;
    }
    const float scale = rms_scale_from(sumsq256(xt, E, sh), E, d.eps);
    if (FA) {
        const size_t b16 = (size_t)t * (E / 16);
        quant_row(E, v.nx_q + (size_t)t * E, v.nx_s + b16, v.nx_c + b16, [&](int i) { return __fmul_rn(__fmul_rn(xt[i], scale), __ldg(L.ffn_norm + i)); });
        quant_row(E, v.in_q + (size_t)t * E, v.in_s + b16, v.in_c + b16, [&](int i) { return __fmul_rn(__fmul_rn(xt[i], scale), __ldg(L.pre_ffw2 + i)); });
        if (rows_f)                                             /* the routed experts' input as fp32 rows (expert-parallel dispatch) */
            for (int i = tid; i < E; i += 256) rows_f[(size_t)t * E + i] = __fmul_rn(__fmul_rn(xt[i], scale), __ldg(L.pre_ffw2 + i));
    } else {
        for (int i = tid; i < E; i += 256) {
            const float xs = __fmul_rn(xt[i], scale);
            v.nx_f[(size_t)t * E + i] = __fmul_rn(xs, __ldg(L.ffn_norm + i));
            const float iv = __fmul_rn(xs, __ldg(L.pre_ffw2 + i));
            v.in_f[(size_t)t * E + i] = iv;
            if (rows_f) rows_f[(size_t)t * E + i] = iv;
        }
    }
    for (int i = tid; i < E; i += 256)
        v.rin[(size_t)t * E + i] = __fmul_rn(__fmul_rn(__fmul_rn(xt[i], scale), d.inv_sqrt_e), __ldg(L.router_scale + i));
}

/* ---------------------------------------------------------------- K2: router logits, fp32, fixed order
 * lane l takes the float4 groups q = l, l+32, ... with acc = fma(w, x, acc) over the four
 * elements in order, then the shuffle tree (the same order the decode kernel uses). One block =
 * 32 experts x 16 tokens; E is walked in chunks of 32 float4 groups staged in shared memory, and
 * each warp keeps an 8-expert x 8-token register tile (16 shared-memory loads per 256 FMAs), so every
 * (expert, token) chain keeps the order above while 64 independent chains hide the FMA latency. */
constexpr int kRouterTE = 32, kRouterTT = 16;
constexpr size_t kRouterSmem = 2 * (size_t)(kRouterTE + kRouterTT) * 32 * sizeof(float4);     /* two stages of 24 KB */
/* 16-byte asynchronous copy that writes zeros when `take` is false (the source address stays valid either way) */
__device__ __forceinline__ void cp_async16_zfill(void *smem_dst, const void *src, bool take) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" :: "r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src), "r"(take ? 16 : 0) : "memory");
}
__global__ void __launch_bounds__(256, 2) k_b_router(SpDims d, SpLayerDev L, BView v, int M) {
    extern __shared__ __align__(16) float4 rsm[];              /* [2] x { w[32][32], x[16][32] }: the next chunk lands while this one is used */
    const int E = d.E, G = E >> 2, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int we = warp & 3, wt = warp >> 2;
    const int e0 = blockIdx.x * kRouterTE, t0 = blockIdx.y * kRouterTT;
    float acc[8][8];
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) acc[i][j] = 0.0f;
    auto stage = [&](int c0, int buf) {                         /* warp w stages expert rows w, w+8, w+16, w+24 and token rows w, w+8 */
        float4 *wS = rsm + (size_t)buf * (kRouterTE + kRouterTT) * 32, *xS = wS + kRouterTE * 32;
        const int gg = c0 + lane; const bool gok = gg < G; const int gc = gok ? gg : 0;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int row = warp + 8 * k; const bool ok = gok && e0 + row < d.NE;
            cp_async16_zfill(wS + row * 32 + lane, reinterpret_cast<const float4 *>(L.router_w + (size_t)(ok ? e0 + row : 0) * E) + gc, ok);
        }
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const int row = warp + 8 * k; const bool ok = gok && t0 + row < M;
            cp_async16_zfill(xS + row * 32 + lane, reinterpret_cast<const float4 *>(v.rin + (size_t)(ok ? t0 + row : 0) * E) + gc, ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const int nch = (G + 31) >> 5;
    stage(0, 0);
    for (int c = 0; c < nch; c++) {
        if (c + 1 < nch) { stage(32 * (c + 1), (c + 1) & 1); asm volatile("cp.async.wait_group 1;" ::: "memory"); }
        else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float4 *wS = rsm + (size_t)(c & 1) * (kRouterTE + kRouterTT) * 32, *xS = wS + kRouterTE * 32;
        float4 w[8];                                            /* zero padding beyond E leaves acc unchanged: fma(0, 0, acc) = acc */
#pragma unroll
        for (int i = 0; i < 8; i++) w[i] = wS[(8 * we + i) * 32 + lane];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float4 x = xS[(8 * wt + j) * 32 + lane];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                float a = acc[i][j];
                a = __fmaf_rn(w[i].x, x.x, a); a = __fmaf_rn(w[i].y, x.y, a);
                a = __fmaf_rn(w[i].z, x.z, a); a = __fmaf_rn(w[i].w, x.w, a);
                acc[i][j] = a;
            }
        }
        __syncthreads();                                        /* this stage is overwritten two chunks on */
    }
#pragma unroll
    for (int i = 0; i < 8; i++)
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float r = warp_tree(acc[i][j]);
            const int e = e0 + 8 * we + i, t = t0 + 8 * wt + j;
            if (lane == 0 && e < d.NE && t < M)
                v.logits[(size_t)t * d.NE + e] = L.router_bias ? __fadd_rn(r, __ldg(L.router_bias + e)) : r;
        }
}

/* The same logits for a handful of tokens: one block per (expert, eight tokens), so that a small batch
 * still spreads over the machine (it is bound by the latency of one block's loop, not by arithmetic).
 * The expert's row is staged in shared memory; warp w takes token 8*blockIdx.y + w, lane l the float4
 * groups l, l+32, ... in the order given above. */
__global__ void __launch_bounds__(256) k_b_router_small(SpDims d, SpLayerDev L, BView v, int M) {
    extern __shared__ __align__(16) float4 rw[];               /* [E/4] */
    const int E = d.E, G = E >> 2, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, e = blockIdx.x;
    const float4 *wrow = reinterpret_cast<const float4 *>(L.router_w + (size_t)e * E);
    for (int g = threadIdx.x; g < G; g += 256) rw[g] = __ldg(wrow + g);
    __syncthreads();
    const int t = blockIdx.y * 8 + warp;
    if (t >= M) return;
    const float4 *x = reinterpret_cast<const float4 *>(v.rin + (size_t)t * E);
    float acc = 0.0f;
#pragma unroll 8
    for (int g = lane; g < G; g += 32) {
        const float4 w = rw[g], xv = x[g];
        acc = __fmaf_rn(w.x, xv.x, acc); acc = __fmaf_rn(w.y, xv.y, acc);
        acc = __fmaf_rn(w.z, xv.z, acc); acc = __fmaf_rn(w.w, xv.w, acc);
    }
    const float r = warp_tree(acc);
    if (lane == 0) v.logits[(size_t)t * d.NE + e] = L.router_bias ? __fadd_rn(r, __ldg(L.router_bias + e)) : r;
}
#ifndef SP_ROUTER_SMALL_M
#define SP_ROUTER_SMALL_M 64
#endif
constexpr int kRouterSmallM = SP_ROUTER_SMALL_M;   /* up to this many tokens the per-(expert, eight tokens) blocks beat the tiled kernel */
void launch_router(const SpDims &d, const SpLayerDev &L, BView &v, int M, cudaStream_t st, int *nl) {
    if (M <= kRouterSmallM && (size_t)d.E * 4 <= 48 * 1024) k_b_router_small<<<dim3((unsigned)d.NE, (unsigned)((M + 7) / 8)), 256, (size_t)d.E * 4, st>>>(d, L, v, M);
    else k_b_router<<<dim3((d.NE + kRouterTE - 1) / kRouterTE, (M + kRouterTT - 1) / kRouterTT), 256, kRouterSmem, st>>>(d, L, v, M);
    (*nl)++;
}

/* ---------------------------------------------------------------- K3: moe_topk_host (CF:6220-6240) + bucketing by expert (CF:8594-8624) */
__global__ void __launch_bounds__(256) k_b_topk(SpDims d, SpLayerDev L, BView v, int M, int32_t *sel_out, float *wts_out, int *status) {
    extern __shared__ __align__(16) unsigned char tsm[];
    const int NE = d.NE, NU = d.NU, t = threadIdx.x, tok = blockIdx.x;
    double *ex = reinterpret_cast<double *>(tsm);               /* [NE] */
    float *p = reinterpret_cast<float *>(ex + NE);              /* [NE] */
    __shared__ double red[8];
    __shared__ float wmax[8];
    __shared__ int sel_desc[SP_MAX_NU];
    __shared__ float p_desc[SP_MAX_NU];
    const float *lg = v.logits + (size_t)tok * NE;
    float mx = -INFINITY; int bad = 0;
    for (int i = t; i < NE; i += 256) { const float l = lg[i]; if (l != l) bad = 1; mx = fmaxf(mx, l); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); bad |= __shfl_xor_sync(0xffffffffu, bad, o); }
    if ((t & 31) == 0) wmax[t >> 5] = mx;
    if (bad && (t & 31) == 0) atomicExch(status, SP_KERR_NAN_ROUTER);
    __syncthreads();
    mx = wmax[0];
#pragma unroll
    for (int w = 1; w < 8; w++) mx = fmaxf(mx, wmax[w]);
    double part = 0.0;
    for (int i = t; i < NE; i += 256) { const double e = exp((double)lg[i] - (double)mx); ex[i] = e; part += e; }
    part = warp_sum_f64(part);
    if ((t & 31) == 0) red[t >> 5] = part;
    __syncthreads();
    double sum = 0.0;
#pragma unroll
    for (int w = 0; w < 8; w++) sum += red[w];
    for (int i = t; i < NE; i += 256) p[i] = (float)(ex[i] / sum);
    if (t < SP_MAX_NU) { sel_desc[t] = t < NE ? t : 0; p_desc[t] = 0.0f; }
    __syncthreads();
    for (int i = t; i < NE; i += 256) {
        const float pi = p[i]; int r = 0;
        for (int j = 0; j < NE; j++) { const float pj = p[j]; r += (pj > pi) || (pj == pi && j < i); }
        if (r < NU && pi == pi) { sel_desc[r] = i; p_desc[r] = pi; }
    }
    __syncthreads();
    if (t < NU) {
        float wsum = 0.0f;
        for (int k = 0; k < NU; k++) wsum = __fadd_rn(wsum, p_desc[k]);
        if (wsum < 6.103515625e-5f) wsum = 6.103515625e-5f;
        const int e = sel_desc[t];
        const float w = __fdiv_rn(p_desc[t], wsum);
        int slot = 0;
        for (int j = 0; j < NU; j++) slot += (sel_desc[j] < e);
        const int pair = tok * NU + slot;
        v.sel_asc[pair] = e;
        v.cw[pair] = __fmul_rn(w, __ldg(L.dexps_scale + e));             /* CF:8709 */
        const int pos = atomicAdd(&v.count[e], 1);
        v.pairpos[pair] = pos;
        if (pos < M) v.list[(size_t)e * M + pos] = pair; else atomicExch(status, SP_KERR_OVERFLOW);
        if (sel_out) sel_out[(size_t)tok * NU + t] = e;
        if (wts_out) wts_out[(size_t)tok * NU + t] = w;
    }
}

/* ---------------------------------------------------------------- K5: per-row activation quant (CF:1725-1746) */
__global__ void __launch_bounds__(256) k_b_quant_rows(const float *x, int n, signed char *q, float *sx, int *corr) {
    const size_t r = blockIdx.x;
    const float *xr = x + r * n;
    if (n <= 256 * kPrepK) {                                    /* all of the row's loads first, then the dependent steps */
        float v[kPrepK];
#pragma unroll
        for (int k = 0; k < kPrepK; k++) { const int i = (int)threadIdx.x + 256 * k; v[k] = i < n ? xr[i] : 0.0f; }
#pragma unroll
        for (int k = 0; k < kPrepK; k++)
            if (256 * k < n) {
                const int i = (int)threadIdx.x + 256 * k, b = i >> 4;
                quant_elem16(v[k], i < n, q + r * n + 16 * b, sx + r * (n / 16) + b, corr + r * (n / 16) + b);
            }
        return;
    }
    quant_row(n, q + r * n, sx + r * (n / 16), corr + r * (n / 16), [&](int i) { return xr[i]; });
}

/* ---------------------------------------------------------------- K4/K6: Q4B rows x a list of activations
 * One warp per output row (or gate/up row pair); its codes and block scales are loaded ONCE into
 * registers and reused for every activation in the group's list, so each weight byte is read from
 * HBM once per layer however many tokens share the expert. grid.y = group (expert, or 0 for the
 * shared expert whose list is every token). */
struct GroupArgs {
    const uint8_t *codes; const uint16_t *bs;      /* tensor base */
    long long rows_per_group;                      /* row stride between groups */
    const int *count, *list; int list_stride;      /* per-group lists (NULL list = identity 0..M-1) */
    const int *offset;                             /* or: group g owns items [offset[g], offset[g+1]) (rows sorted by expert) */
    const int *index;                              /* with offset: sorted position -> row in the buffers (NULL = identity) */
    int M, in, rows;                               /* rows (or pairs) per group */
    int up_off;                                    /* PAIR: row offset of the up row */
    const uint8_t *ucodes; const uint16_t *ubs;    /* PAIR with a separate up tensor (shared expert), else NULL */
    int act_div;                                   /* activation row = item / act_div (NU for routed gate|up, 1 otherwise) */
    const int *act_index;                          /* with offset: sorted position -> activation row, when it is not the item's own row (NULL = item / act_div) */
    /* flavour A */
    const signed char *q; const float *sx; const int *corr;
    /* flavour B */
    const float *xf;
    float *out; int out_stride;                    /* out[item * out_stride + row] */
};

template <int NIT>
__device__ __forceinline__ void load_row(const uint8_t *codes, const uint16_t *bs, int n32, int lane, int4 (&w)[NIT], float (&sc)[NIT]) {
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) { w[i] = ld_stream16(codes + 16 * (size_t)c); sc[i] = h2f(ld_stream_u16(bs + c)); }
        else { w[i] = make_int4(0, 0, 0, 0); sc[i] = 0.0f; }
    }
}
template <int NIT>
__device__ __forceinline__ float dot_a(const int4 (&w)[NIT], const float (&sc)[NIT], int n32, int lane,
                                       const int4 *q, const float *sx, const int *corr) {
    float facc = 0.0f;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) {
            const int2 cr = *reinterpret_cast<const int2 *>(corr + 2 * c);
            const float2 s2 = *reinterpret_cast<const float2 *>(sx + 2 * c);
            int a0, a1;
            q4b_chunk_dot(w[i], q[2 * c], q[2 * c + 1], cr.x, cr.y, a0, a1);
            facc = __fmaf_rn(sc[i], __fmaf_rn((float)a0, s2.x, __fmul_rn((float)a1, s2.y)), facc);
        }
    }
    return warp_tree(facc);
}
/* flavour B: w = code * scale exactly (CF:1459-1463), fp32 dot */
template <int NIT>
__device__ __forceinline__ float dot_b(const int4 (&w)[NIT], const float (&sc)[NIT], int n32, int lane, const float *x) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) {
            const float4 *xv = reinterpret_cast<const float4 *>(x + 32 * c);
            const int words[4] = {w[i].x, w[i].y, w[i].z, w[i].w};
            float blk = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const float4 x0 = xv[2 * k], x1 = xv[2 * k + 1];
                const int wd = words[k];
                blk = __fmaf_rn((float)(((wd & 0xF) ^ 8) - 8), x0.x, blk);
                blk = __fmaf_rn((float)((((wd >> 4) & 0xF) ^ 8) - 8), x0.y, blk);
                blk = __fmaf_rn((float)((((wd >> 8) & 0xF) ^ 8) - 8), x0.z, blk);
                blk = __fmaf_rn((float)((((wd >> 12) & 0xF) ^ 8) - 8), x0.w, blk);
                blk = __fmaf_rn((float)((((wd >> 16) & 0xF) ^ 8) - 8), x1.x, blk);
                blk = __fmaf_rn((float)((((wd >> 20) & 0xF) ^ 8) - 8), x1.y, blk);
                blk = __fmaf_rn((float)((((wd >> 24) & 0xF) ^ 8) - 8), x1.z, blk);
                blk = __fmaf_rn((float)((((wd >> 28) & 0xF) ^ 8) - 8), x1.w, blk);
            }
            acc = __fmaf_rn(sc[i], blk, acc);
        }
    }
    return warp_tree(acc);
}

template <bool FA, bool PAIR, int NIT>
__global__ void __launch_bounds__(256) k_b_rows(GroupArgs g) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int grp = blockIdx.y;
    int first = 0, cnt;
    if (g.offset) {                      /* caller-supplied ranges: keep them inside the g.M rows that exist */
        int last = g.offset[grp + 1];
        first = g.offset[grp];
        first = first < 0 ? 0 : (first > g.M ? g.M : first);
        last = last > g.M ? g.M : last;
        cnt = last - first;
    } else cnt = g.count ? g.count[grp] : g.M;
    if (cnt <= 0) return;
    const int r = blockIdx.x * 8 + warp;
    if (r >= g.rows) return;
    const int n32 = g.in >> 5;
    const size_t rb = (size_t)g.in / 2;
    const size_t row = (size_t)grp * g.rows_per_group + r;
    int4 w0[NIT], w1[PAIR ? NIT : 1]; float s0[NIT], s1[PAIR ? NIT : 1];
    load_row<NIT>(g.codes + row * rb, g.bs + row * n32, n32, lane, w0, s0);
    if (PAIR) {
        if (g.ucodes) load_row<NIT>(g.ucodes + row * rb, g.ubs + row * n32, n32, lane, reinterpret_cast<int4(&)[NIT]>(w1), reinterpret_cast<float(&)[NIT]>(s1));
        else load_row<NIT>(g.codes + (row + g.up_off) * rb, g.bs + (row + g.up_off) * n32, n32, lane, reinterpret_cast<int4(&)[NIT]>(w1), reinterpret_cast<float(&)[NIT]>(s1));
    }
    const int *list = g.list ? g.list + (size_t)grp * g.list_stride : nullptr;
    const int b16 = g.in >> 4;
    for (int i = 0; i < cnt; i++) {
        const int item = list ? list[i] : (g.index ? g.index[first + i] : first + i);
        const size_t arow = (size_t)(g.act_index ? g.act_index[first + i] : item / g.act_div);
        float o;
        if (FA) {
            const int4 *q = reinterpret_cast<const int4 *>(g.q + arow * g.in);
            const float *sx = g.sx + arow * b16; const int *corr = g.corr + arow * b16;
            o = dot_a<NIT>(w0, s0, n32, lane, q, sx, corr);
            if (PAIR) o = gelu_mul(o, dot_a<NIT>(reinterpret_cast<int4(&)[NIT]>(w1), reinterpret_cast<float(&)[NIT]>(s1), n32, lane, q, sx, corr));
        } else {
            const float *x = g.xf + arow * g.in;
            o = dot_b<NIT>(w0, s0, n32, lane, x);
            if (PAIR) o = gelu_mul(o, dot_b<NIT>(reinterpret_cast<int4(&)[NIT]>(w1), reinterpret_cast<float(&)[NIT]>(s1), n32, lane, x));
        }
        if (lane == 0) g.out[(size_t)item * g.out_stride + r] = o;
    }
}

/* ---------------------------------------------------------------- K4/K6 on the tensor cores (integer flavour)
 * The same sums as dot_a, bit for bit, with the 16-weight block dots taken by mma.sync m16n8k32
 * (s8 x s8 -> s32) instead of dp4a chains. A warp owns 16 weight rows. Four chunks (4 x 32 weights)
 * go through four MMAs that accumulate into one C tile: the activation operand of MMA i is non-zero
 * only in the column (chunk, half) its k-slots belong to, so column 2q+h of C ends up holding the
 * integer dot of half h of chunk 4j+q, and lane (g, q) of the warp reads the two block sums of
 * "its" chunk for rows g and g+8 straight out of its C registers. Lane (g, q) therefore plays the
 * part that lane (4j+q) % 32 plays in dot_a: it keeps one fp32 accumulator per slot and adds its
 * chunks in ascending order; the 32 slots of a row are then added in the pairing of warp_tree.
 *   A operand: code nibbles moved to the top of a byte (value 16*code as s8, no +8 bias, no
 *              correction term); low nibbles feed k-slots 4q..4q+3, high nibbles 16+4q..16+4q+3.
 *   B operand: the activations' int8 values; the quantiser already stores every 8 of them as
 *              4 even-index then 4 odd-index bytes, which is the order the nibble split needs.
 *   C starts at 0x4B400000 (1.5 * 2^23): the s32 result read as a float is 12582912 + 16*S, and one
 *              fma by 1/16 gives float(S) exactly, without an integer-to-float conversion.
 * KS = warps per 16-row unit: 1 (in <= 768: a warp covers the whole row) or 4 (in <= 3072: warp wq
 * covers slots 8wq..8wq+7 and the slot sums meet in shared memory). */
constexpr int kMmaTB = 4, kMmaG = 6, kMmaPartStride = 33;
constexpr int kMmaMagic = 0x4B400000;

__device__ __forceinline__ void mma_s8(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float magic_to_float(int c) { return __fmaf_rn(__int_as_float(c), 0.0625f, -786432.0f); }
/* the 32 slot sums of one row, added in warp_tree's pairing */
__device__ __forceinline__ float slot_tree(const float *p) {
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = p[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < o; i++) v[i] += v[i + o];
    return v[0];
}

/* shared-memory row stride of the staged codes: the two rows a quarter-warp reads (64 B each) must fall in different banks */
__host__ __device__ constexpr int mma_a_stride(int in) { return in / 2 + ((64 - (in / 2) % 128 + 128) % 128); }
template <int KS>
constexpr size_t mma_smem_bytes(int in) {
    return (size_t)kMmaTB * (in + 16) + (size_t)kMmaTB * (in / 16) * 4 + 16
         + (KS == 4 ? (size_t)2 * kMmaTB * 16 * kMmaPartStride * 4 : (size_t)8 * kMmaTB * 16 * 4)
         + (size_t)(8 / KS) * 16 * mma_a_stride(in);
}
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((unsigned)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
/* D = A*B + {c, c, c, c}: the first MMA of a chain reads its start value from one register */
__device__ __forceinline__ void mma_s8_first(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1, int c) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}

template <bool PAIR, int KS>
__global__ void __launch_bounds__(256, 2) k_b_rows_mma(GroupArgs g) {
    constexpr int TB = kMmaTB, UNITS = 8 / KS, TPC = PAIR ? UNITS / 2 : UNITS, NACC = KS == 4 ? 2 : 8;
    extern __shared__ __align__(16) unsigned char sm[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, q = lane & 3;
    const int grp = blockIdx.y;
    int first = 0, cnt;
    if (g.offset) {
        int last = g.offset[grp + 1];
        first = g.offset[grp];
        first = first < 0 ? 0 : (first > g.M ? g.M : first);
        last = last > g.M ? g.M : last;
        cnt = last - first;
    } else cnt = g.count ? g.count[grp] : g.M;
    if ((int)blockIdx.z * TB >= cnt) return;
    const int in = g.in, n32 = in >> 5, b16 = in >> 4, ngroups = (n32 + 3) >> 2, astride = mma_a_stride(in), pstride = in + 16;
    unsigned char *P = sm;                                      /* [TB][in + 16]: a token's activations as the quantiser stored them, then 16 zero bytes */
    float *sxs = reinterpret_cast<float *>(P + (size_t)TB * pstride);   /* [TB][in/16] activation block scales */
    int *items = reinterpret_cast<int *>(sxs + (size_t)TB * b16);      /* [TB] (+ padding to 16 bytes) */
    float *part = reinterpret_cast<float *>(items + 4);         /* KS=4: [2][TB][16][33] slot sums; KS=1: [8][TB][16] row sums */
    unsigned char *A = reinterpret_cast<unsigned char *>(part + (KS == 4 ? 2 * TB * 16 * kMmaPartStride : 8 * TB * 16));   /* [UNITS][16][astride] codes */
    const size_t rb = (size_t)in / 2;

    /* the block's weight rows go to shared memory once, in one burst: warp w copies rows w, w+8, ... */
    {
        const int ppr = (int)(rb >> 4);
        for (int ur = warp; ur < UNITS * 16; ur += 8) {
            const int u = ur >> 4, r = ur & 15;
            const int tile_u = blockIdx.x * TPC + (PAIR ? u >> 1 : u);
            if (tile_u * 16 < g.rows) {
                const bool up_u = PAIR && (u & 1);
                const size_t row = (size_t)grp * g.rows_per_group + tile_u * 16 + r + (up_u && !g.ucodes ? g.up_off : 0);
                const uint8_t *src = (up_u && g.ucodes ? g.ucodes : g.codes) + row * rb;
                unsigned char *dst = A + (size_t)ur * astride;
                for (int k = lane; k < ppr; k += 32) cp_async16(dst + 16 * k, src + 16 * (size_t)k);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const int unit = warp / KS, wq = warp % KS;
    const int tile = blockIdx.x * TPC + (PAIR ? unit >> 1 : unit);
    const bool up = PAIR && (unit & 1);
    const bool tile_ok = tile * 16 < g.rows;
    const int r0 = tile_ok ? tile * 16 : 0;                     /* a warp past the last tile keeps valid pointers and computes nothing */
    const unsigned char *A0 = A + ((size_t)unit * 16 + gq) * astride, *A1 = A0 + 8 * (size_t)astride;
    float sc[kMmaG][2];                                         /* this lane's block scales: rows gq and gq+8, one chunk per group */
    {
        const size_t row = (size_t)grp * g.rows_per_group + r0 + gq + (up && !g.ucodes ? g.up_off : 0);
        const uint16_t *bs0 = (up && g.ucodes ? g.ubs : g.bs) + row * n32, *bs1 = bs0 + 8 * (size_t)n32;
#pragma unroll
        for (int jj = 0; jj < kMmaG; jj++) {
            const int j = KS == 4 ? 8 * (jj >> 1) + 2 * wq + (jj & 1) : jj;
            const int c = 4 * j + q, cc = c < n32 ? c : n32 - 1;
            sc[jj][0] = h2f(ld_stream_u16(bs0 + cc)); sc[jj][1] = h2f(ld_stream_u16(bs1 + cc));
        }
    }
    const int *list = g.list ? g.list + (size_t)grp * g.list_stride : nullptr;
    const bool bvalid = (gq >> 1) == q;                         /* this lane's k-slots belong to column pair (2q, 2q+1) */
    const int bh = gq & 1;
    if (tid < 4 * TB) reinterpret_cast<int *>(P + (size_t)(tid >> 2) * pstride + in)[tid & 3] = 0;
    const bool vec_sx = (b16 & 3) == 0;                         /* 16-byte copies of the scales need 16-byte rows */

    for (int b0 = blockIdx.z * TB; b0 < cnt; b0 += gridDim.z * TB) {   /* token batches are dealt round-robin over grid.z */
        const int nb = cnt - b0 < TB ? cnt - b0 : TB;
        __syncthreads();                                        /* the previous batch's readers are done */
        /* warps 2t and 2t+1 fetch token t: its int8 row and its block scales */
        {
            const int t = warp >> 1, hw = warp & 1;
            if (t < nb) {
                const int item = list ? list[b0 + t] : (g.index ? g.index[first + b0 + t] : first + b0 + t);
                if (hw == 0 && lane == 0) items[t] = item;
                const size_t arow = (size_t)(g.act_index ? g.act_index[first + b0 + t] : item / g.act_div);
                const signed char *qs = g.q + arow * in;
                unsigned char *pd = P + (size_t)t * pstride;
                for (int k = lane + 32 * hw; k < b16; k += 64) cp_async16(pd + 16 * k, qs + 16 * (size_t)k);
                const float *ss = g.sx + arow * b16;
                if (vec_sx) { for (int k = lane + 32 * hw; k < (b16 >> 2); k += 64) cp_async16(sxs + t * b16 + 4 * k, ss + 4 * k); }
                else { for (int k = lane + 32 * hw; k < b16; k += 64) sxs[t * b16 + k] = ss[k]; }
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();

        if (tile_ok) {
            float acc[TB][NACC][2];
#pragma unroll
            for (int t = 0; t < TB; t++)
#pragma unroll
                for (int a = 0; a < NACC; a++) acc[t][a][0] = acc[t][a][1] = 0.0f;
#pragma unroll
            for (int jj = 0; jj < kMmaG; jj++) {
                const int j = KS == 4 ? 8 * (jj >> 1) + 2 * wq + (jj & 1) : jj;
                if (j < ngroups) {
                    const int ai = KS == 4 ? (jj & 1) : jj;
                    const int c = 4 * j + q;
                    const bool cv = c < n32;
                    const int cc = cv ? c : n32 - 1;                    /* a lane past the row's end reads the last chunk and drops it */
                    uint4 w0 = *reinterpret_cast<const uint4 *>(A0 + 16 * cc), w1 = *reinterpret_cast<const uint4 *>(A1 + 16 * cc);
                    if (!cv) { w0 = make_uint4(0, 0, 0, 0); w1 = w0; }
                    const float s0 = sc[jj][0], s1 = sc[jj][1];
                    const unsigned x0[4] = {w0.x, w0.y, w0.z, w0.w};
                    const unsigned x1[4] = {w1.x, w1.y, w1.z, w1.w};
                    unsigned a[4][4];
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        a[i][0] = (x0[i] << 4) & 0xF0F0F0F0u; a[i][1] = (x1[i] << 4) & 0xF0F0F0F0u;
                        a[i][2] = x0[i] & 0xF0F0F0F0u;        a[i][3] = x1[i] & 0xF0F0F0F0u;
                    }
                    /* a lane whose k-slots are not in column (chunk, half) reads the token's 16 zero bytes */
                    const int off0 = bvalid && cv && bh == 0 ? c * 32 : in, off1 = bvalid && cv && bh == 1 ? c * 32 + 16 : in;
#pragma unroll
                    for (int t = 0; t < TB; t++) {
                        if (t < nb) {
                            const unsigned char *pt = P + (size_t)t * pstride;
                            const uint4 l0 = *reinterpret_cast<const uint4 *>(pt + off0);
                            const uint4 l1 = *reinterpret_cast<const uint4 *>(pt + off1);
                            int ca[4], cb[4];
                            mma_s8_first(ca, a[0][0], a[0][1], a[0][2], a[0][3], l0.x, l0.y, kMmaMagic);
                            mma_s8_first(cb, a[2][0], a[2][1], a[2][2], a[2][3], l1.x, l1.y, kMmaMagic);
                            mma_s8(ca, a[1][0], a[1][1], a[1][2], a[1][3], l0.z, l0.w);
                            mma_s8(cb, a[3][0], a[3][1], a[3][2], a[3][3], l1.z, l1.w);
                            if (cv) {
                                const float2 s2 = *reinterpret_cast<const float2 *>(sxs + t * b16 + 2 * c);
                                acc[t][ai][0] = __fmaf_rn(s0, __fmaf_rn(magic_to_float(ca[0]), s2.x, __fmul_rn(magic_to_float(cb[1]), s2.y)), acc[t][ai][0]);
                                acc[t][ai][1] = __fmaf_rn(s1, __fmaf_rn(magic_to_float(ca[2]), s2.x, __fmul_rn(magic_to_float(cb[3]), s2.y)), acc[t][ai][1]);
                            }
                        }
                    }
                }
            }
            if (KS == 4) {
#pragma unroll
                for (int t = 0; t < TB; t++)
                    if (t < nb)
#pragma unroll
                        for (int a2 = 0; a2 < NACC; a2++)
#pragma unroll
                            for (int r = 0; r < 2; r++)
                                part[((size_t)(unit * TB + t) * 16 + gq + 8 * r) * kMmaPartStride + 8 * wq + 4 * a2 + q] = acc[t][a2][r];
            } else {
#pragma unroll
                for (int t = 0; t < TB; t++)
                    if (t < nb)
#pragma unroll
                        for (int r = 0; r < 2; r++) {
                            float v[8];
#pragma unroll
                            for (int a2 = 0; a2 < 8; a2++) v[a2] = acc[t][a2][r];
#pragma unroll
                            for (int o = 4; o > 0; o >>= 1)
#pragma unroll
                                for (int i = 0; i < o; i++) v[i] += v[i + o];      /* slots s+16, s+8, s+4 sit in this lane */
                            float s = v[0];
                            s += __shfl_down_sync(0xffffffffu, s, 2);
                            s += __shfl_down_sync(0xffffffffu, s, 1);
                            if (q == 0) part[(size_t)(unit * TB + t) * 16 + gq + 8 * r] = s;
                        }
            }
        }
        __syncthreads();
        /* one thread per (unit, token, row); with PAIR the gate thread (even lane) takes the up value from its neighbour */
        {
            const int per = nb * 16 * (PAIR ? 2 : 1);           /* threads per tile */
            for (int w0 = 0; w0 < TPC * per; w0 += 256) {
                const int w = w0 + tid;
                const bool act = w < TPC * per;
                const int tl = act ? w / per : 0, rem = act ? w - tl * per : 0;
                const int half = PAIR ? rem & 1 : 0, tr = PAIR ? rem >> 1 : rem, t = tr >> 4, row = tr & 15;
                const int u = PAIR ? 2 * tl + half : tl;
                float o = 0.0f;
                if (act) o = KS == 4 ? slot_tree(part + ((size_t)(u * TB + t) * 16 + row) * kMmaPartStride) : part[(size_t)(u * TB + t) * 16 + row];
                if (PAIR) { const float other = __shfl_down_sync(0xffffffffu, o, 1); if (half == 0) o = gelu_mul(o, other); }
                const int r = (blockIdx.x * TPC + tl) * 16 + row;
                if (act && half == 0 && r < g.rows) g.out[(size_t)items[t] * g.out_stride + r] = o;
            }
        }
    }
}
/* the staged rows need more than the default 48 KB of shared memory: a per-device setting */
cudaError_t mma_rows_prepare() {
    const int lim = 200 * 1024;
    cudaError_t e = cudaFuncSetAttribute(k_b_rows_mma<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_b_rows_mma<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_b_rows_mma<true, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(k_b_rows_mma<false, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, lim);
    return e;
}

template <bool FA, bool PAIR>
void launch_rows(const GroupArgs &g, int groups, cudaStream_t st, int *nl) {
    if (FA && (g.rows & 15) == 0 && (g.in & 31) == 0 && g.in <= 3072) {
        const int tiles = g.rows / 16;
        /* one group holding every token (the shared expert) spreads its token batches over grid.z; routed
         * groups hold M*NU/groups tokens on average, so two CTAs per tile cover the long lists */
        const int batches = (g.M + kMmaTB - 1) / kMmaTB;
        const unsigned z = (unsigned)(groups == 1 ? (batches < 32 ? batches : 32) : (batches > 2 ? 2 : 1));
        if (g.in <= 768) {
            const int tpc = PAIR ? 4 : 8;
            k_b_rows_mma<PAIR, 1><<<dim3((unsigned)((tiles + tpc - 1) / tpc), (unsigned)groups, z), 256, mma_smem_bytes<1>(g.in), st>>>(g);
        } else {
            const int tpc = PAIR ? 1 : 2;
            k_b_rows_mma<PAIR, 4><<<dim3((unsigned)((tiles + tpc - 1) / tpc), (unsigned)groups, z), 256, mma_smem_bytes<4>(g.in), st>>>(g);
        }
        (*nl)++;
        return;
    }
    const dim3 grid((unsigned)((g.rows + 7) / 8), (unsigned)groups);
    const int nit = ((g.in >> 5) + 31) >> 5;
    if (nit <= 1) k_b_rows<FA, PAIR, 1><<<grid, 256, 0, st>>>(g);
    else if (nit == 2) k_b_rows<FA, PAIR, 2><<<grid, 256, 0, st>>>(g);
    else if (nit == 3) k_b_rows<FA, PAIR, 3><<<grid, 256, 0, st>>>(g);
    else k_b_rows<FA, PAIR, 4><<<grid, 256, 0, st>>>(g);
    (*nl)++;
}

/* ---------------------------------------------------------------- K7: ordered combine + recombine (CF:6071-6077, 9014-9019) */
__global__ void __launch_bounds__(256) k_b_finish(SpDims d, SpLayerDev L, const float *x, BView v, const float *eo, const int *pair_index, float *y) {
    extern __shared__ __align__(16) float fsm[];              /* [2][E] */
    __shared__ double sh[256];
    const int t = blockIdx.x, E = d.E, NU = d.NU, tid = threadIdx.x;
    float cw[SP_MAX_NU]; size_t er[SP_MAX_NU];
#pragma unroll
    for (int k = 0; k < SP_MAX_NU; k++) {
        cw[k] = k < NU ? v.cw[(size_t)t * NU + k] : 0.0f;
        er[k] = k < NU ? (size_t)(pair_index ? pair_index[(size_t)t * NU + k] : t * NU + k) * E : 0;
    }
    float *va = fsm, *vb = fsm + E;
#pragma unroll 4
    for (int i = threadIdx.x; i < E; i += 256) {
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < SP_MAX_NU; k++) if (k < NU) acc = __fadd_rn(acc, __fmul_rn(cw[k], eo[er[k] + i]));
        vb[i] = acc;
        va[i] = v.dn[(size_t)t * E + i];
    }
    __syncthreads();
    const float sc1 = rms_scale_from(sumsq256(va, E, sh), E, d.eps);
    const float sc2 = rms_scale_from(sumsq256(vb, E, sh), E, d.eps);
    for (int i = threadIdx.x; i < E; i += 256) {
        const float mlp = __fmul_rn(__fmul_rn(va[i], sc1), __ldg(L.post_ffw1 + i));
        const float t1 = __fmul_rn(__fmul_rn(vb[i], sc2), __ldg(L.post_ffw2 + i));
        va[i] = __fadd_rn(mlp, t1);
    }
    __syncthreads();
    const float sc3 = rms_scale_from(sumsq256(va, E, sh), E, d.eps);
    for (int i = threadIdx.x; i < E; i += 256)
        y[(size_t)t * E + i] = __fadd_rn(x[(size_t)t * E + i], __fmul_rn(__fmul_rn(va[i], sc3), __ldg(L.post_ffw + i)));
}

static size_t finish_smem(int E) { return (size_t)2 * E * 4; }

template <bool FA>
cudaError_t run_layer(const SpDims &d, const SpLayerDev &L, int M, const float *x, float *y, int32_t *sel, float *wts,
                      BView &v, SpTcPlan *tc, int *status, cudaStream_t st, int *nl) {
    const int E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;
    k_b_prep<FA><<<M, 256, 0, st>>>(d, L, x, v, nullptr); (*nl)++;
    launch_router(d, L, v, M, st, nl);
    k_b_topk<<<M, 256, (size_t)NE * 12, st>>>(d, L, v, M, sel, wts, status); (*nl)++;
    if (!FA && tc) {                                            /* prefill arithmetic on the tensor cores */
        cudaError_t e = sp_tc_shared_expert(tc, d, L, M, v.nx_f, v.dn, status, st, nl);
        if (e != cudaSuccess) return e;
        const int *off, *gather, *rowmap;
        e = sp_tc_sort_pairs(tc, d, M, v.sel_asc, v.count, v.pairpos, &off, &gather, &rowmap, st, nl);
        if (e != cudaSuccess) return e;
        e = sp_tc_routed(tc, d, L, M * NU, v.in_f, gather, off, rowmap, v.eo, status, st, nl);
        if (e != cudaSuccess) return e;
        k_b_finish<<<M, 256, finish_smem(E), st>>>(d, L, x, v, v.eo, nullptr, y); (*nl)++;
        return cudaGetLastError();
    }
    GroupArgs g{};
    g.M = M;
    /* shared expert gate/up -> hd (CF:8348-8356) */
    g.codes = L.sg_codes; g.bs = L.sg_bs; g.ucodes = L.su_codes; g.ubs = L.su_bs; g.rows_per_group = 0; g.count = nullptr; g.list = nullptr;
    g.in = E; g.rows = FFS; g.up_off = 0; g.act_div = 1; g.q = v.nx_q; g.sx = v.nx_s; g.corr = v.nx_c; g.xf = v.nx_f; g.out = v.hd; g.out_stride = FFS;
    launch_rows<FA, true>(g, 1, st, nl);
    /* routed gate|up -> h (CF:8733-8737, 8958-8959) */
    g.codes = L.gu_codes; g.bs = L.gu_bs; g.ucodes = nullptr; g.ubs = nullptr; g.rows_per_group = 2LL * FFE; g.count = v.count; g.list = v.list; g.list_stride = M;
    g.in = E; g.rows = FFE; g.up_off = FFE; g.act_div = NU; g.q = v.in_q; g.sx = v.in_s; g.corr = v.in_c; g.xf = v.in_f; g.out = v.h; g.out_stride = FFE;
    launch_rows<FA, true>(g, NE, st, nl);
    if (FA) {
        k_b_quant_rows<<<M, 256, 0, st>>>(v.hd, FFS, v.hd_q, v.hd_s, v.hd_c); (*nl)++;
        k_b_quant_rows<<<M * NU, 256, 0, st>>>(v.h, FFE, v.h_q, v.h_s, v.h_c); (*nl)++;
    }
    /* shared down -> dn (CF:8358) */
    g.codes = L.sd_codes; g.bs = L.sd_bs; g.rows_per_group = 0; g.count = nullptr; g.list = nullptr;
    g.in = FFS; g.rows = E; g.act_div = 1; g.q = v.hd_q; g.sx = v.hd_s; g.corr = v.hd_c; g.xf = v.hd; g.out = v.dn; g.out_stride = E;
    launch_rows<FA, false>(g, 1, st, nl);
    /* routed down -> eo (CF:8739-8742, 8961) */
    g.codes = L.dn_codes; g.bs = L.dn_bs; g.rows_per_group = E; g.count = v.count; g.list = v.list; g.list_stride = M;
    g.in = FFE; g.rows = E; g.act_div = 1; g.q = v.h_q; g.sx = v.h_s; g.corr = v.h_c; g.xf = v.h; g.out = v.eo; g.out_stride = E;
    launch_rows<FA, false>(g, NE, st, nl);
    k_b_finish<<<M, 256, finish_smem(E), st>>>(d, L, x, v, v.eo, nullptr, y); (*nl)++;
    return cudaGetLastError();
}

/* per-expert counts -> exclusive offsets (NE is at most 1024: one block) */
__global__ void __launch_bounds__(1024) k_b_scan(const int *count, int n, int *off) {
    __shared__ int sh[1024];
    const int t = threadIdx.x;
    sh[t] = t < n ? count[t] : 0;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) { const int v = t >= d ? sh[t - d] : 0; __syncthreads(); sh[t] += v; __syncthreads(); }
    if (t < n) off[t + 1] = sh[t];
    if (t == 0) off[0] = 0;
}
/* one block per (token, expert) pair: its input row goes to position off[e] + pairpos of the send buffer.
 * With a capacity (rows per destination rank, experts owned in blocks of epr) the buffer is padded: the rows
 * for rank r start at r * capacity, so the exchange needs no split sizes; a block that would not fit is
 * reported through the error word. */
__global__ void __launch_bounds__(256) k_b_dispatch_rows(const float *in_f, const int *sel_asc, const int *pairpos, const int *off, int NU, int E,
                                                         int epr, int capacity, float *rows, int *pair_index, int *status) {
    const int p = blockIdx.x;
    const int e = sel_asc[p];
    int pos = off[e] + pairpos[p];
    if (capacity > 0) {
        const int owner = e / epr, in_block = pos - off[owner * epr];
        if (in_block >= capacity) {
            if (threadIdx.x == 0) { pair_index[p] = owner * capacity; atomicExch(status, SP_KERR_OVERFLOW); }
            return;
        }
        pos = owner * capacity + in_block;
    }
    if (threadIdx.x == 0) pair_index[p] = pos;
    if (!rows) return;                           /* positions only: the caller sends token rows instead of pair rows */
    const float4 *src = reinterpret_cast<const float4 *>(in_f + (size_t)(p / NU) * E);
    float4 *dst = reinterpret_cast<float4 *>(rows + (size_t)pos * E);
    for (int i = threadIdx.x; i < E / 4; i += 256) dst[i] = src[i];
}
/* ---- token dispatch: a token's input row goes to a destination rank once, however many of its NU experts live
 * there. Per destination r: the tokens with at least one expert on r, in token order (slot = rank among them), up to
 * cap_tokens rows; per pair (at its position in the padded pair order, pair_index) the slot of its token. The receiver
 * multiplies row  source * cap_tokens + slot  for the pair. */
__global__ void __launch_bounds__(1024) k_b_tok_scan(const int *sel_asc, int M, int NU, int epr, int n_ranks, int cap_tokens, int *slot, int *status) {
    __shared__ int wsum[32];
    __shared__ int carry;
    const int r = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    if (t == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < M; base += 1024) {
        const int tok = base + t;
        int flag = 0;
        if (tok < M) for (int k = 0; k < NU; k++) flag |= (sel_asc[tok * NU + k] / epr == r);
        const unsigned bal = __ballot_sync(0xffffffffu, flag);
        const int within = __popc(bal & ((1u << lane) - 1u));
        if (lane == 0) wsum[warp] = __popc(bal);
        __syncthreads();
        int before = carry;
        for (int w = 0; w < warp; w++) before += wsum[w];
        if (tok < M) {
            const int sl = before + within;
            slot[tok * n_ranks + r] = flag ? sl : -1;
            if (flag && sl >= cap_tokens) atomicExch(status, SP_KERR_OVERFLOW);
        }
        __syncthreads();
        if (t == 0) { int tot = 0; for (int w = 0; w < 32; w++) tot += wsum[w]; carry += tot; }
        __syncthreads();
    }
}
__global__ void __launch_bounds__(256) k_b_tok_rows(const float *in_f, const int *slot, int n_ranks, int cap_tokens, int E, float *tokrows) {
    const int tok = blockIdx.x, r = blockIdx.y;
    const int sl = slot[tok * n_ranks + r];
    if (sl < 0 || sl >= cap_tokens) return;
    const float4 *src = reinterpret_cast<const float4 *>(in_f + (size_t)tok * E);
    float4 *dst = reinterpret_cast<float4 *>(tokrows + ((size_t)r * cap_tokens + sl) * E);
    for (int i = threadIdx.x; i < E / 4; i += 256) dst[i] = src[i];
}
__global__ void __launch_bounds__(256) k_b_tok_idx(const int *sel_asc, const int *pair_index, const int *slot, int np, int NU, int epr, int n_ranks, int cap_tokens, int *tokidx) {
    const int p = blockIdx.x * 256 + threadIdx.x;
    if (p >= np) return;
    const int r = sel_asc[p] / epr;
    int sl = slot[(p / NU) * n_ranks + r];
    sl = sl < 0 ? 0 : (sl >= cap_tokens ? cap_tokens - 1 : sl);
    tokidx[pair_index[p]] = sl;
}
/* receiver: sorted position p -> the row of the pair's token among the token rows that arrived */
__global__ void __launch_bounds__(256) k_b_in_index(const int *row_index, const int *tokidx_recv, int n, int capacity, int cap_tokens, int n_ranks, int *in_index) {
    const int p = blockIdx.x * 256 + threadIdx.x;
    if (p >= n) return;
    const int a = row_index[p];                              /* arrival slot of the pair: source * capacity + position in the source's block */
    const int src = a / capacity;
    int sl = tokidx_recv[a];
    sl = sl < 0 ? 0 : (sl >= cap_tokens ? cap_tokens - 1 : sl);
    in_index[p] = (src < n_ranks ? src : n_ranks - 1) * cap_tokens + sl;
}
/* what a rank received through the padded exchange: source s's block starts at row s * capacity and holds
 * its rows for this rank's experts, sorted by expert. counts_all[s][e] = pairs of expert e on rank s.
 * Writes offsets[NE+1] (sorted position range of every expert; empty outside this rank's experts) and
 * row_index[n_ranks * capacity] (sorted position -> arrival row; 0 beyond the rows that exist). */
__global__ void __launch_bounds__(256) k_b_recv_layout(const int *counts_all, int NE, int n_ranks, int rank, int capacity, int *offsets, int *row_index) {
    extern __shared__ int lsm[];                 /* cnt[nb], sorted_start[nb + 1], arrival_start[nb], all in (expert, source) order */
    const int epr = NE / n_ranks, nb = epr * n_ranks, e0 = rank * epr;
    int *cnt = lsm, *sorted_start = lsm + nb, *arrival_start = lsm + 2 * nb + 1;
    for (int b = threadIdx.x; b < nb; b += 256) cnt[b] = counts_all[(b % n_ranks) * NE + e0 + b / n_ranks];
    __syncthreads();
    /* A source whose block for this rank overflowed kept only its first `capacity` rows, in expert order
     * (k_b_dispatch_rows drops the rest and sets the error word) but still reports its full counts: clamp
     * each source's running total to the capacity, so every index below stays inside the receive buffer. */
    for (int s_ = threadIdx.x; s_ < n_ranks; s_ += 256) {
        int a = 0;
        for (int e = 0; e < epr; e++) {
            int c = cnt[e * n_ranks + s_];
            c = c < 0 ? 0 : c;
            if (c > capacity - a) c = capacity - a;
            cnt[e * n_ranks + s_] = c;
            arrival_start[e * n_ranks + s_] = s_ * capacity + a;
            a += c;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int acc = 0;
        for (int b = 0; b < nb; b++) { sorted_start[b] = acc; acc += cnt[b]; }
        sorted_start[nb] = acc;
    }
    __syncthreads();
    const int total = sorted_start[nb];
    for (int e = threadIdx.x; e <= NE; e += 256)
        offsets[e] = e < e0 ? 0 : (e >= e0 + epr ? total : sorted_start[(e - e0) * n_ranks]);
    for (int p = threadIdx.x; p < n_ranks * capacity; p += 256) {
        int v = 0;
        if (p < total) {
            int lo = 0, hi = nb - 1;               /* the block that holds sorted position p */
            while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (sorted_start[mid] <= p) lo = mid; else hi = mid - 1; }
            v = arrival_start[lo] + (p - sorted_start[lo]);
        }
        row_index[p] = v;
    }
}

/* ---------------------------------------------------------------- expert-parallel stages
 * The layer cut at the two places where (token, expert) pairs change GPU:
 *   route   : norms, router, top-k, the shared expert (kept in this handle's scratch), and the
 *             routed experts' input rows;
 *   experts : gate|up GeGLU + down for rows that arrive sorted by expert, on whichever GPU owns
 *             those experts (any subset: empty groups cost nothing);
 *   finish  : ordered combine of the returned pair rows + the recombine.
 * The arithmetic of each pair is the single-GPU batched path's, so a split run is bit-identical. */
/* the shared (always-on) expert of the tokens the last route call prepared: nx -> dn in the scratch */
/* phase 0 = the whole shared expert; 1 = gate/up + GeGLU only (hd stays in the scratch); 2 = the down rows only */
template <bool FA>
cudaError_t ep_shared(const SpDims &d, const SpLayerDev &L, int M, BView &v, SpTcPlan *tc, int *status, cudaStream_t st, int *nl, int phase) {
    const int E = d.E, FFS = d.FFS;
    if (!FA && tc) return sp_tc_shared_expert(tc, d, L, M, v.nx_f, v.dn, status, st, nl, phase);
    GroupArgs g{};
    g.M = M; g.act_div = 1;
    if (phase != 2) {
        g.codes = L.sg_codes; g.bs = L.sg_bs; g.ucodes = L.su_codes; g.ubs = L.su_bs;
        g.in = E; g.rows = FFS; g.q = v.nx_q; g.sx = v.nx_s; g.corr = v.nx_c; g.xf = v.nx_f; g.out = v.hd; g.out_stride = FFS;
        launch_rows<FA, true>(g, 1, st, nl);
        if (FA) { k_b_quant_rows<<<M, 256, 0, st>>>(v.hd, FFS, v.hd_q, v.hd_s, v.hd_c); (*nl)++; }
    }
    if (phase != 1) {
        g.codes = L.sd_codes; g.bs = L.sd_bs; g.ucodes = nullptr; g.ubs = nullptr;
        g.in = FFS; g.rows = E; g.q = v.hd_q; g.sx = v.hd_s; g.corr = v.hd_c; g.xf = v.hd; g.out = v.dn; g.out_stride = E;
        launch_rows<FA, false>(g, 1, st, nl);
    }
    return cudaGetLastError();
}

template <bool FA>
cudaError_t ep_route(const SpDims &d, const SpLayerDev &L, int M, const float *x, int32_t *sel_asc, float *cw, float *rows, int32_t *counts,
                     int32_t *pair_index, int32_t *sel, float *wts, int defer_shared, int n_ranks, int capacity, BView &v, SpTcPlan *tc, int *status,
                     cudaStream_t st, int *nl) {
    const int E = d.E, NE = d.NE, NU = d.NU;
    k_b_prep<FA><<<M, 256, 0, st>>>(d, L, x, v, FA ? v.in_f : nullptr); (*nl)++;
    cudaError_t e = cudaSuccess;
    launch_router(d, L, v, M, st, nl);
    k_b_topk<<<M, 256, (size_t)NE * 12, st>>>(d, L, v, M, sel, wts, status); (*nl)++;
    /* the send buffer: rows sorted by expert (so also by owner), ready for the all-to-all */
    k_b_scan<<<1, 1024, 0, st>>>(v.count, NE, v.ep_off); (*nl)++;
    k_b_dispatch_rows<<<M * NU, 256, 0, st>>>(v.in_f, v.sel_asc, v.pairpos, v.ep_off, NU, E, capacity > 0 ? NE / n_ranks : NE, capacity, rows, pair_index, status); (*nl)++;
    e = cudaMemcpyAsync(counts, v.count, (size_t)4 * NE, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return e;
    e = cudaMemcpyAsync(sel_asc, v.sel_asc, (size_t)4 * M * NU, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return e;
    e = cudaMemcpyAsync(cw, v.cw, (size_t)4 * M * NU, cudaMemcpyDeviceToDevice, st);
    if (e != cudaSuccess) return e;
    if (defer_shared) return cudaGetLastError();
    return ep_shared<FA>(d, L, M, v, tc, status, st, nl, 0);
}

/* in_index (optional, with n_in input rows): sorted position -> input row, when several pairs share one input row
 * (token dispatch); the outputs still go to the pair's own row (row_index). */
template <bool FA>
cudaError_t ep_experts(const SpDims &d, const SpLayerDev &L, int R, const float *rows_in, const int32_t *row_index, const int32_t *offsets, float *rows_out,
                       const int32_t *in_index, int n_in, BView &v, SpTcPlan *tc, int *status, cudaStream_t st, int *nl) {
    const int E = d.E, NE = d.NE, FFE = d.FFE;
    if (R == 0) return cudaSuccess;
    if (!FA && tc) return sp_tc_routed(tc, d, L, R, rows_in, in_index ? in_index : row_index, offsets, row_index, rows_out, status, st, nl);
    if (FA) { k_b_quant_rows<<<in_index ? n_in : R, 256, 0, st>>>(rows_in, E, v.ep_q, v.ep_s, v.ep_c); (*nl)++; }
    GroupArgs g{};
    g.M = R; g.offset = offsets; g.index = row_index; g.act_index = in_index;
    g.codes = L.gu_codes; g.bs = L.gu_bs; g.rows_per_group = 2LL * FFE;
    g.in = E; g.rows = FFE; g.up_off = FFE; g.act_div = 1; g.q = v.ep_q; g.sx = v.ep_s; g.corr = v.ep_c; g.xf = rows_in; g.out = v.h; g.out_stride = FFE;
    launch_rows<FA, true>(g, NE, st, nl);
    if (FA) { k_b_quant_rows<<<R, 256, 0, st>>>(v.h, FFE, v.h_q, v.h_s, v.h_c); (*nl)++; }
    g.codes = L.dn_codes; g.bs = L.dn_bs; g.rows_per_group = E; g.act_index = nullptr;          /* h has one row per pair */
    g.in = FFE; g.rows = E; g.q = v.h_q; g.sx = v.h_s; g.corr = v.h_c; g.xf = v.h; g.out = rows_out; g.out_stride = E;
    launch_rows<FA, false>(g, NE, st, nl);
    return cudaGetLastError();
}

}  // namespace

cudaError_t sp_batched_ep_route(const SpDims &d, const SpLayerDev &L, int flavour, int M, const float *x, int32_t *sel_asc, float *cw,
                                float *rows, int32_t *counts, int32_t *pair_index, int32_t *sel, float *wts, int defer_shared, int n_ranks, int capacity,
                                SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch, int t0, int slice) {
    *nlaunch = 0;
    if (!s->base || t0 < 0 || t0 + M > s->max_tokens || slice < 0 || slice >= kSlices) return cudaErrorInvalidValue;
    BView v = bview_slice(d, s, t0, slice);
    return flavour == SP_MOE_FLAVOUR_DECODE ? ep_route<true>(d, L, M, x, sel_asc, cw, rows, counts, pair_index, sel, wts, defer_shared, n_ranks, capacity, v, s->tc, status, st, nlaunch)
                                            : ep_route<false>(d, L, M, x, sel_asc, cw, rows, counts, pair_index, sel, wts, defer_shared, n_ranks, capacity, v, s->tc, status, st, nlaunch);
}
cudaError_t sp_batched_ep_recv_layout(const SpDims &d, const int32_t *counts_all, int n_ranks, int rank, int capacity, int32_t *offsets, int32_t *row_index,
                                      cudaStream_t st, int *nlaunch) {
    *nlaunch = 1;
    const int nb = d.NE;                                    /* epr * n_ranks */
    k_b_recv_layout<<<1, 256, (size_t)(3 * nb + 1) * sizeof(int), st>>>(counts_all, d.NE, n_ranks, rank, capacity, offsets, row_index);
    return cudaGetLastError();
}
cudaError_t sp_batched_ep_shared(const SpDims &d, const SpLayerDev &L, int flavour, int M, SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch, int t0, int slice, int phase) {
    *nlaunch = 0;
    if (!s->base || t0 < 0 || t0 + M > s->max_tokens || slice < 0 || slice >= kSlices || phase < 0 || phase > 2) return cudaErrorInvalidValue;
    BView v = bview_slice(d, s, t0, slice);
    return flavour == SP_MOE_FLAVOUR_DECODE ? ep_shared<true>(d, L, M, v, s->tc, status, st, nlaunch, phase) : ep_shared<false>(d, L, M, v, s->tc, status, st, nlaunch, phase);
}
cudaError_t sp_batched_ep_experts(const SpDims &d, const SpLayerDev &L, int flavour, int R, const float *rows_in, const int32_t *row_index, const int32_t *offsets,
                                  float *rows_out, SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch, const int32_t *in_index, int n_in) {
    *nlaunch = 0;
    if (!s->base || R > s->max_rows || (in_index && (n_in <= 0 || n_in > s->max_rows))) return cudaErrorInvalidValue;
    BView v = bview(d, s);
    return flavour == SP_MOE_FLAVOUR_DECODE ? ep_experts<true>(d, L, R, rows_in, row_index, offsets, rows_out, in_index, n_in, v, s->tc, status, st, nlaunch)
                                            : ep_experts<false>(d, L, R, rows_in, row_index, offsets, rows_out, in_index, n_in, v, s->tc, status, st, nlaunch);
}
/* token dispatch, sender side (after sp_batched_ep_route of the same tokens with rows == NULL): tokrows
 * [n_ranks][cap_tokens][E], tokidx [n_ranks][capacity] (the pair order of the padded exchange), slot = scratch of
 * M * n_ranks ints */
cudaError_t sp_batched_ep_tokens(const SpDims &d, int M, int n_ranks, int capacity, int cap_tokens, const int32_t *sel_asc, const int32_t *pair_index,
                                 float *tokrows, int32_t *tokidx, int32_t *slot, SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch, int t0, int slice) {
    *nlaunch = 0;
    if (!s->base || t0 < 0 || t0 + M > s->max_tokens || slice < 0 || slice >= kSlices || n_ranks <= 0 || d.NE % n_ranks || capacity <= 0 || cap_tokens <= 0) return cudaErrorInvalidValue;
    BView v = bview_slice(d, s, t0, slice);
    const int epr = d.NE / n_ranks;
    k_b_tok_scan<<<n_ranks, 1024, 0, st>>>(sel_asc, M, d.NU, epr, n_ranks, cap_tokens, slot, status); (*nlaunch)++;
    k_b_tok_rows<<<dim3((unsigned)M, (unsigned)n_ranks), 256, 0, st>>>(v.in_f, slot, n_ranks, cap_tokens, d.E, tokrows); (*nlaunch)++;
    k_b_tok_idx<<<(M * d.NU + 255) / 256, 256, 0, st>>>(sel_asc, pair_index, slot, M * d.NU, d.NU, epr, n_ranks, cap_tokens, tokidx); (*nlaunch)++;
    return cudaGetLastError();
}
/* token dispatch, receiver side (after sp_batched_ep_recv_layout): in_index[n_ranks * capacity] */
cudaError_t sp_batched_ep_in_index(const int32_t *row_index, const int32_t *tokidx_recv, int n_ranks, int capacity, int cap_tokens, int32_t *in_index,
                                   cudaStream_t st, int *nlaunch) {
    *nlaunch = 1;
    const int n = n_ranks * capacity;
    k_b_in_index<<<(n + 255) / 256, 256, 0, st>>>(row_index, tokidx_recv, n, capacity, cap_tokens, n_ranks, in_index);
    return cudaGetLastError();
}
cudaError_t sp_batched_ep_finish(const SpDims &d, const SpLayerDev &L, int M, const float *x, const float *pair_rows, const int32_t *pair_index, float *y,
                                 SpBatchedScratch *s, cudaStream_t st, int *nlaunch, int t0, int slice) {
    *nlaunch = 0;
    if (!s->base || t0 < 0 || t0 + M > s->max_tokens || slice < 0 || slice >= kSlices) return cudaErrorInvalidValue;
    BView v = bview_slice(d, s, t0, slice);
    k_b_finish<<<M, 256, finish_smem(d.E), st>>>(d, L, x, v, pair_rows, pair_index, y); (*nlaunch)++;
    return cudaGetLastError();
}

cudaError_t sp_batched_alloc(const SpDims &d, int max_tokens, int max_rows, SpBatchedScratch *s, size_t *bytes) {
    s->base = nullptr; s->bytes = 0; s->max_tokens = max_tokens; *bytes = 0;
    s->max_rows = max_rows > max_tokens * d.NU ? max_rows : max_tokens * d.NU;
    s->bytes = blayout(d, max_tokens, s->max_rows, [](int, size_t) {});
    s->tc = nullptr;
    cudaError_t e = mma_rows_prepare();
    if (e != cudaSuccess) return e;
    e = cudaMalloc(&s->base, s->bytes);
    if (e != cudaSuccess) { s->base = nullptr; return e; }
    *bytes = s->bytes;
    /* house convention: behaviour switches are SP_* variables read once. "simt" keeps prefill on the fp32 CUDA-core kernels. */
    const char *ev = getenv("SP_MOE_PREFILL_IMPL");
    if (max_tokens > 1 && sp_tc_supported(d) && !(ev && ev[0] == 's')) {
        size_t tb = 0;
        e = sp_tc_create(d, max_tokens, s->max_rows, &s->tc, &tb);
        if (e != cudaSuccess) { cudaFree(s->base); s->base = nullptr; return e; }
        *bytes += tb;
    }
    return cudaSuccess;
}
void sp_batched_free(SpBatchedScratch *s) {
    if (!s) return;
    if (s->tc) { sp_tc_destroy(s->tc); s->tc = nullptr; }
    if (s->base) cudaFree(s->base);
    s->base = nullptr;
}

cudaError_t sp_batched_forward(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl_, int flavour, int M,
                               const float *x, float *y, int32_t *sel, float *wts,
                               SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch) {
    *nlaunch = 0;
    if (!s->base || M > s->max_tokens) return cudaErrorInvalidValue;
    BView v = bview(d, s);
    const float *cur = x;
    for (int li = 0; li < nl_; li++) {
        float *dst = (li == nl_ - 1) ? y : ((li & 1) ? v.xb : v.xa);
        int32_t *sl = sel ? sel + (size_t)li * M * d.NU : nullptr;
        float *wl = wts ? wts + (size_t)li * M * d.NU : nullptr;
        const cudaError_t e = (flavour == SP_MOE_FLAVOUR_DECODE)
            ? run_layer<true>(d, layers_host[lf + li], M, cur, dst, sl, wl, v, s->tc, status, st, nlaunch)
            : run_layer<false>(d, layers_host[lf + li], M, cur, dst, sl, wl, v, s->tc, status, st, nlaunch);
        if (e != cudaSuccess) return e;
        cur = dst;
    }
    return cudaSuccess;
}
