/* decode_graph.cu — the M=1 decode path as three kernels per layer, replayed from a CUDA graph,
 * weight rows read by the warps straight from global memory. Works for every geometry the handle
 * accepts; decode_staged.cu is the faster form for geometries whose per-CTA slices fit shared
 * memory.
 *
 * Replaces, for n_tok == 1, the ~20 launches + one host round trip per layer of g4_ffn_apply
 * (CF:8314-9050 of src/backends/cuda/cuda_forward.cu): k_rmsnorm, gemv_w_packed x3 (shared
 * expert), k_gelu_mul, k_moe_router_prep, router SGEMM, D2H + moe_topk_host, k_quant_act_int8,
 * k_gemv_q4b_dp4a_grp x2, k_moe_gelu_split_batch, k_moe_combine_ord and the recombine norms.
 * The layer is cut at the three points where every CTA needs every other CTA's results, so the
 * kernel boundary is the grid-wide exchange:
 *
 *   K1  [recombine of the previous layer] -> norms of x, int8 quantisation, router input
 *       router rows (fp32) + shared-expert gate/up row pairs            -> logits, hd
 *   K2  softmax/top-NU/renorm, quantise hd
 *       shared-expert down rows + routed gate|up row pairs              -> dn, h
 *   K3  quantise h
 *       routed down rows, ordered combine (ascending expert id)         -> acc
 *   KF  recombine of the last layer                                      -> y
 *
 * Every CTA repeats the small per-layer prologue (norms, top-k, quantisation) for itself; only
 * the weight rows are partitioned. Later kernels are launched with programmatic dependent launch
 * so their CTAs are resident and have their first weight rows in flight before the previous
 * kernel has drained.
 */
#include "common.cuh"
#include "decode.cuh"


namespace {

constexpr int kT = 512;                 /* threads per CTA */
constexpr int kW = kT / 32;

struct GArgs {
    SpLayerDev L;
    SpDims d;
    const float *x_prev;      /* residual entering this layer (K1: before the previous layer's recombine is added) */
    float *x_cur;             /* K1 writes the residual entering this layer (CTA 0) */
    SpGraphScratch s;
    int32_t *sel_out; float *wts_out;
    int first;                /* K1: no previous layer to recombine */
    SpLayerDev Ln;            /* the next layer (K3 asks L2 for its routing-independent rows) */
    int has_next;
};

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

/* sum over the CTA in double: shuffle tree per warp, warp totals in order */
__device__ __forceinline__ double cta_sum(double v, double *sh) {
    v = warp_sum_f64(v);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int w = 0; w < kW; w++) r += sh[w];
    __syncthreads();
    return r;
}
__device__ __forceinline__ float rms_scale(double ss, double inv_n, float eps) {
    const float ms = (float)(ss * inv_n);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
}
__device__ __forceinline__ float warp_tree(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}
struct ActS { const int4 *q; const float *sx; const int *corr; };
/* ask L2 for [p, p+bytes): one 128-byte line per lane per instruction. The row loops below then
 * find their weights in L2 instead of paying an HBM round trip per row. */
__device__ __forceinline__ void l2_prefetch(const void *p, int bytes, int lane) {
    const unsigned char *b = reinterpret_cast<const unsigned char *>(p);
    for (int off = lane * 128; off < bytes; off += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(b + off));
}

template <int NIT>
__device__ __forceinline__ void row_load(const uint8_t *codes, const uint16_t *bs, int n32, int lane, int4 (&w)[NIT], unsigned short (&sc)[NIT]) {
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) { w[i] = ld_stream16(codes + 16 * (size_t)c); sc[i] = ld_stream_u16(bs + c); }
    }
}
template <int NIT>
__device__ __forceinline__ float row_fma(const int4 (&w)[NIT], const unsigned short (&sc)[NIT], int n32, int lane, const ActS &a) {
    float facc = 0.0f;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) {
            int a0, a1;
            const int2 corr = *reinterpret_cast<const int2 *>(a.corr + 2 * c);
            const float2 sx = *reinterpret_cast<const float2 *>(a.sx + 2 * c);
            q4b_chunk_dot(w[i], a.q[2 * c], a.q[2 * c + 1], corr.x, corr.y, a0, a1);
            facc = __fmaf_rn(h2f(sc[i]), __fmaf_rn((float)a0, sx.x, __fmul_rn((float)a1, sx.y)), facc);
        }
    }
    return warp_tree(facc);
}
#define NIT_SWITCH(n32, ...)                                     \
    do { const int nit_ = ((n32) + 31) >> 5;                     \
         if (nit_ <= 1) { constexpr int NIT = 1; __VA_ARGS__; }         \
         else if (nit_ == 2) { constexpr int NIT = 2; __VA_ARGS__; }    \
         else if (nit_ == 3) { constexpr int NIT = 3; __VA_ARGS__; }    \
         else { constexpr int NIT = 4; __VA_ARGS__; } } while (0)

template <int NIT>
__device__ __forceinline__ float one_row(const uint8_t *c, const uint16_t *s, int n32, int lane, const ActS &a) {
    int4 w[NIT]; unsigned short sc[NIT];
    row_load<NIT>(c, s, n32, lane, w, sc);
    return row_fma<NIT>(w, sc, n32, lane, a);
}

template <int NIT>
__device__ __forceinline__ float pair_gelu(const uint8_t *gc, const uint16_t *gs, const uint8_t *uc, const uint16_t *us, int n32, int lane, const ActS &a) {
    int4 wg[NIT], wu[NIT]; unsigned short sg[NIT], su[NIT];
    row_load<NIT>(gc, gs, n32, lane, wg, sg);
    row_load<NIT>(uc, us, n32, lane, wu, su);
    const float g = row_fma<NIT>(wg, sg, n32, lane, a);
    const float u = row_fma<NIT>(wu, su, n32, lane, a);
    return gelu_mul(g, u);
}
/* quantise n floats (read through get) into shared memory, one thread per 16-block */
template <class F>
__device__ __forceinline__ void quant_blocks(int n, signed char *q, float *sx, int *corr, F get) {
    for (int b = threadIdx.x; b < (n >> 4); b += kT) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = get(16 * b + i);
        quant_block16_store(v, reinterpret_cast<int4 *>(q) + b, sx + b, corr + b);
    }
}

/* ---------------------------------------------------------------- K1
 * KE = elements of an [E] vector per thread. Everything the prologue needs from global memory is
 * requested up front, in one batch of independent loads: a load inside a dependent loop costs a
 * full L2 round trip per iteration, and the prologue is a serial chain every CTA waits on. */
template <int KE>
__global__ void __launch_bounds__(kT, 1) k_dg_router_shared(GArgs a) {
    extern __shared__ __align__(16) unsigned char sm[];
    const SpDims d = a.d; const int E = d.E, t = threadIdx.x, lane = t & 31, warp = t >> 5, G = gridDim.x, b = blockIdx.x;
    float *va = reinterpret_cast<float *>(sm);           /* [E] */
    float *vb = va + E;                                  /* [E] */
    signed char *q_nx = reinterpret_cast<signed char *>(vb + E);
    signed char *q_in = q_nx + E;
    float *s_nx = reinterpret_cast<float *>(q_in + E); float *s_in = s_nx + E / 16;
    int *c_nx = reinterpret_cast<int *>(s_in + E / 16); int *c_in = c_nx + E / 16;
    double *red = reinterpret_cast<double *>(c_in + E / 16);   /* [32] */
    const double inv_n = 1.0 / (double)E;
    const SpLayerDev &L = a.L;
    /* weights do not depend on the previous kernel: request them before waiting for it */
    float wn[KE], wp[KE], rs[KE], w1[KE], w2[KE], w3[KE];
#pragma unroll
    for (int k = 0; k < KE; k++) {
        const int i = t + kT * k;
        wn[k] = wp[k] = rs[k] = w1[k] = w2[k] = w3[k] = 0.0f;
        if (i < E) {
            wn[k] = __ldg(L.ffn_norm + i); wp[k] = __ldg(L.pre_ffw2 + i); rs[k] = __ldg(L.router_scale + i);
            if (!a.first) { w1[k] = __ldg(a.s.prev_post_ffw1 + i); w2[k] = __ldg(a.s.prev_post_ffw2 + i); w3[k] = __ldg(a.s.prev_post_ffw + i); }
        }
    }
    {   /* this warp's weight rows: static, so they can be requested before the previous kernel is done */
        const int r0 = (int)((long long)b * d.NE / G), r1 = (int)((long long)(b + 1) * d.NE / G);
        const int p0 = (int)((long long)b * d.FFS / G), p1 = (int)((long long)(b + 1) * d.FFS / G);
        const int nr = r1 - r0, np = p1 - p0;
        for (int u = warp; u < nr + np; u += kW) {
            if (u < nr) l2_prefetch(L.router_w + (size_t)(r0 + u) * E, E * 4, lane);
            else { const size_t c = (size_t)(p0 + u - nr);
                l2_prefetch(L.sg_codes + c * (E / 2), E / 2, lane); l2_prefetch(L.su_codes + c * (E / 2), E / 2, lane);
                l2_prefetch(L.sg_bs + c * (E / 32), E / 16, lane); l2_prefetch(L.su_bs + c * (E / 32), E / 16, lane); }
        }
    }
    pdl_wait();
    float x[KE];
    if (a.first) {
#pragma unroll
        for (int k = 0; k < KE; k++) { const int i = t + kT * k; x[k] = i < E ? a.x_prev[i] : 0.0f; }
    } else {
        /* recombine of the previous layer (CF:9014-9019) */
        float dn[KE], ac[KE];
#pragma unroll
        for (int k = 0; k < KE; k++) { const int i = t + kT * k; const bool in = i < E; dn[k] = in ? __ldcg(a.s.dn + i) : 0.0f; ac[k] = in ? __ldcg(a.s.acc + i) : 0.0f; x[k] = in ? __ldcg(a.x_prev + i) : 0.0f; }
        double p1 = 0.0, p2 = 0.0;
#pragma unroll
        for (int k = 0; k < KE; k++) { p1 += (double)dn[k] * dn[k]; p2 += (double)ac[k] * ac[k]; }
        p1 = warp_sum_f64(p1); p2 = warp_sum_f64(p2);
        if (lane == 0) { red[warp] = p1; red[16 + warp] = p2; }
        __syncthreads();
        double s1 = 0.0, s2 = 0.0;
#pragma unroll
        for (int w = 0; w < kW; w++) { s1 += red[w]; s2 += red[16 + w]; }
        __syncthreads();
        const float sc1 = rms_scale(s1, inv_n, d.eps), sc2 = rms_scale(s2, inv_n, d.eps);
        double p3 = 0.0;
#pragma unroll
        for (int k = 0; k < KE; k++) {
            const float mlp = __fmul_rn(__fmul_rn(dn[k], sc1), w1[k]);
            const float t1 = __fmul_rn(__fmul_rn(ac[k], sc2), w2[k]);
            dn[k] = __fadd_rn(mlp, t1); p3 += (double)dn[k] * dn[k];
        }
        const float sc3 = rms_scale(cta_sum(p3, red), inv_n, d.eps);
#pragma unroll
        for (int k = 0; k < KE; k++) x[k] = __fadd_rn(x[k], __fmul_rn(__fmul_rn(dn[k], sc3), w3[k]));
    }
    if (b == 0) {
#pragma unroll
        for (int k = 0; k < KE; k++) { const int i = t + kT * k; if (i < E) a.x_cur[i] = x[k]; }
    }
    /* A: norms of x (CF:8347, 8402-8404, 8425) */
    double part = 0.0;
#pragma unroll
    for (int k = 0; k < KE; k++) part += (double)x[k] * x[k];
    const float scale = rms_scale(cta_sum(part, red), inv_n, d.eps);
#pragma unroll
    for (int k = 0; k < KE; k++) { const int i = t + kT * k; if (i < E) { const float xs = __fmul_rn(x[k], scale); va[i] = __fmul_rn(xs, wn[k]); vb[i] = __fmul_rn(xs, wp[k]); } }
    __syncthreads();
    const int nb = E >> 4;
    for (int bq = t; bq < 2 * nb; bq += kT) {
        const bool first = bq < nb; const int bb = first ? bq : bq - nb;
        const float *src = first ? va : vb;
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; i++) { const float4 f = reinterpret_cast<const float4 *>(src + 16 * bb)[i]; v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w; }
        quant_block16_store(v, reinterpret_cast<int4 *>(first ? q_nx : q_in) + bb, (first ? s_nx : s_in) + bb, (first ? c_nx : c_in) + bb);
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < KE; k++) { const int i = t + kT * k; if (i < E) va[i] = __fmul_rn(__fmul_rn(__fmul_rn(x[k], scale), d.inv_sqrt_e), rs[k]); }
    if (b == 0) {                                        /* the routed experts' input, for K2 */
        for (int i = t; i < E / 16; i += kT) { reinterpret_cast<int4 *>(a.s.in_q)[i] = reinterpret_cast<const int4 *>(q_in)[i]; a.s.in_s[i] = s_in[i]; a.s.in_c[i] = c_in[i]; }
    }
    __syncthreads();
    pdl_launch();
    {   /* the next kernel's routing-independent rows (shared-expert down): ask L2 for them now */
        const int j0 = (int)((long long)b * E / G), nj = (int)((long long)(b + 1) * E / G) - j0;
        if (warp == kW - 1) { l2_prefetch(L.sd_codes + (size_t)j0 * (d.FFS / 2), nj * (d.FFS / 2), lane); l2_prefetch(L.sd_bs + (size_t)j0 * (d.FFS / 32), nj * (d.FFS / 16), lane); }
    }
    /* B: router rows + shared gate/up pairs */
    const int r0 = (int)((long long)b * d.NE / G), r1 = (int)((long long)(b + 1) * d.NE / G);
    const int p0 = (int)((long long)b * d.FFS / G), p1 = (int)((long long)(b + 1) * d.FFS / G);
    const int nr = r1 - r0, np = p1 - p0, n32 = E >> 5;
    const size_t rb = (size_t)E / 2;
    const ActS act{reinterpret_cast<const int4 *>(q_nx), s_nx, c_nx};
    for (int u = warp; u < nr + np; u += kW) {
        if (u < nr) {
            const int r = r0 + u;
            const float *wrow = L.router_w + (size_t)r * E;
            float acc = 0.0f;
            for (int q0 = lane; q0 < (E >> 2); q0 += 32 * 8) {
                float4 w[8];
#pragma unroll
                for (int i = 0; i < 8; i++) { const int q = q0 + 32 * i; if (q < (E >> 2)) w[i] = ld_stream_f4(wrow + 4 * q); }
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const int q = q0 + 32 * i;
                    if (q < (E >> 2)) {
                        const float4 xv = *reinterpret_cast<const float4 *>(va + 4 * q);
                        acc = __fmaf_rn(w[i].x, xv.x, acc); acc = __fmaf_rn(w[i].y, xv.y, acc); acc = __fmaf_rn(w[i].z, xv.z, acc); acc = __fmaf_rn(w[i].w, xv.w, acc);
                    }
                }
            }
            acc = warp_tree(acc);
            if (lane == 0) { if (L.router_bias) acc = __fadd_rn(acc, __ldg(L.router_bias + r)); a.s.logits[r] = acc; }
        } else {
            const int c = p0 + (u - nr);
            float h;
            NIT_SWITCH(n32, h = pair_gelu<NIT>(L.sg_codes + c * rb, L.sg_bs + (size_t)c * n32, L.su_codes + c * rb, L.su_bs + (size_t)c * n32, n32, lane, act));
            if (lane == 0) a.s.hd[c] = h;
        }
    }
    __syncthreads();
}

/* moe_topk_host (CF:6220-6240), whole CTA */
__device__ void topk_cta(const float *logits_g, const SpDims &d, const float *dscale_s, float *lg, double *ex, float *p, double *red,
                         int *sel_desc, float *p_desc, int *sel_asc, float *cw, int *status) {
    const int NE = d.NE, NU = d.NU, t = threadIdx.x;
    float *wmaxf = reinterpret_cast<float *>(red + 16);
    float mx = -INFINITY; int bad = 0;
    for (int i = t; i < NE; i += kT) { const float l = __ldcg(logits_g + i); lg[i] = l; if (l != l) bad = 1; mx = fmaxf(mx, l); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); bad |= __shfl_xor_sync(0xffffffffu, bad, o); }
    if ((t & 31) == 0) wmaxf[t >> 5] = mx;
    if (bad && (t & 31) == 0) atomicExch(status, SP_KERR_NAN_ROUTER);
    if (t < SP_MAX_NU) { sel_desc[t] = t < NE ? t : 0; p_desc[t] = 0.0f; }
    __syncthreads();
    mx = wmaxf[0];
#pragma unroll
    for (int w = 1; w < kW; w++) mx = fmaxf(mx, wmaxf[w]);
    double part = 0.0;
    for (int i = t; i < NE; i += kT) { const double e = exp((double)lg[i] - (double)mx); ex[i] = e; part += e; }
    const double sum = cta_sum(part, red);
    const double rsum = 1.0 / sum;
    for (int i = t; i < NE; i += kT) p[i] = (float)(ex[i] * rsum);
    __syncthreads();
    for (int i = t; i < NE; i += kT) {
        const float pi = p[i]; int r = 0;
        for (int j = 0; j < NE; j++) { const float pj = p[j]; r += (pj > pi) || (pj == pi && j < i); }
        if (r < NU && pi == pi) { sel_desc[r] = i; p_desc[r] = pi; }
    }
    __syncthreads();
    if (t < 32) {
        float wnorm = 0.0f; int e = 0, slot = 0;
        if (t < NU) {
            float ws = 0.0f;
            for (int k = 0; k < NU; k++) ws = __fadd_rn(ws, p_desc[k]);
            if (ws < 6.103515625e-5f) ws = 6.103515625e-5f;
            e = sel_desc[t];
            wnorm = __fdiv_rn(p_desc[t], ws);
            for (int j = 0; j < NU; j++) slot += (sel_desc[j] < e);
        }
        __syncwarp();
        if (t < NU) { sel_asc[slot] = e; cw[slot] = __fmul_rn(wnorm, dscale_s[e]); p_desc[t] = wnorm; }
    }
    __syncthreads();
}

/* ---------------------------------------------------------------- K2 */
__global__ void __launch_bounds__(kT, 1) k_dg_experts_up(GArgs a) {
    extern __shared__ __align__(16) unsigned char sm[];
    const SpDims d = a.d; const int E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, G = gridDim.x, b = blockIdx.x;
    signed char *q_in = reinterpret_cast<signed char *>(sm);
    signed char *q_hd = q_in + E;
    float *s_in = reinterpret_cast<float *>(q_hd + FFS); float *s_hd = s_in + E / 16;
    int *c_in = reinterpret_cast<int *>(s_hd + FFS / 16); int *c_hd = c_in + E / 16;
    double *red = reinterpret_cast<double *>(((uintptr_t)(c_hd + FFS / 16) + 7) & ~(uintptr_t)7);   /* [48] */
    double *ex = red + 48;                                /* [NE] */
    float *lg = reinterpret_cast<float *>(ex + NE); float *p = lg + NE;
    int *sel_desc = reinterpret_cast<int *>(p + 2 * NE); float *p_desc = reinterpret_cast<float *>(sel_desc + SP_MAX_NU);
    int *sel_asc = reinterpret_cast<int *>(p_desc + SP_MAX_NU); float *cw = reinterpret_cast<float *>(sel_asc + SP_MAX_NU);
    const SpLayerDev &L = a.L;
    float *dsc = p + NE;                                  /* [NE] per-expert down scales */
    for (int i = t; i < NE; i += kT) dsc[i] = __ldg(L.dexps_scale + i);      /* weights: before the wait */
    pdl_wait();
    /* the activations this CTA needs, requested in one batch before the top-k chain */
    for (int i = t; i < E / 16; i += kT) { reinterpret_cast<int4 *>(q_in)[i] = __ldcg(reinterpret_cast<const int4 *>(a.s.in_q) + i); s_in[i] = __ldcg(a.s.in_s + i); c_in[i] = __ldcg(a.s.in_c + i); }
    {
        const int nbh = FFS >> 4, bq0 = kT - 1 - t;       /* the LAST threads take the hd blocks; the first NE run the top-k */
        const bool mine = bq0 < nbh;
        float hv[16];
        if (mine) {
#pragma unroll
            for (int i = 0; i < 16; i++) hv[i] = __ldcg(a.s.hd + 16 * bq0 + i);
        }
        topk_cta(a.s.logits, d, dsc, lg, ex, p, red, sel_desc, p_desc, sel_asc, cw, a.s.status);
        if (mine) quant_block16_store(hv, reinterpret_cast<int4 *>(q_hd) + bq0, s_hd + bq0, c_hd + bq0);
        for (int bq = bq0 + kT; bq < nbh; bq += kT) {      /* only when FFS/16 exceeds the CTA */
            float v[16];
#pragma unroll
            for (int i = 0; i < 16; i++) v[i] = __ldcg(a.s.hd + 16 * bq + i);
            quant_block16_store(v, reinterpret_cast<int4 *>(q_hd) + bq, s_hd + bq, c_hd + bq);
        }
    }
    if (b == 0 && t < NU) {
        a.s.sel_asc[t] = sel_asc[t]; a.s.cw[t] = cw[t];
        if (a.sel_out) a.sel_out[t] = sel_desc[t];
        if (a.wts_out) a.wts_out[t] = p_desc[t];
    }
    __syncthreads();
    pdl_launch();
    {   /* the routed down rows the next kernel will read in this CTA's slice: known now, ask L2 for them */
        const int j0p = (int)((long long)b * E / G), njp = (int)((long long)(b + 1) * E / G) - j0p;
        for (int sl = warp; sl < NU; sl += kW) {
            const size_t row = (size_t)sel_asc[sl] * E + j0p;
            l2_prefetch(L.dn_codes + row * (FFE / 2), njp * (FFE / 2), lane);
            l2_prefetch(L.dn_bs + row * (FFE / 32), njp * (FFE / 16), lane);
        }
    }
    const int NP = NU * FFE;
    const int P0 = (int)((long long)b * NP / G), P1 = (int)((long long)(b + 1) * NP / G);
    const int j0 = (int)((long long)b * E / G), j1 = (int)((long long)(b + 1) * E / G);
    const int np = P1 - P0, nj = j1 - j0, n32 = E >> 5, n32s = FFS >> 5;
    for (int u = warp; u < np; u += kW) {                  /* the routed rows of this warp, now that the selection is known */
        const int pu = P0 + u, slot = pu / FFE, c = pu - slot * FFE;
        const size_t grow = (size_t)sel_asc[slot] * 2 * FFE + c, urow = grow + FFE;
        l2_prefetch(L.gu_codes + grow * (E / 2), E / 2, lane); l2_prefetch(L.gu_codes + urow * (E / 2), E / 2, lane);
        l2_prefetch(L.gu_bs + grow * (E / 32), E / 16, lane); l2_prefetch(L.gu_bs + urow * (E / 32), E / 16, lane);
    }
    const ActS act_in{reinterpret_cast<const int4 *>(q_in), s_in, c_in}, act_hd{reinterpret_cast<const int4 *>(q_hd), s_hd, c_hd};
    const size_t rb = (size_t)E / 2, rbs = (size_t)FFS / 2;
    /* shared-expert down rows: two per warp iteration, loads of both in flight */
    for (int q0 = warp * 2; q0 < nj; q0 += kW * 2) {
        const int ja = j0 + q0, jb = (q0 + 1 < nj) ? ja + 1 : ja;
        float oa, ob;
        NIT_SWITCH(n32s, {
            int4 wa[NIT], wb[NIT]; unsigned short sa[NIT], sb[NIT];
            row_load<NIT>(L.sd_codes + ja * rbs, L.sd_bs + (size_t)ja * n32s, n32s, lane, wa, sa);
            row_load<NIT>(L.sd_codes + jb * rbs, L.sd_bs + (size_t)jb * n32s, n32s, lane, wb, sb);
            oa = row_fma<NIT>(wa, sa, n32s, lane, act_hd); ob = row_fma<NIT>(wb, sb, n32s, lane, act_hd); });
        if (lane == 0) { a.s.dn[ja] = oa; if (jb != ja) a.s.dn[jb] = ob; }
    }
    /* routed gate|up pairs: the next pair's rows are requested before this pair is computed */
    NIT_SWITCH(n32, {
        int4 wg[NIT], wu[NIT], ng[NIT], nu[NIT]; unsigned short sg[NIT], su[NIT], tg[NIT], tu[NIT];
        auto load = [&](int u, int4 (&g_)[NIT], unsigned short (&gs_)[NIT], int4 (&u_)[NIT], unsigned short (&us_)[NIT]) {
            const int pu = P0 + u, slot = pu / FFE, c = pu - slot * FFE;
            const size_t grow = (size_t)sel_asc[slot] * 2 * FFE + c, urow = grow + FFE;
            row_load<NIT>(L.gu_codes + grow * rb, L.gu_bs + grow * n32, n32, lane, g_, gs_);
            row_load<NIT>(L.gu_codes + urow * rb, L.gu_bs + urow * n32, n32, lane, u_, us_);
        };
        if (warp < np) load(warp, wg, sg, wu, su);
        for (int u = warp; u < np; u += kW) {
            const bool more = u + kW < np;
            if (more) load(u + kW, ng, tg, nu, tu);
            const float g = row_fma<NIT>(wg, sg, n32, lane, act_in);
            const float uu = row_fma<NIT>(wu, su, n32, lane, act_in);
            const float h = gelu_mul(g, uu);
            if (lane == 0) a.s.h[P0 + u] = h;
            if (more) {
#pragma unroll
                for (int i = 0; i < NIT; i++) { wg[i] = ng[i]; wu[i] = nu[i]; sg[i] = tg[i]; su[i] = tu[i]; }
            }
        } });
    __syncthreads();
}

/* ---------------------------------------------------------------- K3 */
__global__ void __launch_bounds__(kT, 1) k_dg_experts_down(GArgs a) {
    extern __shared__ __align__(16) unsigned char sm[];
    const SpDims d = a.d; const int E = d.E, NU = d.NU, FFE = d.FFE;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, G = gridDim.x, b = blockIdx.x;
    const int nblk = (NU * FFE) >> 4, rows_max = (E + G - 1) / G + 1;
    signed char *q_h = reinterpret_cast<signed char *>(sm);
    float *s_h = reinterpret_cast<float *>(q_h + (size_t)NU * FFE);
    int *c_h = reinterpret_cast<int *>(s_h + nblk);
    float *out = reinterpret_cast<float *>(c_h + nblk);                   /* [NU][rows_max] */
    int *sel_asc = reinterpret_cast<int *>(out + (size_t)NU * rows_max); float *cw = reinterpret_cast<float *>(sel_asc + SP_MAX_NU);
    const SpLayerDev &L = a.L;
    pdl_wait();
    quant_blocks(NU * FFE, q_h, s_h, c_h, [&](int i) { return __ldcg(a.s.h + i); });
    if (t < NU) { sel_asc[t] = __ldcg(a.s.sel_asc + t); cw[t] = __ldcg(a.s.cw + t); }
    __syncthreads();
    pdl_launch();
    if (a.has_next) {   /* the next layer's router rows and shared gate/up pairs of this CTA's slice */
        const SpLayerDev &N = a.Ln;
        const int r0 = (int)((long long)b * d.NE / G), nr = (int)((long long)(b + 1) * d.NE / G) - r0;
        const int p0 = (int)((long long)b * d.FFS / G), np = (int)((long long)(b + 1) * d.FFS / G) - p0;
        if (warp == kW - 1) l2_prefetch(N.router_w + (size_t)r0 * E, nr * E * 4, lane);
        if (warp == kW - 2) { l2_prefetch(N.sg_codes + (size_t)p0 * (E / 2), np * (E / 2), lane); l2_prefetch(N.sg_bs + (size_t)p0 * (E / 32), np * (E / 16), lane); }
        if (warp == kW - 3) { l2_prefetch(N.su_codes + (size_t)p0 * (E / 2), np * (E / 2), lane); l2_prefetch(N.su_bs + (size_t)p0 * (E / 32), np * (E / 16), lane); }
    }
    const int j0 = (int)((long long)b * E / G), j1 = (int)((long long)(b + 1) * E / G), nj = j1 - j0;
    const int n32 = FFE >> 5, blk16 = FFE >> 4, U = nj * NU;
    const size_t rb = (size_t)FFE / 2;
    constexpr int R = 8;
    for (int u0 = warp * R; u0 < U; u0 += kW * R) {
        /* R rows at a time: their loads are in flight together */
        int4 w[R]; unsigned short sc[R]; int sl[R], jr[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            const int u = (u0 + r < U) ? u0 + r : u0;
            jr[r] = u / NU; sl[r] = u - jr[r] * NU;
            const size_t row = (size_t)sel_asc[sl[r]] * E + (j0 + jr[r]);
            if (lane < n32) { w[r] = ld_stream16(L.dn_codes + row * rb + 16 * lane); sc[r] = ld_stream_u16(L.dn_bs + row * n32 + lane); }
        }
        if (n32 > 32) {                                                /* wider experts: the general row routine */
#pragma unroll
            for (int r = 0; r < R; r++) if (u0 + r < U) {
                const size_t row = (size_t)sel_asc[sl[r]] * E + (j0 + jr[r]);
                const ActS act{reinterpret_cast<const int4 *>(q_h) + (size_t)sl[r] * blk16, s_h + (size_t)sl[r] * blk16, c_h + (size_t)sl[r] * blk16};
                float o;
                NIT_SWITCH(n32, o = one_row<NIT>(L.dn_codes + row * rb, L.dn_bs + row * n32, n32, lane, act));
                if (lane == 0) out[sl[r] * rows_max + jr[r]] = o;
            }
            continue;
        }
        float f[R];
#pragma unroll
        for (int r = 0; r < R; r++) {
            f[r] = 0.0f;
            if (lane < n32) {
                const int4 *q = reinterpret_cast<const int4 *>(q_h) + (size_t)sl[r] * blk16;
                const int2 corr = *reinterpret_cast<const int2 *>(c_h + (size_t)sl[r] * blk16 + 2 * lane);
                const float2 sx = *reinterpret_cast<const float2 *>(s_h + (size_t)sl[r] * blk16 + 2 * lane);
                int a0, a1;
                q4b_chunk_dot(w[r], q[2 * lane], q[2 * lane + 1], corr.x, corr.y, a0, a1);
                f[r] = __fmaf_rn(h2f(sc[r]), __fmaf_rn((float)a0, sx.x, __fmul_rn((float)a1, sx.y)), 0.0f);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int r = 0; r < R; r++) f[r] += __shfl_down_sync(0xffffffffu, f[r], o);
        if (lane == 0) {
#pragma unroll
            for (int r = 0; r < R; r++) if (u0 + r < U) out[sl[r] * rows_max + jr[r]] = f[r];
        }
    }
    __syncthreads();
    for (int jj = t; jj < nj; jj += kT) {                                  /* k_moe_combine_ord, CF:6071-6077 */
        float acc = 0.0f;
        for (int k = 0; k < NU; k++) acc = __fadd_rn(acc, __fmul_rn(cw[k], out[k * rows_max + jj]));
        a.s.acc[j0 + jj] = acc;
    }
}

/* ---------------------------------------------------------------- KF: recombine of the last layer (CF:9014-9019) */
__global__ void __launch_bounds__(kT, 1) k_dg_finish(GArgs a, float *y) {
    extern __shared__ __align__(16) unsigned char sm[];
    constexpr int KE = 8;
    const SpDims d = a.d; const int E = d.E, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    double *red = reinterpret_cast<double *>(sm);
    const double inv_n = 1.0 / (double)E;
    float w1[KE], w2[KE], w3[KE], dn[KE], ac[KE], x[KE];
#pragma unroll
    for (int k = 0; k < KE; k++) { const int i = t + kT * k; const bool in = i < E;
        w1[k] = in ? __ldg(a.s.prev_post_ffw1 + i) : 0.0f; w2[k] = in ? __ldg(a.s.prev_post_ffw2 + i) : 0.0f; w3[k] = in ? __ldg(a.s.prev_post_ffw + i) : 0.0f; }
    pdl_wait();
#pragma unroll
    for (int k = 0; k < KE; k++) { const int i = t + kT * k; const bool in = i < E; dn[k] = in ? __ldcg(a.s.dn + i) : 0.0f; ac[k] = in ? __ldcg(a.s.acc + i) : 0.0f; x[k] = in ? __ldcg(a.x_prev + i) : 0.0f; }
    double p1 = 0.0, p2 = 0.0;
#pragma unroll
    for (int k = 0; k < KE; k++) { p1 += (double)dn[k] * dn[k]; p2 += (double)ac[k] * ac[k]; }
    p1 = warp_sum_f64(p1); p2 = warp_sum_f64(p2);
    if (lane == 0) { red[warp] = p1; red[16 + warp] = p2; }
    __syncthreads();
    double s1 = 0.0, s2 = 0.0;
#pragma unroll
    for (int w = 0; w < kW; w++) { s1 += red[w]; s2 += red[16 + w]; }
    __syncthreads();
    const float sc1 = rms_scale(s1, inv_n, d.eps), sc2 = rms_scale(s2, inv_n, d.eps);
    double p3 = 0.0;
#pragma unroll
    for (int k = 0; k < KE; k++) {
        const float mlp = __fmul_rn(__fmul_rn(dn[k], sc1), w1[k]);
        const float t1 = __fmul_rn(__fmul_rn(ac[k], sc2), w2[k]);
        dn[k] = __fadd_rn(mlp, t1); p3 += (double)dn[k] * dn[k];
    }
    const float sc3 = rms_scale(cta_sum(p3, red), inv_n, d.eps);
#pragma unroll
    for (int k = 0; k < KE; k++) { const int i = t + kT * k; if (i < E) y[i] = __fadd_rn(x[k], __fmul_rn(__fmul_rn(dn[k], sc3), w3[k])); }
}

template <class K, class... Args>
cudaError_t launch_pdl(K kernel, int grid, size_t smem, cudaStream_t st, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kT); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization; at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

}  // namespace

cudaError_t sp_graph_prepare() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(k_dg_router_shared<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(k_dg_router_shared<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(k_dg_experts_up, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024)) != cudaSuccess) return e;
    return cudaFuncSetAttribute(k_dg_experts_down, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
}

cudaError_t sp_graph_launch_finish(const SpDims &d, const SpLayerDev &last, const SpGraphScratch &sc, const float *x_prev, float *y_out,
                                   cudaStream_t st, bool pdl) {
    GArgs a{};
    a.d = d; a.s = sc; a.x_prev = x_prev;
    a.s.prev_post_ffw1 = last.post_ffw1; a.s.prev_post_ffw2 = last.post_ffw2; a.s.prev_post_ffw = last.post_ffw;
    return launch_pdl(k_dg_finish, 1, 32 * 8 + 64, st, pdl, a, y_out);
}

/* Enqueues layers [lf, lf+nl) for one token on `st` (capturable into a CUDA graph). */
cudaError_t sp_graph_decode_enqueue(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl, const float *x_in, float *y_out,
                                    int32_t *sel, float *wts, const SpGraphScratch &sc, int sms, cudaStream_t st, bool pdl, int *nlaunch) {
    const int E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;
    const int grid = sms;
    const size_t sm1 = 2 * (size_t)E * 4 + 2 * (size_t)E + 4 * (size_t)(E / 16) * 4 + 32 * 8 + 64;
    const size_t sm2 = (size_t)E + FFS + 2 * ((size_t)(E / 16) + FFS / 16) * 4 + 8 + 48 * 8 + (size_t)NE * 8 + 3 * (size_t)NE * 4 + 4 * SP_MAX_NU * 4 + 64;
    const int rows_max = (E + grid - 1) / grid + 1;
    const size_t sm3 = (size_t)NU * FFE + 2 * (size_t)((NU * FFE) >> 4) * 4 + (size_t)NU * rows_max * 4 + 2 * SP_MAX_NU * 4 + 64;
    if (sm1 > 100 * 1024 || sm2 > 100 * 1024 || sm3 > 100 * 1024) return cudaErrorInvalidValue;
    cudaError_t e = cudaSuccess;
    for (int li = 0; li < nl && e == cudaSuccess; li++) {
        GArgs a{};
        a.L = layers_host[lf + li]; a.d = d; a.s = sc; a.first = (li == 0);
        a.x_prev = (li == 0) ? x_in : sc.xbuf[(li - 1) & 1];
        a.x_cur = sc.xbuf[li & 1];
        if (li > 0) { a.s.prev_post_ffw1 = layers_host[lf + li - 1].post_ffw1; a.s.prev_post_ffw2 = layers_host[lf + li - 1].post_ffw2; a.s.prev_post_ffw = layers_host[lf + li - 1].post_ffw; }
        a.sel_out = sel ? sel + (size_t)li * NU : nullptr; a.wts_out = wts ? wts + (size_t)li * NU : nullptr;
        a.has_next = li + 1 < nl; if (a.has_next) a.Ln = layers_host[lf + li + 1];
        e = (E <= 6 * kT) ? launch_pdl(k_dg_router_shared<6>, grid, sm1, st, pdl && li > 0, a) : launch_pdl(k_dg_router_shared<8>, grid, sm1, st, pdl && li > 0, a); (*nlaunch)++;
        if (e == cudaSuccess) { e = launch_pdl(k_dg_experts_up, grid, sm2, st, pdl, a); (*nlaunch)++; }
        if (e == cudaSuccess) { e = launch_pdl(k_dg_experts_down, grid, sm3, st, pdl, a); (*nlaunch)++; }
    }
    if (e == cudaSuccess) { e = sp_graph_launch_finish(d, layers_host[lf + nl - 1], sc, sc.xbuf[(nl - 1) & 1], y_out, st, pdl); (*nlaunch)++; }
    return e;
}
