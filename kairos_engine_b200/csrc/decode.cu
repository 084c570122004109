/* decode.cu — the M=1 decode path of the MoE feed-forward stack as ONE persistent kernel.
 *
 * Replaces, for n_tok == 1, the ~20 launches + one host round trip per layer of
 * g4_ffn_apply (CF:8314-9050; PRE/MID/TAIL phases CF:8338-8339): k_rmsnorm, gemv_w_packed x3
 * (shared expert), k_gelu_mul, k_moe_router_prep, router SGEMM, D2H + moe_topk_host,
 * k_quant_act_int8, k_gemv_q4b_dp4a_grp x2, k_moe_gelu_split_batch, k_moe_combine_ord and the
 * recombine norms. CF = src/backends/cuda/cuda_forward.cu of nihilistau/kairos-engine.
 *
 * One CTA per SM, launched cooperatively so all CTAs are co-resident; the residual x lives in
 * every CTA's shared memory across layers. Per layer there are three grid-wide barriers:
 *
 *   A (local)  sum x^2 -> ffn_norm / pre_ffw2 / router-prep vectors, int8-quantised in smem
 *   B (grid)   router rows (fp32) + shared-expert gate/up row pairs -> logits, hd = gelu(g)*u
 *   --- barrier 1
 *   C (local)  softmax/top-NU/renorm (moe_topk_host semantics), quantise hd
 *   D (grid)   routed gate|up row pairs of the NU selected experts + shared-expert down rows
 *   --- barrier 2
 *   E (local)  quantise the NU expert activations h
 *   F (grid)   routed down rows; each CTA owns output rows j for ALL experts, so the ordered
 *              combine acc = acc + w*out (ascending expert id) happens inside the CTA
 *   --- barrier 3
 *   G (local)  post_ffw1 / post_ffw2 norms, branch sum, post_ffw norm, residual add -> x
 *
 * Arithmetic is the reference's decode arithmetic (int8 per-16 activation quant, exact int32
 * dots per 16, fp32 scale/accumulate in the order of k_gemv_q4b_dp4a_v2: chunk c in lane c%32,
 * then the shuffle tree), so results differ from the reference only through tanhf's last bits.
 */
#include "common.cuh"
#include "decode.cuh"

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr unsigned kBarrierSpinLimit = 1u << 21;   /* ~1 s of polling: then give up and flag */

struct Act {               /* one quantised activation vector in shared memory */
    const int4 *q;         /* [in/16] blocks of 16 int8, de-interleaved (common.cuh) */
    const float *sx;       /* [in/16] block scales */
    const int *corr;       /* [in/16] 8 * sum(q) per block */
};

struct Smem {
    float *x, *va, *vb;                 /* [E] residual, two work vectors */
    signed char *q_nx, *q_in, *q_hd, *q_h;
    float *s_nx, *s_in, *s_hd, *s_h;
    int *c_nx, *c_in, *c_hd, *c_h;
    double *red;                        /* [256] */
    float *p, *lg;                      /* [NE] probabilities, logits */
    int *flag;                          /* barrier verdict broadcast */
    SpLayerDev *L;                      /* this layer's pointers */
    float *out;                         /* [NU][rows_per_cta_max] */
    int *sel_asc; float *cw;            /* [NU] ascending-id slots, combine weights */
    int *sel_desc; float *p_desc;       /* [NU] */
};

__device__ __forceinline__ size_t align16(size_t v) { return (v + 15) & ~(size_t)15; }

__device__ Smem carve(unsigned char *base, const SpDims &d, int rows_f_max) {
    Smem s; size_t o = 0;
    auto take = [&](size_t bytes) { unsigned char *p = base + o; o = align16(o + bytes); return p; };
    s.x = (float *)take(4 * d.E); s.va = (float *)take(4 * d.E); s.vb = (float *)take(4 * d.E);
    s.q_nx = (signed char *)take(d.E); s.q_in = (signed char *)take(d.E);
    s.q_hd = (signed char *)take(d.FFS); s.q_h = (signed char *)take((size_t)d.NU * d.FFE);
    s.s_nx = (float *)take(4 * (d.E / 16)); s.s_in = (float *)take(4 * (d.E / 16));
    s.s_hd = (float *)take(4 * (d.FFS / 16)); s.s_h = (float *)take(4 * (size_t)d.NU * (d.FFE / 16));
    s.c_nx = (int *)take(4 * (d.E / 16)); s.c_in = (int *)take(4 * (d.E / 16));
    s.c_hd = (int *)take(4 * (d.FFS / 16)); s.c_h = (int *)take(4 * (size_t)d.NU * (d.FFE / 16));
    s.red = (double *)take(8 * 256);
    s.p = (float *)take(4 * d.NE); s.lg = (float *)take(4 * d.NE);
    s.flag = (int *)take(16); s.L = (SpLayerDev *)take(sizeof(SpLayerDev));
    s.out = (float *)take(4 * (size_t)d.NU * rows_f_max);
    s.sel_asc = (int *)take(4 * SP_MAX_NU); s.cw = (float *)take(4 * SP_MAX_NU);
    s.sel_desc = (int *)take(4 * SP_MAX_NU); s.p_desc = (float *)take(4 * SP_MAX_NU);
    return s;
}

/* sum of squares in the reference's order (k_rmsnorm, CF:503-511): 256 strided double
 * partials, then sh[t] += sh[t+o] for o = 128 .. 1. All threads must call. */
__device__ double block_sumsq(const float *v, int n, double *sh) {
    const int t = threadIdx.x;
    if (t < 256) { double s = 0.0; for (int i = t; i < n; i += 256) { const double a = v[i]; s += a * a; } sh[t] = s; }
    __syncthreads();
    if (t < 128) sh[t] += sh[t + 128];
    __syncthreads();
    if (t < 64) sh[t] += sh[t + 64];
    __syncthreads();
    if (t < 32) {
        double a = sh[t] + sh[t + 32];
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

/* Q4B row . int8 activation, this lane's share: chunks c = lane, lane+32, ... (CF:1697-1710). */
template <int NIT>
__device__ __forceinline__ void row_load(const uint8_t *codes, const uint16_t *bs, int n32, int lane,
                                         int4 (&w)[NIT], unsigned short (&s)[NIT]) {
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) { w[i] = ld_stream16(codes + 16 * (size_t)c); s[i] = ld_stream_u16(bs + c); }
    }
}
template <int NIT>
__device__ __forceinline__ float row_fma(const int4 (&w)[NIT], const unsigned short (&s)[NIT], int n32, int lane, const Act &a) {
    float facc = 0.0f;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) {
            int a0, a1;
            q4b_chunk_dot(w[i], a.q[2 * c], a.q[2 * c + 1], a.corr[2 * c], a.corr[2 * c + 1], a0, a1);
            const float t = __fmaf_rn((float)a0, a.sx[2 * c], __fmul_rn((float)a1, a.sx[2 * c + 1]));
            facc = __fmaf_rn(h2f(s[i]), t, facc);
        }
    }
    return facc;
}
__device__ __forceinline__ float warp_tree(float v) {      /* CF:1711: lane 0 holds the row sum */
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

template <int NIT>
__device__ __forceinline__ float pair_gelu(const uint8_t *gc, const uint16_t *gs, const uint8_t *uc, const uint16_t *us,
                                           int n32, int lane, const Act &a) {
    int4 wg[NIT], wu[NIT]; unsigned short sg[NIT], su[NIT];
    row_load<NIT>(gc, gs, n32, lane, wg, sg);
    row_load<NIT>(uc, us, n32, lane, wu, su);
    const float g = warp_tree(row_fma<NIT>(wg, sg, n32, lane, a));
    const float u = warp_tree(row_fma<NIT>(wu, su, n32, lane, a));
    return gelu_mul(g, u);                                   /* meaningful in lane 0 */
}
template <int NIT>
__device__ __forceinline__ float single_row(const uint8_t *c, const uint16_t *s, int n32, int lane, const Act &a) {
    int4 w[NIT]; unsigned short sc[NIT];
    row_load<NIT>(c, s, n32, lane, w, sc);
    return warp_tree(row_fma<NIT>(w, sc, n32, lane, a));
}

#define NIT_SWITCH(n32, EXPR)                                    \
    do { const int nit_ = ((n32) + 31) >> 5;                     \
         if (nit_ <= 1) { constexpr int NIT = 1; EXPR; }         \
         else if (nit_ == 2) { constexpr int NIT = 2; EXPR; }    \
         else if (nit_ == 3) { constexpr int NIT = 3; EXPR; }    \
         else { constexpr int NIT = 4; EXPR; } } while (0)

/* router row in fp32, fixed order: lane l takes the float4 groups q = l, l+32, ... with
 * acc = fma(w, x, acc) over the four elements in order, then the shuffle tree. */
__device__ __forceinline__ float router_row(const float *wrow, const float *rin, int E, int lane) {
    const int nq = E >> 2;
    float acc = 0.0f;
    for (int q0 = lane; q0 < nq; q0 += 32 * 8) {
        float4 w[8];
#pragma unroll
        for (int i = 0; i < 8; i++) { const int q = q0 + 32 * i; if (q < nq) w[i] = ld_stream_f4(wrow + 4 * (size_t)q); }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const int q = q0 + 32 * i;
            if (q < nq) {
                const float4 xv = *reinterpret_cast<const float4 *>(rin + 4 * q);
                acc = __fmaf_rn(w[i].x, xv.x, acc); acc = __fmaf_rn(w[i].y, xv.y, acc);
                acc = __fmaf_rn(w[i].z, xv.z, acc); acc = __fmaf_rn(w[i].w, xv.w, acc);
            }
        }
    }
    return warp_tree(acc);
}

/* quantise a vector (read through `get`) into de-interleaved int8 blocks in shared memory */
template <class F>
__device__ __forceinline__ void quant_vec(int n, signed char *q, float *sx, int *corr, F get) {
    for (int b = threadIdx.x; b < (n >> 4); b += blockDim.x) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = get(16 * b + i);
        sx[b] = quant_block16(v, q + 16 * b, corr + b);
    }
}

/* Grid-wide barrier on a monotonically increasing counter. Every wait is bounded: after
 * kBarrierSpinLimit polls the CTA records SP_KERR_BARRIER_TIMEOUT and every CTA leaves. */
__device__ __forceinline__ bool grid_barrier(unsigned *ctr, unsigned target, int *status, int *verdict) {
    __syncthreads();
    if (threadIdx.x == 0) {
        int ok = 1;
        __threadfence();
        atomicAdd(ctr, 1u);
        unsigned spins = 0;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(ctr) : "memory");
            if ((int)(v - target) >= 0) break;
            if (++spins > kBarrierSpinLimit || *(volatile int *)status == SP_KERR_BARRIER_TIMEOUT) {
                atomicExch(status, SP_KERR_BARRIER_TIMEOUT);
                ok = 0;
                break;
            }
        }
        __threadfence();
        *verdict = ok;
    }
    __syncthreads();
    return *verdict != 0;          /* one value for the whole CTA: no thread leaves alone */
}

/* moe_topk_host (CF:6220-6240) on the device, run redundantly by every CTA. */
__device__ void topk_block(const float *logits_g, const SpDims &d, const float *dscale, Smem &s, int *status) {
    const int NE = d.NE, NU = d.NU, t = threadIdx.x;
    float *wmaxf = reinterpret_cast<float *>(s.red);           /* [kWarps] */
    /* max */
    float mx = -INFINITY; int bad = 0;
    for (int i = t; i < NE; i += blockDim.x) { const float l = ld_cg_f32(logits_g + i); s.lg[i] = l; if (l != l) bad = 1; mx = fmaxf(mx, l); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); bad |= __shfl_xor_sync(0xffffffffu, bad, o); }
    if ((t & 31) == 0) { wmaxf[t >> 5] = mx; }
    if (bad && (t & 31) == 0) atomicExch(status, SP_KERR_NAN_ROUTER);
    __syncthreads();
    mx = wmaxf[0];
    for (int w = 1; w < kWarps; w++) mx = fmaxf(mx, wmaxf[w]);
    __syncthreads();
    /* exp in double, sum in double (fixed tree: strided partials, warp shuffle, warps in order) */
    double part = 0.0;
    for (int i = t; i < NE; i += blockDim.x) part += exp((double)s.lg[i] - (double)mx);
    part = warp_sum_f64(part);
    if ((t & 31) == 0) s.red[t >> 5] = part;
    __syncthreads();
    double sum = 0.0;
    for (int w = 0; w < kWarps; w++) sum += s.red[w];
    /* p = (float)(exp(l - mx) / sum) */
    for (int i = t; i < NE; i += blockDim.x) s.p[i] = (float)(exp((double)s.lg[i] - (double)mx) / sum);
    if (t < SP_MAX_NU) { s.sel_desc[t] = t < NE ? t : 0; s.p_desc[t] = 0.0f; }
    __syncthreads();
    /* insertion with strict > == rank by (p desc, id asc) */
    for (int i = t; i < NE; i += blockDim.x) {
        const float pi = s.p[i]; int r = 0;
        for (int j = 0; j < NE; j++) { const float pj = s.p[j]; r += (pj > pi) || (pj == pi && j < i); }
        if (r < NU && pi == pi) { s.sel_desc[r] = i; s.p_desc[r] = pi; }
    }
    __syncthreads();
    if (t == 0) {
        float wsum = 0.0f;
        for (int k = 0; k < NU; k++) wsum = __fadd_rn(wsum, s.p_desc[k]);
        if (wsum < 6.103515625e-5f) wsum = 6.103515625e-5f;
        for (int k = 0; k < NU; k++) s.p_desc[k] = __fdiv_rn(s.p_desc[k], wsum);
        /* ascending-id slots and combine weights w * dexps_scale[e] (CF:8709) */
        for (int k = 0; k < NU; k++) {
            const int e = s.sel_desc[k]; int slot = 0;
            for (int j = 0; j < NU; j++) slot += (s.sel_desc[j] < e);
            s.sel_asc[slot] = e; s.cw[slot] = __fmul_rn(s.p_desc[k], __ldg(dscale + e));
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kThreads, 1) k_moe_decode_stack(SpDecodeArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const SpDims d = a.d;
    const int G = gridDim.x, b = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;
    const int rows_f_max = (E + G - 1) / G + 1;
    Smem s = carve(smem_raw, d, rows_f_max);
    unsigned bar_target = a.bar_base;

    for (int i = t; i < E; i += kThreads) s.x[i] = a.x_in[i];
    __syncthreads();

    for (int li = 0; li < a.n_layers; li++) {
        if (t < (int)(sizeof(SpLayerDev) / 8))
            reinterpret_cast<unsigned long long *>(s.L)[t] = reinterpret_cast<const unsigned long long *>(a.layers + a.layer_first + li)[t];
        __syncthreads();
        const SpLayerDev &L = *s.L;
        /* ---------------- A: norms of x ---------------- */
        {
            const float scale = rms_scale_from(block_sumsq(s.x, E, s.red), E, d.eps);
            const float *wn = L.ffn_norm, *wp = L.pre_ffw2, *rs = L.router_scale;
            quant_vec(E, s.q_nx, s.s_nx, s.c_nx, [&](int i) { return __fmul_rn(__fmul_rn(s.x[i], scale), __ldg(wn + i)); });
            quant_vec(E, s.q_in, s.s_in, s.c_in, [&](int i) { return __fmul_rn(__fmul_rn(s.x[i], scale), __ldg(wp + i)); });
            for (int i = t; i < E; i += kThreads)
                s.va[i] = __fmul_rn(__fmul_rn(__fmul_rn(s.x[i], scale), d.inv_sqrt_e), __ldg(rs + i));   /* CF:5952-5953 */
            __syncthreads();
        }
        /* ---------------- B: router rows + shared gate/up pairs ---------------- */
        {
            const int r0 = (int)((long long)b * NE / G), r1 = (int)((long long)(b + 1) * NE / G);
            const int p0 = (int)((long long)b * FFS / G), p1 = (int)((long long)(b + 1) * FFS / G);
            const int nr = r1 - r0, np = p1 - p0, n32 = E >> 5;
            const Act act{reinterpret_cast<const int4 *>(s.q_nx), s.s_nx, s.c_nx};
            const size_t rb = (size_t)E / 2;
            for (int u = warp; u < nr + np; u += kWarps) {
                if (u < nr) {
                    const int r = r0 + u;
                    float l = router_row(L.router_w + (size_t)r * E, s.va, E, lane);
                    if (lane == 0) { if (L.router_bias) l = __fadd_rn(l, __ldg(L.router_bias + r)); a.logits[r] = l; }
                } else {
                    const int c = p0 + (u - nr);
                    float h;
                    NIT_SWITCH(n32, h = pair_gelu<NIT>(L.sg_codes + c * rb, L.sg_bs + (size_t)c * n32,
                                                       L.su_codes + c * rb, L.su_bs + (size_t)c * n32, n32, lane, act));
                    if (lane == 0) a.hd[c] = h;
                }
            }
        }
        bar_target += G;
        if (!grid_barrier(a.bar, bar_target, a.status, s.flag)) return;
        /* ---------------- C: top-k, quantise hd ---------------- */
        topk_block(a.logits, d, L.dexps_scale, s, a.status);
        if (b == 0 && t < NU) {
            if (a.sel_out) a.sel_out[(size_t)li * NU + t] = s.sel_desc[t];
            if (a.wts_out) a.wts_out[(size_t)li * NU + t] = s.p_desc[t];
        }
        quant_vec(FFS, s.q_hd, s.s_hd, s.c_hd, [&](int i) { return ld_cg_f32(a.hd + i); });
        __syncthreads();
        /* ---------------- D: routed gate|up pairs + shared down rows ---------------- */
        {
            const int NP = NU * FFE;
            const int p0 = (int)((long long)b * NP / G), p1 = (int)((long long)(b + 1) * NP / G);
            const int j0 = (int)((long long)b * E / G), j1 = (int)((long long)(b + 1) * E / G);
            const int np = p1 - p0, nj = j1 - j0, n32 = E >> 5, n32s = FFS >> 5;
            const Act act_in{reinterpret_cast<const int4 *>(s.q_in), s.s_in, s.c_in};
            const Act act_hd{reinterpret_cast<const int4 *>(s.q_hd), s.s_hd, s.c_hd};
            const size_t rb = (size_t)E / 2, rbs = (size_t)FFS / 2;
            for (int u = warp; u < np + nj; u += kWarps) {
                if (u < np) {
                    const int pu = p0 + u, slot = pu / FFE, c = pu - slot * FFE;
                    const size_t grow = (size_t)s.sel_asc[slot] * 2 * FFE + c, urow = grow + FFE;
                    float h;
                    NIT_SWITCH(n32, h = pair_gelu<NIT>(L.gu_codes + grow * rb, L.gu_bs + grow * n32,
                                                       L.gu_codes + urow * rb, L.gu_bs + urow * n32, n32, lane, act_in));
                    if (lane == 0) a.h[pu] = h;
                } else {
                    const int j = j0 + (u - np);
                    float o;
                    NIT_SWITCH(n32s, o = single_row<NIT>(L.sd_codes + j * rbs, L.sd_bs + (size_t)j * n32s, n32s, lane, act_hd));
                    if (lane == 0) a.dn[j] = o;
                }
            }
        }
        bar_target += G;
        if (!grid_barrier(a.bar, bar_target, a.status, s.flag)) return;
        /* ---------------- E: quantise the expert activations ---------------- */
        quant_vec(NU * FFE, s.q_h, s.s_h, s.c_h, [&](int i) { return ld_cg_f32(a.h + i); });
        __syncthreads();
        /* ---------------- F: routed down rows + ordered combine ---------------- */
        {
            const int j0 = (int)((long long)b * E / G), j1 = (int)((long long)(b + 1) * E / G);
            const int nj = j1 - j0, n32 = FFE >> 5, blk = FFE >> 4;
            const size_t rb = (size_t)FFE / 2;
            for (int u = warp; u < nj * NU; u += kWarps) {
                const int jj = u / NU, slot = u - jj * NU;
                const size_t row = (size_t)s.sel_asc[slot] * E + (j0 + jj);
                const Act act{reinterpret_cast<const int4 *>(s.q_h) + (size_t)slot * blk, s.s_h + (size_t)slot * blk, s.c_h + (size_t)slot * blk};
                float o;
                NIT_SWITCH(n32, o = single_row<NIT>(L.dn_codes + row * rb, L.dn_bs + row * n32, n32, lane, act));
                if (lane == 0) s.out[slot * rows_f_max + jj] = o;
            }
            __syncthreads();
            for (int jj = t; jj < nj; jj += kThreads) {           /* k_moe_combine_ord, CF:6071-6077 */
                float acc = 0.0f;
                for (int k = 0; k < NU; k++) acc = __fadd_rn(acc, __fmul_rn(s.cw[k], s.out[k * rows_f_max + jj]));
                a.acc[j0 + jj] = acc;
            }
        }
        bar_target += G;
        if (!grid_barrier(a.bar, bar_target, a.status, s.flag)) return;
        /* ---------------- G: recombine (CF:9014-9019) ---------------- */
        {
            for (int i = t; i < E; i += kThreads) { s.va[i] = ld_cg_f32(a.dn + i); s.vb[i] = ld_cg_f32(a.acc + i); }
            __syncthreads();
            const float sc1 = rms_scale_from(block_sumsq(s.va, E, s.red), E, d.eps);
            const float sc2 = rms_scale_from(block_sumsq(s.vb, E, s.red), E, d.eps);
            for (int i = t; i < E; i += kThreads) {
                const float mlp = __fmul_rn(__fmul_rn(s.va[i], sc1), __ldg(L.post_ffw1 + i));
                const float t1 = __fmul_rn(__fmul_rn(s.vb[i], sc2), __ldg(L.post_ffw2 + i));
                s.va[i] = __fadd_rn(mlp, t1);
            }
            __syncthreads();
            const float sc3 = rms_scale_from(block_sumsq(s.va, E, s.red), E, d.eps);
            for (int i = t; i < E; i += kThreads)
                s.x[i] = __fadd_rn(s.x[i], __fmul_rn(__fmul_rn(s.va[i], sc3), __ldg(L.post_ffw + i)));
            __syncthreads();
        }
    }
    if (b == 0) for (int i = t; i < E; i += kThreads) a.y_out[i] = s.x[i];
}

}  // namespace

size_t sp_decode_smem_bytes(const SpDims &d, int grid) {
    const int rows_f_max = (d.E + grid - 1) / grid + 1;
    size_t o = 0;
    auto take = [&](size_t bytes) { o = (o + bytes + 15) & ~(size_t)15; };
    take(4 * d.E); take(4 * d.E); take(4 * d.E);
    take(d.E); take(d.E); take(d.FFS); take((size_t)d.NU * d.FFE);
    take(4 * (d.E / 16)); take(4 * (d.E / 16)); take(4 * (d.FFS / 16)); take(4 * (size_t)d.NU * (d.FFE / 16));
    take(4 * (d.E / 16)); take(4 * (d.E / 16)); take(4 * (d.FFS / 16)); take(4 * (size_t)d.NU * (d.FFE / 16));
    take(8 * 256); take(4 * d.NE); take(4 * d.NE); take(16); take(sizeof(SpLayerDev)); take(4 * (size_t)d.NU * rows_f_max);
    take(4 * SP_MAX_NU); take(4 * SP_MAX_NU); take(4 * SP_MAX_NU); take(4 * SP_MAX_NU);
    return o;
}

int sp_decode_threads() { return kThreads; }
int sp_decode_barriers_per_layer() { return 3; }

cudaError_t sp_decode_prepare(size_t smem, int *max_grid) {
    cudaError_t e = cudaFuncSetAttribute(k_moe_decode_stack, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    int per_sm = 0, dev = 0, sms = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_moe_decode_stack, kThreads, smem);
    if (e != cudaSuccess) return e;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    *max_grid = per_sm > 0 ? sms : 0;              /* one CTA per SM */
    return cudaSuccess;
}

cudaError_t sp_decode_launch(const SpDecodeArgs &args, int grid, size_t smem, cudaStream_t st) {
    SpDecodeArgs a = args;
    void *params[] = {&a};
    return cudaLaunchCooperativeKernel((const void *)k_moe_decode_stack, dim3(grid), dim3(kThreads), params, smem, st);
}
