/* decode_staged.cu — the M=1 decode path with every weight row staged through shared memory.
 *
 * Same cut as decode_graph.cu (three kernels per layer at the three points where every CTA needs
 * every other CTA's results, replayed from one CUDA graph, programmatic dependent launch between
 * them) and the same arithmetic (the reference's decode arithmetic: int8 per-16 activation
 * quantisation, exact integer dots per 16, fp32 scale/accumulate with chunk c in lane c%32 and a
 * shuffle tree; CF:1564-1585, 1688-1713, 6071-6077, 6220-6240, 9014-9019 of
 * src/backends/cuda/cuda_forward.cu). What differs is how the weight bytes travel:
 *
 *   - A CTA's slice of each phase is a handful of contiguous row runs. One thread asks the copy
 *     engine for them (cp.async.bulk, completion counted on mbarriers in shared memory), whole
 *     slices at a time: rows whose address does not depend on the routing are requested before
 *     the kernel waits for its predecessor, routed rows the moment the top-NU selection exists.
 *     The copies run while all 16 warps do the per-layer prologue (norms, quantisation, top-k),
 *     so the prologue no longer delays the weight stream and no warp holds registers for loads in
 *     flight.
 *   - The warps then read rows from shared memory. A lane keeps its share of the quantised
 *     activation in registers across the rows it computes; rows are reduced two or eight at a
 *     time with a butterfly that performs exactly the additions of the reference's shuffle tree
 *     (same pairs, same tree shape), so results stay bit-identical.
 *
 * The single-pass layout needs a CTA's slice of every phase to fit shared memory at once
 * (sp_staged_fits); other geometries use decode_graph.cu.
 */
#include "common.cuh"
#include "decode.cuh"

namespace {

constexpr int kT = 512;                 /* threads per CTA */
constexpr int kW = kT / 32;
constexpr unsigned kSpin = 1u << 21;    /* polls before a wait on a copy gives up */
constexpr int kGuBars = 4;              /* the routed gate|up slice lands in up to 4 parts */
constexpr int kDnBars = 4;              /* the routed down slice too */

struct SArgs {
    SpLayerDev L;
    SpDims d;
    const float *x_prev;      /* residual entering this layer (K1: before the previous layer's recombine is added) */
    float *x_cur;             /* K1 writes the residual entering this layer (CTA 0) */
    SpGraphScratch s;
    int32_t *sel_out; float *wts_out;
    int first;                /* K1: no previous layer to recombine */
    SpLayerDev Ln;            /* the next layer (K3 asks L2 for its routing-independent rows) */
    int has_next;
    unsigned flags;           /* SP_STAGED_* */
    long long *stamps;        /* [3][8] device time stamps of CTA 0, or NULL */
};

#define STAMP(k, i) do { if (a.stamps && blockIdx.x == 0 && threadIdx.x == 0) { long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); a.stamps[(k) * 8 + (i)] = t_; } } while (0)

/* ---------------------------------------------------------------- PTX helpers */
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, unsigned bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned mbar_try(uint32_t bar, unsigned parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

/* Waits for the copies counted on `bar` (each barrier is used once per launch: parity 0). Bounded:
 * when the limit runs out the error word is set, every later wait of this CTA falls through, and
 * the kernel runs to its end on whatever the buffers hold. */
__device__ __forceinline__ void bar_wait(uint32_t bar, volatile int *abort_flag, int *status) {
    if (mbar_try(bar, 0)) return;
    for (unsigned i = 0; i < kSpin; i++) {
        if (mbar_try(bar, 0)) return;
        if ((i & 255u) == 255u && *abort_flag) return;
    }
    *abort_flag = 1;
    atomicExch(status, SP_KERR_BARRIER_TIMEOUT);
}

/* ask L2 for [p, p+bytes): one 128-byte line per lane per instruction */
__device__ __forceinline__ void l2_prefetch(const void *p, int bytes, int lane) {
    const unsigned char *b = reinterpret_cast<const unsigned char *>(p);
    for (int off = lane * 128; off < bytes; off += 32 * 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(b + off));
}

/* A bulk copy needs 16-byte aligned ends; a run of block-scale rows starts on any even byte. The
 * span is the enclosing aligned range: `delta` bytes of it precede the first row. It never leaves
 * the tensor's 256-byte aligned slot of the arena. */
struct Span { const unsigned char *src; unsigned bytes, delta; };
__device__ __forceinline__ Span make_span(const void *p, unsigned nbytes) {
    const uintptr_t addr = (uintptr_t)p;
    const unsigned delta = (unsigned)(addr & 15u);
    return Span{reinterpret_cast<const unsigned char *>(addr - delta), (delta + nbytes + 15u) & ~15u, delta};
}

/* ---------------------------------------------------------------- shared-memory layouts (host and device agree) */
__host__ __device__ inline unsigned up16(unsigned v) { return (v + 15u) & ~15u; }
__host__ __device__ inline int cdiv(int a, int b) { return (a + b - 1) / b; }

struct Ctl {
    unsigned long long bar[8];
    int abort;
    int sel_asc[SP_MAX_NU]; float cw[SP_MAX_NU]; int sel_desc[SP_MAX_NU]; float p_desc[SP_MAX_NU];
    unsigned gs_off[2], us_off[2];          /* K2: where the two runs' gate / up scale rows start */
    unsigned sdelta[SP_MAX_NU];             /* K3: bytes before the first scale row of each slot's span */
};

struct Lay1 { unsigned ctl, red, va, vb, ri, q_nx, q_in, s_nx, s_in, c_nx, c_in, st_r, st_gc, st_uc, st_gs, st_us, total; };
__host__ __device__ inline Lay1 lay1(const SpDims &d, int G) {
    Lay1 L; unsigned o = 0;
    auto take = [&](unsigned bytes) { const unsigned at = o; o = up16(o + bytes); return at; };
    const unsigned E = d.E, nb = E / 16, nr = cdiv(d.NE, G), np = cdiv(d.FFS, G), rb = E / 2, sb = E / 16;
    L.ctl = take(sizeof(Ctl)); L.red = take(64 * 8);
    L.va = take(4 * E); L.vb = take(4 * E); L.ri = take(4 * E);
    L.q_nx = take(E); L.q_in = take(E);
    L.s_nx = take(4 * nb); L.s_in = take(4 * nb); L.c_nx = take(4 * nb); L.c_in = take(4 * nb);
    o = (o + 127u) & ~127u;
    L.st_r = take(nr * 4 * E); L.st_gc = take(np * rb); L.st_uc = take(np * rb);
    L.st_gs = take(np * sb + 32); L.st_us = take(np * sb + 32);
    L.total = o;
    return L;
}
struct Lay2 { unsigned ctl, red, ex, lg, p, dsc, wmax, q_in, s_in, c_in, q_hd, s_hd, c_hd, st_sd, st_sds, st_gc, st_uc, st_gs, st_us, total; };
__host__ __device__ inline Lay2 lay2(const SpDims &d, int G) {
    Lay2 L; unsigned o = 0;
    auto take = [&](unsigned bytes) { const unsigned at = o; o = up16(o + bytes); return at; };
    const unsigned E = d.E, NE = d.NE, FFS = d.FFS, nj = cdiv(d.E, G), nP = cdiv(d.NU * d.FFE, G);
    L.ctl = take(sizeof(Ctl)); L.red = take(64 * 8); L.ex = take(8 * NE);
    L.lg = take(4 * NE); L.p = take(4 * NE); L.dsc = take(4 * NE); L.wmax = take(4 * 32);
    L.q_in = take(E); L.s_in = take(4 * (E / 16)); L.c_in = take(4 * (E / 16));
    L.q_hd = take(FFS); L.s_hd = take(4 * (FFS / 16)); L.c_hd = take(4 * (FFS / 16));
    o = (o + 127u) & ~127u;
    L.st_sd = take(nj * (FFS / 2)); L.st_sds = take(nj * (FFS / 16) + 32);
    L.st_gc = take(nP * (E / 2)); L.st_uc = take(nP * (E / 2));
    L.st_gs = take(nP * (E / 16) + 64); L.st_us = take(nP * (E / 16) + 64);
    L.total = o;
    return L;
}
struct Lay3 { unsigned ctl, q_h, s_h, c_h, out, st_c, st_s, span_max, total; };
__host__ __device__ inline Lay3 lay3(const SpDims &d, int G) {
    Lay3 L; unsigned o = 0;
    auto take = [&](unsigned bytes) { const unsigned at = o; o = up16(o + bytes); return at; };
    const unsigned NU = d.NU, FFE = d.FFE, nj = cdiv(d.E, G), nblk = NU * FFE / 16;
    L.ctl = take(sizeof(Ctl));
    L.q_h = take(NU * FFE); L.s_h = take(4 * nblk); L.c_h = take(4 * nblk);
    L.out = take(4 * NU * nj);
    o = (o + 127u) & ~127u;
    L.st_c = take(NU * nj * (FFE / 2));
    L.span_max = up16(nj * (FFE / 16) + 30);
    L.st_s = take(NU * L.span_max);
    L.total = o;
    return L;
}

/* ---------------------------------------------------------------- small math */
__device__ __forceinline__ float rms_scale(double ss, double inv_n, float eps) {
    const float ms = (float)(ss * inv_n);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
}
/* sum over the CTA in double: shuffle tree per warp, warp totals in warp order. Each call site
 * uses its own 16 slots of `sh`, so one barrier per sum is enough. */
__device__ __forceinline__ double cta_sum(double v, double *sh16) {
    v = warp_sum_f64(v);
    if ((threadIdx.x & 31) == 0) sh16[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int w = 0; w < kW; w++) r += sh16[w];
    return r;
}
__device__ __forceinline__ float warp_tree(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}
/* Two rows' lane partials reduced together. Level 16 keeps row 0 in the lower half-warp and row 1
 * in the upper one; every level adds the same pairs as the shuffle-down tree of
 * k_gemv_q4b_dp4a_v2 (CF:1709-1711), so lane 0's two results are bit-identical to two such trees. */
__device__ __forceinline__ void tree2(float f0, float f1, int lane, float &r0, float &r1) {
    const bool hi = (lane & 16) != 0;
    float v = (hi ? f1 : f0) + __shfl_xor_sync(0xffffffffu, hi ? f0 : f1, 16);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    r0 = v; r1 = __shfl_sync(0xffffffffu, v, 16);
}
/* Eight rows at once: after the levels 16, 8 and 4 each group of four lanes owns one row; the
 * lane's row is ((lane>>4)&1)*4 + ((lane>>3)&1)*2 + ((lane>>2)&1). Same pairs, same tree. */
__device__ __forceinline__ float tree8(const float (&f)[8], int lane) {
    const bool b16 = (lane & 16) != 0, b8 = (lane & 8) != 0, b4 = (lane & 4) != 0;
    float g[4], h[2];
#pragma unroll
    for (int r = 0; r < 4; r++) g[r] = (b16 ? f[r + 4] : f[r]) + __shfl_xor_sync(0xffffffffu, b16 ? f[r] : f[r + 4], 16);
#pragma unroll
    for (int r = 0; r < 2; r++) h[r] = (b8 ? g[r + 2] : g[r]) + __shfl_xor_sync(0xffffffffu, b8 ? g[r] : g[r + 2], 8);
    float k = (b4 ? h[1] : h[0]) + __shfl_xor_sync(0xffffffffu, b4 ? h[0] : h[1], 4);
    k += __shfl_xor_sync(0xffffffffu, k, 2);
    k += __shfl_xor_sync(0xffffffffu, k, 1);
    return k;
}

/* ---------------------------------------------------------------- rows from shared memory */
/* this lane's share of one quantised activation vector: chunks c = lane + 32*i */
template <int NIT> struct ActR { int4 qa[NIT], qb[NIT]; float2 sx[NIT]; int2 cr[NIT]; };
template <int NIT>
__device__ __forceinline__ void act_load(ActR<NIT> &r, const signed char *q, const float *sx, const int *corr, int n32, int lane) {
    const int4 *q4 = reinterpret_cast<const int4 *>(q);
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) {
            r.qa[i] = q4[2 * c]; r.qb[i] = q4[2 * c + 1];
            r.sx[i] = *reinterpret_cast<const float2 *>(sx + 2 * c);
            r.cr[i] = *reinterpret_cast<const int2 *>(corr + 2 * c);
        } else {
            r.qa[i] = make_int4(0, 0, 0, 0); r.qb[i] = r.qa[i]; r.sx[i] = make_float2(0.0f, 0.0f); r.cr[i] = make_int2(0, 0);
        }
    }
}
/* lane partial of one Q4B row (codes and f16 block scales in shared memory) against the lane's
 * activation registers: facc = fma(scale, fma(a0, sx0, a1*sx1), facc) over the lane's chunks in
 * increasing c (CF:1697-1708) */
template <int NIT>
__device__ __forceinline__ float row_part(const unsigned char *codes, const unsigned char *scales, const ActR<NIT> &r, int n32, int lane) {
    float facc = 0.0f;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) {
            const int4 w = *reinterpret_cast<const int4 *>(codes + 16 * c);
            const unsigned short sc = *reinterpret_cast<const unsigned short *>(scales + 2 * c);
            int a0, a1;
            q4b_chunk_dot(w, r.qa[i], r.qb[i], r.cr[i].x, r.cr[i].y, a0, a1);
            facc = __fmaf_rn(h2f(sc), __fmaf_rn((float)a0, r.sx[i].x, __fmul_rn((float)a1, r.sx[i].y)), facc);
        }
    }
    return facc;
}
/* the same with the activation read from shared memory per chunk (rows whose activation changes
 * from row to row) */
template <int NIT>
__device__ __forceinline__ float row_part_s(const unsigned char *codes, const unsigned char *scales, const signed char *q, const float *sx,
                                            const int *corr, int n32, int lane) {
    const int4 *q4 = reinterpret_cast<const int4 *>(q);
    float facc = 0.0f;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) {
            const int4 w = *reinterpret_cast<const int4 *>(codes + 16 * c);
            const unsigned short sc = *reinterpret_cast<const unsigned short *>(scales + 2 * c);
            const int2 cr = *reinterpret_cast<const int2 *>(corr + 2 * c);
            const float2 s2 = *reinterpret_cast<const float2 *>(sx + 2 * c);
            int a0, a1;
            q4b_chunk_dot(w, q4[2 * c], q4[2 * c + 1], cr.x, cr.y, a0, a1);
            facc = __fmaf_rn(h2f(sc), __fmaf_rn((float)a0, s2.x, __fmul_rn((float)a1, s2.y)), facc);
        }
    }
    return facc;
}
/* 16 floats at p (16-byte aligned, written by another kernel) -> one quantised block */
__device__ __forceinline__ void quant_from_global(const float *p, int4 *dst, float *sx, int *corr) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 4; i++) { const float4 f = __ldcg(reinterpret_cast<const float4 *>(p) + i); v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w; }
    quant_block16_store(v, dst, sx, corr);
}

/* ---------------------------------------------------------------- K1: recombine, norms, router rows, shared gate/up
 * KE = elements of an [E] vector per thread; NIT = 32-weight chunks per lane of a row of E columns. */
template <int KE, int NIT>
__global__ void __launch_bounds__(kT, 1) k_ds_router_shared(SArgs a) {
    extern __shared__ __align__(128) unsigned char sm[];
    const SpDims d = a.d;
    const int E = d.E, t = threadIdx.x, lane = t & 31, warp = t >> 5, G = gridDim.x, b = blockIdx.x;
    const Lay1 ly = lay1(d, G);
    Ctl *ctl = reinterpret_cast<Ctl *>(sm + ly.ctl);
    double *red = reinterpret_cast<double *>(sm + ly.red);
    float *va = reinterpret_cast<float *>(sm + ly.va), *vb = reinterpret_cast<float *>(sm + ly.vb), *ri = reinterpret_cast<float *>(sm + ly.ri);
    signed char *q_nx = reinterpret_cast<signed char *>(sm + ly.q_nx), *q_in = reinterpret_cast<signed char *>(sm + ly.q_in);
    float *s_nx = reinterpret_cast<float *>(sm + ly.s_nx), *s_in = reinterpret_cast<float *>(sm + ly.s_in);
    int *c_nx = reinterpret_cast<int *>(sm + ly.c_nx), *c_in = reinterpret_cast<int *>(sm + ly.c_in);
    const SpLayerDev &L = a.L;
    const int r0 = (int)((long long)b * d.NE / G), nr = (int)((long long)(b + 1) * d.NE / G) - r0;
    const int p0 = (int)((long long)b * d.FFS / G), np = (int)((long long)(b + 1) * d.FFS / G) - p0;
    const unsigned rb = (unsigned)E >> 1, sb = (unsigned)E >> 4;
    const int n32 = E >> 5;
    const uint32_t bar_r = smem_u32(&ctl->bar[0]), bar_p = smem_u32(&ctl->bar[1]);
    const Span sg = make_span(reinterpret_cast<const unsigned char *>(L.sg_bs) + (size_t)p0 * sb, (unsigned)np * sb);
    const Span su = make_span(reinterpret_cast<const unsigned char *>(L.su_bs) + (size_t)p0 * sb, (unsigned)np * sb);
    STAMP(0, 0);
    if (t == 0) {
        /* every row of this kernel has a fixed address: all copies start before the predecessor is done */
        mbar_init(bar_r, 1); mbar_init(bar_p, 1); ctl->abort = 0;
        fence_barrier_init();
        if (nr > 0) {
            mbar_expect_tx(bar_r, (unsigned)nr * 4u * (unsigned)E);
            bulk_g2s(sm + ly.st_r, L.router_w + (size_t)r0 * E, (unsigned)nr * 4u * (unsigned)E, bar_r);
        }
        if (np > 0) {
            mbar_expect_tx(bar_p, 2u * (unsigned)np * rb + sg.bytes + su.bytes);
            bulk_g2s(sm + ly.st_gc, L.sg_codes + (size_t)p0 * rb, (unsigned)np * rb, bar_p);
            bulk_g2s(sm + ly.st_uc, L.su_codes + (size_t)p0 * rb, (unsigned)np * rb, bar_p);
            bulk_g2s(sm + ly.st_gs, sg.src, sg.bytes, bar_p);
            bulk_g2s(sm + ly.st_us, su.src, su.bytes, bar_p);
        }
    }
    /* norm weights do not depend on the previous kernel either */
    const double inv_n = 1.0 / (double)E;
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
    __syncthreads();                                     /* barriers initialised before any warp can wait on one */
    pdl_launch();
    pdl_wait();
    STAMP(0, 1);
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
        const float sc1 = rms_scale(s1, inv_n, d.eps), sc2 = rms_scale(s2, inv_n, d.eps);
        double p3 = 0.0;
#pragma unroll
        for (int k = 0; k < KE; k++) {
            const float mlp = __fmul_rn(__fmul_rn(dn[k], sc1), w1[k]);
            const float t1 = __fmul_rn(__fmul_rn(ac[k], sc2), w2[k]);
            dn[k] = __fadd_rn(mlp, t1); p3 += (double)dn[k] * dn[k];
        }
        const float sc3 = rms_scale(cta_sum(p3, red + 32), inv_n, d.eps);
#pragma unroll
        for (int k = 0; k < KE; k++) x[k] = __fadd_rn(x[k], __fmul_rn(__fmul_rn(dn[k], sc3), w3[k]));
    }
    if (b == 0) {
#pragma unroll
        for (int k = 0; k < KE; k++) { const int i = t + kT * k; if (i < E) a.x_cur[i] = x[k]; }
    }
    STAMP(0, 2);
    /* norms of x (CF:8347, 8402-8404, 8425) and the router input (CF:5952-5953) */
    double part = 0.0;
#pragma unroll
    for (int k = 0; k < KE; k++) part += (double)x[k] * x[k];
    const float scale = rms_scale(cta_sum(part, red + 48), inv_n, d.eps);
    STAMP(0, 5);
#pragma unroll
    for (int k = 0; k < KE; k++) {
        const int i = t + kT * k;
        if (i < E) {
            const float xs = __fmul_rn(x[k], scale);
            va[i] = __fmul_rn(xs, wn[k]); vb[i] = __fmul_rn(xs, wp[k]);
            ri[i] = __fmul_rn(__fmul_rn(xs, d.inv_sqrt_e), rs[k]);
        }
    }
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
    STAMP(0, 6);
    if (b == 0) {                                        /* the routed experts' input, for K2 */
        for (int i = t; i < nb; i += kT) { reinterpret_cast<int4 *>(a.s.in_q)[i] = reinterpret_cast<const int4 *>(q_in)[i]; a.s.in_s[i] = s_in[i]; a.s.in_c[i] = c_in[i]; }
    }
    STAMP(0, 3);
    if (a.flags & SP_STAGED_PREFETCH_SD) {               /* the next kernel's routing-independent rows: ask L2 for them now */
        const int j0 = (int)((long long)b * E / G), nj = (int)((long long)(b + 1) * E / G) - j0;
        if (warp == kW - 1) { l2_prefetch(L.sd_codes + (size_t)j0 * (d.FFS / 2), nj * (d.FFS / 2), lane); l2_prefetch(reinterpret_cast<const unsigned char *>(L.sd_bs) + (size_t)j0 * (d.FFS / 16), nj * (d.FFS / 16), lane); }
    }
    /* rows: shared gate/up pairs first (warps 0..), router rows after them */
    ActR<NIT> act;
    act_load<NIT>(act, q_nx, s_nx, c_nx, n32, lane);
    const int total = np + nr;
    for (int u = warp; u < total; u += kW) {
        if (u < np) {
            bar_wait(bar_p, &ctl->abort, a.s.status);
            const float g = row_part<NIT>(sm + ly.st_gc + (size_t)u * rb, sm + ly.st_gs + sg.delta + (size_t)u * sb, act, n32, lane);
            const float up = row_part<NIT>(sm + ly.st_uc + (size_t)u * rb, sm + ly.st_us + su.delta + (size_t)u * sb, act, n32, lane);
            float gt, ut;
            tree2(g, up, lane, gt, ut);
            if (lane == 0) a.s.hd[p0 + u] = gelu_mul(gt, ut);
        } else {
            /* fp32 router row, fixed order: lane l takes the float4 groups l, l+32, ... in order, then the tree */
            bar_wait(bar_r, &ctl->abort, a.s.status);
            const int r = u - np;
            const float4 *wrow = reinterpret_cast<const float4 *>(sm + ly.st_r + (size_t)r * 4u * (unsigned)E);
            const float4 *xin = reinterpret_cast<const float4 *>(ri);
            float acc = 0.0f;
#pragma unroll 4
            for (int q = lane; q < (E >> 2); q += 32) {
                const float4 w = wrow[q], xv = xin[q];
                acc = __fmaf_rn(w.x, xv.x, acc); acc = __fmaf_rn(w.y, xv.y, acc); acc = __fmaf_rn(w.z, xv.z, acc); acc = __fmaf_rn(w.w, xv.w, acc);
            }
            acc = warp_tree(acc);
            if (lane == 0) { if (L.router_bias) acc = __fadd_rn(acc, __ldg(L.router_bias + r0 + r)); a.s.logits[r0 + r] = acc; }
        }
    }
    STAMP(0, 4);
}

/* ---------------------------------------------------------------- K2: top-NU, shared down, routed gate|up */
template <int NIT_E, int NIT_S>
__global__ void __launch_bounds__(kT, 1) k_ds_experts_up(SArgs a) {
    extern __shared__ __align__(128) unsigned char sm[];
    const SpDims d = a.d;
    const int E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, G = gridDim.x, b = blockIdx.x;
    const Lay2 ly = lay2(d, G);
    Ctl *ctl = reinterpret_cast<Ctl *>(sm + ly.ctl);
    double *red = reinterpret_cast<double *>(sm + ly.red), *ex = reinterpret_cast<double *>(sm + ly.ex);
    float *lg = reinterpret_cast<float *>(sm + ly.lg), *p = reinterpret_cast<float *>(sm + ly.p), *dsc = reinterpret_cast<float *>(sm + ly.dsc);
    float *wmax = reinterpret_cast<float *>(sm + ly.wmax);
    signed char *q_in = reinterpret_cast<signed char *>(sm + ly.q_in), *q_hd = reinterpret_cast<signed char *>(sm + ly.q_hd);
    float *s_in = reinterpret_cast<float *>(sm + ly.s_in), *s_hd = reinterpret_cast<float *>(sm + ly.s_hd);
    int *c_in = reinterpret_cast<int *>(sm + ly.c_in), *c_hd = reinterpret_cast<int *>(sm + ly.c_hd);
    const SpLayerDev &L = a.L;
    const int j0 = (int)((long long)b * E / G), nj = (int)((long long)(b + 1) * E / G) - j0;
    const int NP = NU * FFE;
    const int P0 = (int)((long long)b * NP / G), nP = (int)((long long)(b + 1) * NP / G) - P0;
    const unsigned rbE = (unsigned)E >> 1, sbE = (unsigned)E >> 4, rbS = (unsigned)FFS >> 1, sbS = (unsigned)FFS >> 4;
    const int n32 = E >> 5, n32s = FFS >> 5;
    const uint32_t bar_sd = smem_u32(&ctl->bar[0]);
    const Span sds = make_span(reinterpret_cast<const unsigned char *>(L.sd_bs) + (size_t)j0 * sbS, (unsigned)nj * sbS);
    /* the routed pairs of this CTA lie in at most two expert slots: run 0 = n0 pairs of slot0 from
     * column c0, run 1 = the rest, from column 0 of the next slot. They land in up to kGuBars parts
     * of SG pairs each (a multiple of the 16 pairs one pass of the warps consumes). */
    const int slot0 = nP > 0 ? P0 / FFE : 0, c0 = P0 - slot0 * FFE;
    const int n0 = nP < FFE - c0 ? nP : FFE - c0;
    const int SG = 16 * cdiv(cdiv(nP > 0 ? nP : 1, 16), kGuBars);
    STAMP(1, 0);
    if (t == 0) {
        for (int i = 0; i < 1 + kGuBars; i++) mbar_init(smem_u32(&ctl->bar[i]), 1);
        ctl->abort = 0;
        fence_barrier_init();
        if (nj > 0) {                                     /* shared-expert down rows: fixed addresses */
            mbar_expect_tx(bar_sd, (unsigned)nj * rbS + sds.bytes);
            bulk_g2s(sm + ly.st_sd, L.sd_codes + (size_t)j0 * rbS, (unsigned)nj * rbS, bar_sd);
            bulk_g2s(sm + ly.st_sds, sds.src, sds.bytes, bar_sd);
        }
    }
    for (int i = t; i < NE; i += kT) dsc[i] = __ldg(L.dexps_scale + i);
    __syncthreads();
    pdl_launch();
    pdl_wait();
    STAMP(1, 1);
    /* everything this CTA needs from the previous kernel, requested in one batch */
    float mx = -INFINITY; int bad = 0;
    for (int i = t; i < NE; i += kT) { const float l = __ldcg(a.s.logits + i); lg[i] = l; if (l != l) bad = 1; mx = fmaxf(mx, l); }
    for (int i = t; i < E / 16; i += kT) { reinterpret_cast<int4 *>(q_in)[i] = __ldcg(reinterpret_cast<const int4 *>(a.s.in_q) + i); s_in[i] = __ldcg(a.s.in_s + i); c_in[i] = __ldcg(a.s.in_c + i); }
    const int nbh = FFS >> 4, bqh = kT - 1 - t;          /* the LAST threads quantise hd (one block each); the first ones run the softmax */
    float hv[16];
    if (bqh < nbh) {
#pragma unroll
        for (int i = 0; i < 4; i++) { const float4 f = __ldcg(reinterpret_cast<const float4 *>(a.s.hd + 16 * bqh) + i); hv[4 * i] = f.x; hv[4 * i + 1] = f.y; hv[4 * i + 2] = f.z; hv[4 * i + 3] = f.w; }
    }
    /* moe_topk_host (CF:6220-6240): double softmax, rank by (p descending, id ascending), clamp, renormalise */
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); bad |= __shfl_xor_sync(0xffffffffu, bad, o); }
    if (lane == 0) wmax[warp] = mx;
    if (bad && lane == 0) atomicExch(a.s.status, SP_KERR_NAN_ROUTER);
    if (t < SP_MAX_NU) { ctl->sel_desc[t] = t < NE ? t : 0; ctl->p_desc[t] = 0.0f; }
    __syncthreads();
    STAMP(1, 5);
    mx = wmax[0];
#pragma unroll
    for (int w = 1; w < kW; w++) mx = fmaxf(mx, wmax[w]);
    double part = 0.0;
    for (int i = t; i < NE; i += kT) { const double e = exp((double)lg[i] - (double)mx); ex[i] = e; part += e; }
    if (bqh < nbh) quant_block16_store(hv, reinterpret_cast<int4 *>(q_hd) + bqh, s_hd + bqh, c_hd + bqh);
    const double sum = cta_sum(part, red);
    const double rsum = 1.0 / sum;
    for (int i = t; i < NE; i += kT) p[i] = (float)(ex[i] * rsum);
    __syncthreads();
    STAMP(1, 6);
    for (int i0 = 0; i0 < NE; i0 += kT / 4) {            /* four threads share one candidate's rank count */
        const int i = i0 + (t >> 2), qt = t & 3;
        const bool live = i < NE;
        const float pi = live ? p[i] : 0.0f;
        int r = 0;
        if (live) {
            const int ja = (int)((long long)qt * NE / 4), jb = (int)((long long)(qt + 1) * NE / 4);
            for (int j = ja; j < jb; j++) { const float pj = p[j]; r += (pj > pi) || (pj == pi && j < i); }
        }
        r += __shfl_xor_sync(0xffffffffu, r, 1);
        r += __shfl_xor_sync(0xffffffffu, r, 2);
        if (live && qt == 0 && r < NU && pi == pi) { ctl->sel_desc[r] = i; ctl->p_desc[r] = pi; }
    }
    __syncthreads();
    STAMP(1, 7);
    if (warp == 0) {
        float wnorm = 0.0f; int e = 0, slot = 0;
        if (lane < NU) {
            float ws = 0.0f;
            for (int k = 0; k < NU; k++) ws = __fadd_rn(ws, ctl->p_desc[k]);
            if (ws < 6.103515625e-5f) ws = 6.103515625e-5f;
            e = ctl->sel_desc[lane];
            wnorm = __fdiv_rn(ctl->p_desc[lane], ws);
            for (int j = 0; j < NU; j++) slot += (ctl->sel_desc[j] < e);
        }
        __syncwarp();
        if (lane < NU) { ctl->sel_asc[slot] = e; ctl->cw[slot] = __fmul_rn(wnorm, dsc[e]); ctl->p_desc[lane] = wnorm; }
        __syncwarp();
        if (lane == 0 && nP > 0) {                        /* the selection exists: start the routed rows at once */
            const int e0 = ctl->sel_asc[slot0], n1 = nP - n0, e1 = n1 > 0 ? ctl->sel_asc[slot0 + 1] : e0;
            const size_t rg0 = (size_t)e0 * 2 * FFE + c0, rg1 = (size_t)e1 * 2 * FFE;
            const unsigned char *bs = reinterpret_cast<const unsigned char *>(L.gu_bs);
            const Span g0 = make_span(bs + rg0 * sbE, (unsigned)n0 * sbE), u0 = make_span(bs + (rg0 + FFE) * sbE, (unsigned)n0 * sbE);
            const Span g1 = make_span(bs + rg1 * sbE, (unsigned)n1 * sbE), u1 = make_span(bs + (rg1 + FFE) * sbE, (unsigned)n1 * sbE);
            ctl->gs_off[0] = ly.st_gs + g0.delta; ctl->gs_off[1] = ly.st_gs + g0.bytes + g1.delta;
            ctl->us_off[0] = ly.st_us + u0.delta; ctl->us_off[1] = ly.st_us + u0.bytes + u1.delta;
            const int nsub = cdiv(nP, SG);
            for (int g = 0; g < nsub; g++) {
                const uint32_t bar = smem_u32(&ctl->bar[1 + g]);
                const int a0 = g * SG, a1 = (a0 + SG < nP) ? a0 + SG : nP;
                unsigned bytes = 2u * (unsigned)(a1 - a0) * rbE;
                if (g == 0) bytes += g0.bytes + u0.bytes + (n1 > 0 ? g1.bytes + u1.bytes : 0u);
                mbar_expect_tx(bar, bytes);
                if (a0 < n0) {                             /* the part of this range in run 0 */
                    const int e_ = a1 < n0 ? a1 : n0;
                    const unsigned cb = (unsigned)(e_ - a0) * rbE;
                    bulk_g2s(sm + ly.st_gc + (size_t)a0 * rbE, L.gu_codes + (rg0 + a0) * rbE, cb, bar);
                    bulk_g2s(sm + ly.st_uc + (size_t)a0 * rbE, L.gu_codes + (rg0 + FFE + a0) * rbE, cb, bar);
                }
                if (a1 > n0) {                             /* the part in run 1 */
                    const int s_ = a0 > n0 ? a0 : n0;
                    const unsigned cb = (unsigned)(a1 - s_) * rbE;
                    bulk_g2s(sm + ly.st_gc + (size_t)s_ * rbE, L.gu_codes + (rg1 + (s_ - n0)) * rbE, cb, bar);
                    bulk_g2s(sm + ly.st_uc + (size_t)s_ * rbE, L.gu_codes + (rg1 + FFE + (s_ - n0)) * rbE, cb, bar);
                }
                if (g == 0) {
                    bulk_g2s(sm + ly.st_gs, g0.src, g0.bytes, bar);
                    bulk_g2s(sm + ly.st_us, u0.src, u0.bytes, bar);
                    if (n1 > 0) { bulk_g2s(sm + ly.st_gs + g0.bytes, g1.src, g1.bytes, bar); bulk_g2s(sm + ly.st_us + u0.bytes, u1.src, u1.bytes, bar); }
                }
            }
        }
    }
    __syncthreads();
    STAMP(1, 2);
    if (b == 0 && t < NU) {
        a.s.sel_asc[t] = ctl->sel_asc[t]; a.s.cw[t] = ctl->cw[t];
        if (a.sel_out) a.sel_out[t] = ctl->sel_desc[t];
        if (a.wts_out) a.wts_out[t] = ctl->p_desc[t];
    }
    if ((a.flags & SP_STAGED_PREFETCH_DN) && nj > 0) {    /* the routed down rows the next kernel will stage: known now */
        for (int sl = warp; sl < NU; sl += kW) {
            const size_t row = (size_t)ctl->sel_asc[sl] * E + j0;
            l2_prefetch(L.dn_codes + row * (FFE / 2), nj * (FFE / 2), lane);
            l2_prefetch(reinterpret_cast<const unsigned char *>(L.dn_bs) + row * (FFE / 16), nj * (FFE / 16), lane);
        }
    }
    /* shared-expert down rows, two per warp pass */
    {
        ActR<NIT_S> act;
        act_load<NIT_S>(act, q_hd, s_hd, c_hd, n32s, lane);
        for (int j = warp; j < nj; j += 2 * kW) {
            const int j2 = j + kW; const bool two = j2 < nj;
            bar_wait(bar_sd, &ctl->abort, a.s.status);
            const float fa = row_part<NIT_S>(sm + ly.st_sd + (size_t)j * rbS, sm + ly.st_sds + sds.delta + (size_t)j * sbS, act, n32s, lane);
            const float fb = two ? row_part<NIT_S>(sm + ly.st_sd + (size_t)j2 * rbS, sm + ly.st_sds + sds.delta + (size_t)j2 * sbS, act, n32s, lane) : 0.0f;
            float oa, ob;
            tree2(fa, fb, lane, oa, ob);
            if (lane == 0) { a.s.dn[j0 + j] = oa; if (two) a.s.dn[j0 + j2] = ob; }
        }
    }
    STAMP(1, 3);
    /* routed gate|up pairs, as their part lands */
    {
        ActR<NIT_E> act;
        act_load<NIT_E>(act, q_in, s_in, c_in, n32, lane);
        for (int i = warp; i < nP; i += kW) {
            bar_wait(smem_u32(&ctl->bar[1 + i / SG]), &ctl->abort, a.s.status);
            if (i >= SG) bar_wait(smem_u32(&ctl->bar[1]), &ctl->abort, a.s.status);       /* the scale rows travel with part 0 */
            const int run = i >= n0, idx = run ? i - n0 : i;
            const float g = row_part<NIT_E>(sm + ly.st_gc + (size_t)i * rbE, sm + ctl->gs_off[run] + (size_t)idx * sbE, act, n32, lane);
            const float up = row_part<NIT_E>(sm + ly.st_uc + (size_t)i * rbE, sm + ctl->us_off[run] + (size_t)idx * sbE, act, n32, lane);
            float gt, ut;
            tree2(g, up, lane, gt, ut);
            if (lane == 0) a.s.h[P0 + i] = gelu_mul(gt, ut);
        }
    }
    STAMP(1, 4);
}

/* ---------------------------------------------------------------- K3: routed down rows + ordered combine */
template <int NIT, int R>
__device__ __forceinline__ void down_round(const unsigned char *sm, const Lay3 &ly, Ctl *ctl, int *status, int u0, int cnt, int nj, int njm, int SGs,
                                           unsigned rb, unsigned sb, int n32, int blk16, int lane, float *out) {
    float f[R]; int sl[R], jr[R];
    const int s_first = u0 / nj, s_last = (u0 + cnt - 1) / nj;
    for (int g = s_first / SGs; g <= s_last / SGs; g++) bar_wait(smem_u32(&ctl->bar[g]), &ctl->abort, status);
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int u = u0 + (r < cnt ? r : cnt - 1);
        sl[r] = u / nj; jr[r] = u - sl[r] * nj;
        const unsigned char *codes = sm + ly.st_c + ((size_t)sl[r] * njm + jr[r]) * rb;
        const unsigned char *scales = sm + ly.st_s + (size_t)sl[r] * ly.span_max + ctl->sdelta[sl[r]] + (size_t)jr[r] * sb;
        f[r] = row_part_s<NIT>(codes, scales, reinterpret_cast<const signed char *>(sm + ly.q_h) + (size_t)sl[r] * blk16 * 16,
                               reinterpret_cast<const float *>(sm + ly.s_h) + (size_t)sl[r] * blk16,
                               reinterpret_cast<const int *>(sm + ly.c_h) + (size_t)sl[r] * blk16, n32, lane);
    }
    if (R == 8) {
        float f8[8];
#pragma unroll
        for (int r = 0; r < 8; r++) f8[r] = f[r < R ? r : 0];
        const float k = tree8(f8, lane);
        const int r = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
        if ((lane & 3) == 0 && r < cnt) {
            const int u = u0 + r, s = u / nj;
            out[s * njm + (u - s * nj)] = k;
        }
    } else {
        float o0, o1;
        tree2(f[0], f[R > 1 ? 1 : 0], lane, o0, o1);
        if (lane == 0) { out[sl[0] * njm + jr[0]] = o0; if (cnt > 1) out[sl[R > 1 ? 1 : 0] * njm + jr[R > 1 ? 1 : 0]] = o1; }
    }
}

template <int NIT>
__global__ void __launch_bounds__(kT, 1) k_ds_experts_down(SArgs a) {
    extern __shared__ __align__(128) unsigned char sm[];
    const SpDims d = a.d;
    const int E = d.E, NU = d.NU, FFE = d.FFE;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, G = gridDim.x, b = blockIdx.x;
    const Lay3 ly = lay3(d, G);
    Ctl *ctl = reinterpret_cast<Ctl *>(sm + ly.ctl);
    signed char *q_h = reinterpret_cast<signed char *>(sm + ly.q_h);
    float *s_h = reinterpret_cast<float *>(sm + ly.s_h); int *c_h = reinterpret_cast<int *>(sm + ly.c_h);
    float *out = reinterpret_cast<float *>(sm + ly.out);
    const SpLayerDev &L = a.L;
    const int j0 = (int)((long long)b * E / G), nj = (int)((long long)(b + 1) * E / G) - j0, njm = cdiv(E, G);
    const unsigned rb = (unsigned)FFE >> 1, sb = (unsigned)FFE >> 4;
    const int n32 = FFE >> 5, blk16 = FFE >> 4, nblk = (NU * FFE) >> 4;
    const int SGs = cdiv(NU, kDnBars);                    /* expert slots per landing part */
    STAMP(2, 0);
    if (t == 0) {
        for (int i = 0; i < kDnBars; i++) mbar_init(smem_u32(&ctl->bar[i]), 1);
        ctl->abort = 0;
        fence_barrier_init();
    }
    __syncthreads();
    pdl_launch();
    pdl_wait();
    STAMP(2, 1);
    if (warp == 0 && nj > 0) {                            /* the selection is in memory: start this CTA's rows of every selected expert */
        const int e = lane < NU ? __ldcg(a.s.sel_asc + lane) : 0;
        const unsigned char *bs = reinterpret_cast<const unsigned char *>(L.dn_bs);
        const Span sp = make_span(bs + ((size_t)e * E + j0) * sb, (unsigned)nj * sb);
        if (lane < NU) ctl->sdelta[lane] = sp.delta;
        /* bytes per landing part: the lanes of its slots add up */
        unsigned mine = lane < NU ? (unsigned)nj * rb + sp.bytes : 0u;
        for (int g = 0; g * SGs < NU; g++) {
            unsigned v = (lane >= g * SGs && lane < (g + 1) * SGs) ? mine : 0u;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) mbar_expect_tx(smem_u32(&ctl->bar[g]), v);
        }
        __syncwarp();
        if (lane < NU) {
            const uint32_t bar = smem_u32(&ctl->bar[lane / SGs]);
            bulk_g2s(sm + ly.st_c + (size_t)lane * njm * rb, L.dn_codes + ((size_t)e * E + j0) * rb, (unsigned)nj * rb, bar);
            bulk_g2s(sm + ly.st_s + (size_t)lane * ly.span_max, sp.src, sp.bytes, bar);
        }
    }
    STAMP(2, 5);
    if (t < NU) { ctl->sel_asc[t] = __ldcg(a.s.sel_asc + t); ctl->cw[t] = __ldcg(a.s.cw + t); }
    for (int bq = t; bq < nblk; bq += kT) quant_from_global(a.s.h + 16 * bq, reinterpret_cast<int4 *>(q_h) + bq, s_h + bq, c_h + bq);
    STAMP(2, 6);
    __syncthreads();
    STAMP(2, 2);
    if ((a.flags & SP_STAGED_PREFETCH_NEXT) && a.has_next) {   /* the next layer's router rows and shared gate/up pairs of this CTA's slice */
        const SpLayerDev &N = a.Ln;
        const int r0 = (int)((long long)b * d.NE / G), nr = (int)((long long)(b + 1) * d.NE / G) - r0;
        const int p0 = (int)((long long)b * d.FFS / G), np = (int)((long long)(b + 1) * d.FFS / G) - p0;
        if (warp == kW - 1) l2_prefetch(N.router_w + (size_t)r0 * E, nr * E * 4, lane);
        if (warp == kW - 2) { l2_prefetch(N.sg_codes + (size_t)p0 * (E / 2), np * (E / 2), lane); l2_prefetch(reinterpret_cast<const unsigned char *>(N.sg_bs) + (size_t)p0 * (E / 16), np * (E / 16), lane); }
        if (warp == kW - 3) { l2_prefetch(N.su_codes + (size_t)p0 * (E / 2), np * (E / 2), lane); l2_prefetch(reinterpret_cast<const unsigned char *>(N.su_bs) + (size_t)p0 * (E / 16), np * (E / 16), lane); }
    }
    /* unit u = slot * nj + row: slot-major, the order the parts land in. Each warp takes an equal share. */
    {
        const int U = NU * nj;
        const int ua = (int)((long long)warp * U / kW), ub = (int)((long long)(warp + 1) * U / kW);
        int u = ua;
        for (; u + 8 <= ub; u += 8) down_round<NIT, 8>(sm, ly, ctl, a.s.status, u, 8, nj, njm, SGs, rb, sb, n32, blk16, lane, out);
        for (; u < ub; u += 2) down_round<NIT, 2>(sm, ly, ctl, a.s.status, u, ub - u < 2 ? ub - u : 2, nj, njm, SGs, rb, sb, n32, blk16, lane, out);
    }
    __syncthreads();
    STAMP(2, 3);
    for (int jj = t; jj < nj; jj += kT) {                 /* k_moe_combine_ord, CF:6071-6077 */
        float acc = 0.0f;
        for (int k = 0; k < NU; k++) acc = __fadd_rn(acc, __fmul_rn(ctl->cw[k], out[k * njm + jj]));
        a.s.acc[j0 + jj] = acc;
    }
    STAMP(2, 4);
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

/* the Gemma-4-26B-A4B class of geometries gets instances sized for it; everything else the widest ones */
bool narrow(const SpDims &d) { return d.E <= 3072 && d.FFS <= 3072 && d.FFE <= 1024; }

}  // namespace

bool sp_staged_fits(const SpDims &d, int sms, size_t smem_optin) {
    if (d.E > 8 * kT || d.FFS / 16 > kT) return false;
    return lay1(d, sms).total <= smem_optin && lay2(d, sms).total <= smem_optin && lay3(d, sms).total <= smem_optin;
}

/* per device: the kernels need more than the default 48 KB of dynamic shared memory */
cudaError_t sp_staged_prepare(const SpDims &d, int sms) {
    const int s1 = (int)lay1(d, sms).total, s2 = (int)lay2(d, sms).total, s3 = (int)lay3(d, sms).total;
    cudaError_t e;
    if (narrow(d)) {
        if ((e = cudaFuncSetAttribute(k_ds_router_shared<6, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, s1)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(k_ds_experts_up<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, s2)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(k_ds_experts_down<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, s3)) != cudaSuccess) return e;
    } else {
        if ((e = cudaFuncSetAttribute(k_ds_router_shared<8, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, s1)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(k_ds_experts_up<4, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, s2)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(k_ds_experts_down<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, s3)) != cudaSuccess) return e;
    }
    return cudaSuccess;
}

/* Enqueues layers [lf, lf+nl) for one token on `st` (capturable into a CUDA graph). */
cudaError_t sp_staged_decode_enqueue(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl, const float *x_in, float *y_out,
                                     int32_t *sel, float *wts, const SpGraphScratch &sc, int sms, unsigned flags, long long *stamps,
                                     cudaStream_t st, bool pdl, int *nlaunch) {
    const int NU = d.NU, grid = sms;
    const size_t sm1 = lay1(d, grid).total, sm2 = lay2(d, grid).total, sm3 = lay3(d, grid).total;
    const bool nw = narrow(d);
    cudaError_t e = cudaSuccess;
    for (int li = 0; li < nl && e == cudaSuccess; li++) {
        SArgs a{};
        a.L = layers_host[lf + li]; a.d = d; a.s = sc; a.first = (li == 0);
        a.x_prev = (li == 0) ? x_in : sc.xbuf[(li - 1) & 1];
        a.x_cur = sc.xbuf[li & 1];
        if (li > 0) { a.s.prev_post_ffw1 = layers_host[lf + li - 1].post_ffw1; a.s.prev_post_ffw2 = layers_host[lf + li - 1].post_ffw2; a.s.prev_post_ffw = layers_host[lf + li - 1].post_ffw; }
        a.sel_out = sel ? sel + (size_t)li * NU : nullptr; a.wts_out = wts ? wts + (size_t)li * NU : nullptr;
        a.has_next = li + 1 < nl; if (a.has_next) a.Ln = layers_host[lf + li + 1];
        a.flags = flags; a.stamps = (li == nl - 1) ? stamps : nullptr;
        e = nw ? launch_pdl(k_ds_router_shared<6, 3>, grid, sm1, st, pdl && li > 0, a) : launch_pdl(k_ds_router_shared<8, 4>, grid, sm1, st, pdl && li > 0, a);
        (*nlaunch)++;
        if (e == cudaSuccess) { e = nw ? launch_pdl(k_ds_experts_up<3, 3>, grid, sm2, st, pdl, a) : launch_pdl(k_ds_experts_up<4, 4>, grid, sm2, st, pdl, a); (*nlaunch)++; }
        if (e == cudaSuccess) { e = nw ? launch_pdl(k_ds_experts_down<1>, grid, sm3, st, pdl, a) : launch_pdl(k_ds_experts_down<4>, grid, sm3, st, pdl, a); (*nlaunch)++; }
    }
    if (e == cudaSuccess) { e = sp_graph_launch_finish(d, layers_host[lf + nl - 1], sc, sc.xbuf[(nl - 1) & 1], y_out, st, pdl); (*nlaunch)++; }
    return e;
}
