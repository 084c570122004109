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
#include <cstring>

namespace {

#ifndef SP_DS_THREADS
#define SP_DS_THREADS 640
#endif
constexpr int kT = SP_DS_THREADS;       /* threads per CTA (a multiple of 128, at least 256) */
constexpr int kW = kT / 32;
constexpr int kRW = 4;                  /* K2: warps that run the softmax / top-NU while the others do the shared-expert rows */
constexpr unsigned kSpin = 1u << 15;    /* suspended polls before a wait on a copy gives up (each may sleep kWaitNs) */
constexpr unsigned kWaitNs = 20000;     /* upper bound the hardware may keep a polling thread suspended, per poll */
#ifndef SP_DS_AHEAD
#define SP_DS_AHEAD 3
#endif
#ifndef SP_DS_LP
#define SP_DS_LP 3
#endif
constexpr int kGuBars = 10;             /* the routed gate|up slice lands in up to 10 parts ... */
constexpr int kGuAhead = SP_DS_AHEAD;             /* ... of which this many are in flight at a time, so they land in the order they are consumed */
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
    long long *stamps;        /* [3][16] device time stamps of CTA 0, or NULL */
    unsigned lay[20];         /* this kernel's shared-memory layout (Lay1 / Lay2 / Lay3), computed on the host */
};

#define STAMP(k, i) do { if (a.stamps && blockIdx.x == 0 && threadIdx.x == 0) { long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); a.stamps[(k) * 16 + (i)] = t_; } } while (0)

/* ---------------------------------------------------------------- PTX helpers */
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, unsigned bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(bar), "r"(bytes) : "memory");
}
/* one poll; the thread may be suspended until the phase completes or kWaitNs pass, so a waiting warp
 * does not take issue slots from the warps that still have work */
__device__ __forceinline__ unsigned mbar_try(uint32_t bar, unsigned parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(kWaitNs) : "memory");
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
#pragma unroll 1
    for (unsigned i = 0; i < kSpin; i++) {
        if (mbar_try(bar, 0)) return;
        if (*abort_flag) return;
    }
    *abort_flag = 1;
    atomicExch(status, SP_KERR_BARRIER_TIMEOUT);
}

/* ask L2 for [p, p+bytes): one 128-byte line per lane per instruction */
__device__ __forceinline__ void l2_prefetch(const void *p, int bytes, int lane) {
    const unsigned char *b = reinterpret_cast<const unsigned char *>(p);
#pragma unroll 1
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
    unsigned long long bar[12];
    int abort;
    int sel_asc[SP_MAX_NU]; float cw[SP_MAX_NU]; int sel_desc[SP_MAX_NU]; float p_desc[SP_MAX_NU];
    unsigned gs_off[2], us_off[2];          /* K2: where the two runs' gate / up scale rows start */
    unsigned sdelta[SP_MAX_NU];             /* K3: bytes before the first scale row of each slot's span */
    alignas(16) int zero[4];                /* K3: the activation operand of an MMA column that is not the lane's */
};

struct Lay1 { unsigned ctl, red, va, vb, ri, q_nx, q_in, s_nx, s_in, c_nx, c_in, st_r, st_gc, st_uc, st_gs, st_us, total; };
__host__ __device__ inline Lay1 lay1(const SpDims &d, int G) {
    Lay1 L; unsigned o = 0;
    auto take = [&](unsigned bytes) { const unsigned at = o; o = up16(o + bytes); return at; };
    const unsigned E = d.E, nb = E / 16, nr = cdiv(d.NE, G), np = cdiv(d.FFS, G), rb = E / 2, sb = E / 16;
    L.ctl = take(sizeof(Ctl)); L.red = take(128 * 8);
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
    L.ctl = take(sizeof(Ctl)); L.red = take(128 * 8); L.ex = take(8 * NE);
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
struct Lay3 { unsigned ctl, q_h, s_h, c_h, out, st_c, st_s, span_max, njm, total; };
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
    L.njm = nj;
    L.total = o;
    return L;
}

/* ---------------------------------------------------------------- small math */
__device__ __forceinline__ float rms_scale(double ss, double inv_n, float eps) {
    const float ms = (float)(ss * inv_n);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
}
/* sum over the CTA in double: shuffle tree per warp, warp totals in warp order. Each call site
 * uses its own 32 slots of `sh`, so one barrier per sum is enough. */
__device__ __forceinline__ double cta_sum(double v, double *sh32) {
    v = warp_sum_f64(v);
    if ((threadIdx.x & 31) == 0) sh32[threadIdx.x >> 5] = v;
    __syncthreads();
    double r = 0.0;
#pragma unroll
    for (int w = 0; w < kW; w++) r += sh32[w];
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
/* Integer block sums become floats without a conversion instruction: the dp4a chains start from the bit
 * pattern of 1.5 * 2^23, so their int results ARE floats C + n (exact for |n| < 2^22). With lo = C + (even-
 * nibble sum - correction) and hi = C + 16 * (odd-nibble sum), fma(hi, 1/16, lo) = (C + C/16) + a exactly
 * (every intermediate is an integer below 2^24), and subtracting C + C/16 leaves float(a) - the value
 * k_gemv_q4b_dp4a_v2's int -> float conversion gives (CF:1700-1708), bit for bit. */
constexpr int kMagicBits = 0x4B400000;                   /* 12582912.0f */
constexpr float kMagicSum = 13369344.0f;                 /* 12582912 + 12582912 / 16 */

/* this lane's share of one quantised activation vector: chunks c = lane + 32*i; cr holds kMagicBits - correction */
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
            const int2 cr = *reinterpret_cast<const int2 *>(corr + 2 * c);
            r.cr[i] = make_int2(kMagicBits - cr.x, kMagicBits - cr.y);
        } else {
            r.qa[i] = make_int4(0, 0, 0, 0); r.qb[i] = r.qa[i]; r.sx[i] = make_float2(0.0f, 0.0f); r.cr[i] = make_int2(kMagicBits, kMagicBits);
        }
    }
}
/* one row's bytes for this lane, fetched from shared memory before any arithmetic starts */
template <int NIT> struct RowW { int4 w[NIT]; unsigned short sc[NIT]; };
template <int NIT>
__device__ __forceinline__ void row_fetch(RowW<NIT> &r, const unsigned char *codes, const unsigned char *scales, int n32, int lane) {
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int c = lane + 32 * i;
        if (c < n32) { r.w[i] = *reinterpret_cast<const int4 *>(codes + 16 * c); r.sc[i] = *reinterpret_cast<const unsigned short *>(scales + 2 * c); }
        else { r.w[i] = make_int4(0, 0, 0, 0); r.sc[i] = 0; }
    }
}
/* lane partial of one Q4B row against the lane's activation registers:
 * facc = fma(scale, fma(a0, sx0, a1*sx1), facc) over the lane's chunks in increasing c (CF:1697-1708).
 * A chunk beyond the row holds zero codes, a zero scale and a zero activation: its term is +0. */
template <int NIT>
__device__ __forceinline__ float row_dot(const RowW<NIT> &r, const ActR<NIT> &a) {
    float facc = 0.0f;
#pragma unroll
    for (int i = 0; i < NIT; i++) {
        const int4 &w = r.w[i];
        const unsigned t0 = (unsigned)w.x ^ 0x88888888u, t1 = (unsigned)w.y ^ 0x88888888u;
        const unsigned t2 = (unsigned)w.z ^ 0x88888888u, t3 = (unsigned)w.w ^ 0x88888888u;
        const int l0 = dp4a_us(t1 & 0x0F0F0F0Fu, a.qa[i].z, dp4a_us(t0 & 0x0F0F0F0Fu, a.qa[i].x, a.cr[i].x));
        const int h0 = dp4a_us(t1 & 0xF0F0F0F0u, a.qa[i].w, dp4a_us(t0 & 0xF0F0F0F0u, a.qa[i].y, kMagicBits));
        const int l1 = dp4a_us(t3 & 0x0F0F0F0Fu, a.qb[i].z, dp4a_us(t2 & 0x0F0F0F0Fu, a.qb[i].x, a.cr[i].y));
        const int h1 = dp4a_us(t3 & 0xF0F0F0F0u, a.qb[i].w, dp4a_us(t2 & 0xF0F0F0F0u, a.qb[i].y, kMagicBits));
        const float a0 = __fadd_rn(__fmaf_rn(__int_as_float(h0), 0.0625f, __int_as_float(l0)), -kMagicSum);
        const float a1 = __fadd_rn(__fmaf_rn(__int_as_float(h1), 0.0625f, __int_as_float(l1)), -kMagicSum);
        facc = __fmaf_rn(h2f(r.sc[i]), __fmaf_rn(a0, a.sx[i].x, __fmul_rn(a1, a.sx[i].y)), facc);
    }
    return facc;
}
template <int NIT>
__device__ __forceinline__ float row_part(const unsigned char *codes, const unsigned char *scales, const ActR<NIT> &a, int n32, int lane) {
    RowW<NIT> r;
    row_fetch<NIT>(r, codes, scales, n32, lane);
    return row_dot<NIT>(r, a);
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
    const Lay1 &ly = *reinterpret_cast<const Lay1 *>(a.lay);
    Ctl *ctl = reinterpret_cast<Ctl *>(sm + ly.ctl);
    double *red = reinterpret_cast<double *>(sm + ly.red);
    float *va = reinterpret_cast<float *>(sm + ly.va), *vb = reinterpret_cast<float *>(sm + ly.vb), *ri = reinterpret_cast<float *>(sm + ly.ri);
    signed char *q_nx = reinterpret_cast<signed char *>(sm + ly.q_nx), *q_in = reinterpret_cast<signed char *>(sm + ly.q_in);
    float *s_nx = reinterpret_cast<float *>(sm + ly.s_nx), *s_in = reinterpret_cast<float *>(sm + ly.s_in);
    int *c_nx = reinterpret_cast<int *>(sm + ly.c_nx), *c_in = reinterpret_cast<int *>(sm + ly.c_in);
    const SpLayerDev &L = a.L;
    /* this CTA's share of every phase, from the table the host built (no division in the kernel) */
    const int4 sl0 = __ldg(reinterpret_cast<const int4 *>(a.s.slices) + 3 * b), sl1 = __ldg(reinterpret_cast<const int4 *>(a.s.slices) + 3 * b + 1);
    const int r0 = sl0.x, nr = sl0.y, p0 = sl0.z, np = sl0.w;
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
        if (lane == 0) { red[warp] = p1; red[32 + warp] = p2; }
        __syncthreads();
        double s1 = 0.0, s2 = 0.0;
#pragma unroll
        for (int w = 0; w < kW; w++) { s1 += red[w]; s2 += red[32 + w]; }
        const float sc1 = rms_scale(s1, inv_n, d.eps), sc2 = rms_scale(s2, inv_n, d.eps);
        double p3 = 0.0;
#pragma unroll
        for (int k = 0; k < KE; k++) {
            const float mlp = __fmul_rn(__fmul_rn(dn[k], sc1), w1[k]);
            const float t1 = __fmul_rn(__fmul_rn(ac[k], sc2), w2[k]);
            dn[k] = __fadd_rn(mlp, t1); p3 += (double)dn[k] * dn[k];
        }
        const float sc3 = rms_scale(cta_sum(p3, red + 64), inv_n, d.eps);
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
    const float scale = rms_scale(cta_sum(part, red + 96), inv_n, d.eps);
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
#pragma unroll 1
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
#pragma unroll 1
        for (int i = t; i < nb; i += kT) { reinterpret_cast<int4 *>(a.s.in_q)[i] = reinterpret_cast<const int4 *>(q_in)[i]; a.s.in_s[i] = s_in[i]; a.s.in_c[i] = c_in[i]; }
    }
    STAMP(0, 3);
    if (a.flags & SP_STAGED_PREFETCH_SD) {               /* the next kernel's routing-independent rows: ask L2 for them now */
        const int j0 = sl1.x, nj = sl1.y;
        if (warp == kW - 1) { l2_prefetch(L.sd_codes + (size_t)j0 * (d.FFS / 2), nj * (d.FFS / 2), lane); l2_prefetch(reinterpret_cast<const unsigned char *>(L.sd_bs) + (size_t)j0 * (d.FFS / 16), nj * (d.FFS / 16), lane); }
    }
    /* rows: shared gate/up pairs first (warps 0..), router rows after them */
    ActR<NIT> act;
    act_load<NIT>(act, q_nx, s_nx, c_nx, n32, lane);
    const int total = np + nr;
#pragma unroll 1
    for (int u = warp; u < total; u += kW) {
        if (u < np) {
            bar_wait(bar_p, &ctl->abort, a.s.status);
            RowW<NIT> wg, wu;
            row_fetch<NIT>(wg, sm + ly.st_gc + (unsigned)u * rb, sm + ly.st_gs + sg.delta + (unsigned)u * sb, n32, lane);
            row_fetch<NIT>(wu, sm + ly.st_uc + (unsigned)u * rb, sm + ly.st_us + su.delta + (unsigned)u * sb, n32, lane);
            const float g = row_dot<NIT>(wg, act), up = row_dot<NIT>(wu, act);
            float gt, ut;
            tree2(g, up, lane, gt, ut);
            if (lane == 0) a.s.hd[p0 + u] = gelu_mul(gt, ut);
        } else {
            /* fp32 router row, fixed order: lane l takes the float4 groups l, l+32, ... in order, then the tree */
            bar_wait(bar_r, &ctl->abort, a.s.status);
            const int r = u - np;
            const float4 *wrow = reinterpret_cast<const float4 *>(sm + ly.st_r + (unsigned)r * 4u * (unsigned)E);
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

/* ---------------------------------------------------------------- K2: top-NU, shared down, routed gate|up
 * The first kRW warps run the softmax and the selection and start the routed copies; the other warps
 * quantise the shared expert's hidden vector and compute its down rows meanwhile (nothing there depends
 * on the routing). All warps then take the routed pairs as their parts land. */
__device__ __forceinline__ void bar_named(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

/* The routed gate|up rows of this CTA, parts [g_lo, g_hi) of PP pairs each, requested by one warp: lane
 * 4*(g - g_lo) + q copies the codes of (run q>>1, gate/up q&1) that fall into part g; with g_lo == 0 the first
 * four lanes instead copy the block-scale rows of the four (run, gate/up) tensors, which count on part 0's barrier
 * (the code lanes follow them). Run 0 = the
 * first n0 pairs (expert e0 from column c0), run 1 = the rest (expert e1 from column 0). */
struct GuGeo { int nP, n0, c0, e0, e1, PP, FFE; unsigned rbE, sbE; };
__device__ __forceinline__ void gu_issue(unsigned char *sm, const Lay2 &ly, Ctl *ctl, const SpLayerDev &L, const GuGeo &gg, int g_lo, int g_hi, int lane) {
    const int nsc = g_lo == 0 ? 4 : 0, ncode = 4 * (g_hi - g_lo);     /* the scale rows go out first: part 0 cannot complete before them */
    const bool is_scale = lane < nsc;
    const int q = lane & 3;
    const int g = is_scale ? 0 : g_lo + ((lane - nsc) >> 2), run = (q >> 1) & 1, up = q & 1;
    const size_t row0 = (size_t)(run ? gg.e1 : gg.e0) * 2 * gg.FFE + (run ? 0 : gg.c0) + (up ? gg.FFE : 0);      /* first row of this (run, gate/up) */
    const int rlo = run ? gg.n0 : 0, rhi = run ? gg.nP : gg.n0;                                                  /* its pair range */
    unsigned sz = 0, dst = 0; const unsigned char *src = nullptr;
    /* every lane forms the span (the shuffle below needs all of them); only the scale lanes use it */
    const Span sp = make_span(reinterpret_cast<const unsigned char *>(L.gu_bs) + row0 * gg.sbE, (unsigned)(rhi > rlo ? rhi - rlo : 0) * gg.sbE);
    const unsigned prev = __shfl_up_sync(0xffffffffu, sp.bytes, 2);            /* the run-0 span of the same tensor precedes run 1's */
    if (is_scale) {
        const unsigned base = (up ? ly.st_us : ly.st_gs) + (run ? prev : 0u);
        if (rhi > rlo) { sz = sp.bytes; dst = base; src = sp.src; }
        (up ? ctl->us_off : ctl->gs_off)[run] = base + sp.delta;
    } else if (lane < nsc + ncode) {
        int a0 = g * gg.PP, a1 = a0 + gg.PP < gg.nP ? a0 + gg.PP : gg.nP;
        a0 = a0 > rlo ? a0 : rlo; a1 = a1 < rhi ? a1 : rhi;
        if (a1 > a0) {
            sz = (unsigned)(a1 - a0) * gg.rbE; dst = (up ? ly.st_uc : ly.st_gc) + (unsigned)a0 * gg.rbE;
            src = L.gu_codes + (row0 + (size_t)(a0 - rlo)) * gg.rbE;
        }
    }
#pragma unroll 1
    for (int p = g_lo; p < g_hi; p++) {
        const unsigned v = __reduce_add_sync(0xffffffffu, g == p ? sz : 0u);
        if (lane == 0 && v) mbar_expect_tx(smem_u32(&ctl->bar[1 + p]), v);
    }
    __syncwarp();
    if (sz) bulk_g2s(sm + dst, src, sz, smem_u32(&ctl->bar[1 + g]));
}

template <int NIT_E, int NIT_S>
__global__ void __launch_bounds__(kT, 1) k_ds_experts_up(SArgs a) {
    extern __shared__ __align__(128) unsigned char sm[];
    const SpDims d = a.d;
    const int E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, b = blockIdx.x;
    const Lay2 &ly = *reinterpret_cast<const Lay2 *>(a.lay);
    Ctl *ctl = reinterpret_cast<Ctl *>(sm + ly.ctl);
    double *red = reinterpret_cast<double *>(sm + ly.red), *ex = reinterpret_cast<double *>(sm + ly.ex);
    float *lg = reinterpret_cast<float *>(sm + ly.lg), *p = reinterpret_cast<float *>(sm + ly.p), *dsc = reinterpret_cast<float *>(sm + ly.dsc);
    float *wmax = reinterpret_cast<float *>(sm + ly.wmax);
    signed char *q_in = reinterpret_cast<signed char *>(sm + ly.q_in), *q_hd = reinterpret_cast<signed char *>(sm + ly.q_hd);
    float *s_in = reinterpret_cast<float *>(sm + ly.s_in), *s_hd = reinterpret_cast<float *>(sm + ly.s_hd);
    int *c_in = reinterpret_cast<int *>(sm + ly.c_in), *c_hd = reinterpret_cast<int *>(sm + ly.c_hd);
    const SpLayerDev &L = a.L;
    const int4 sl1 = __ldg(reinterpret_cast<const int4 *>(a.s.slices) + 3 * b + 1), sl2 = __ldg(reinterpret_cast<const int4 *>(a.s.slices) + 3 * b + 2);
    const int j0 = sl1.x, nj = sl1.y, P0 = sl1.z, nP = sl1.w;
    const unsigned rbE = (unsigned)E >> 1, sbE = (unsigned)E >> 4, rbS = (unsigned)FFS >> 1, sbS = (unsigned)FFS >> 4;
    const int n32 = E >> 5, n32s = FFS >> 5;
    const uint32_t bar_sd = smem_u32(&ctl->bar[0]);
    const Span sds = make_span(reinterpret_cast<const unsigned char *>(L.sd_bs) + (size_t)j0 * sbS, (unsigned)nj * sbS);
    /* the routed pairs of this CTA lie in at most two expert slots: run 0 = n0 pairs of slot0 from
     * column c0, run 1 = the rest, from column 0 of the next slot. They land in up to kGuBars
     * parts; kGuAhead parts are in flight at a time, so they arrive in the order the warps consume them. */
    const int slot0 = sl2.x, c0 = sl2.y;
    const int n0 = nP < FFE - c0 ? nP : FFE - c0;
    int LP = SP_DS_LP;                                    /* part = 2^LP pairs: the smallest power of two (from 2^SP_DS_LP) that needs at most kGuBars parts */
#pragma unroll 1
    while (((nP + (1 << LP) - 1) >> LP) > kGuBars) LP++;
    const int nparts = (nP + (1 << LP) - 1) >> LP;
    constexpr int TR = 32 * kRW, TS = kT - TR;            /* threads of the two groups */
    STAMP(1, 0);
    if (t == 0) {
#pragma unroll 1
        for (int i = 0; i < 1 + kGuBars; i++) mbar_init(smem_u32(&ctl->bar[i]), 1);
        ctl->abort = 0;
        fence_barrier_init();
        if (nj > 0) {                                     /* shared-expert down rows: fixed addresses */
            mbar_expect_tx(bar_sd, (unsigned)nj * rbS + sds.bytes);
            bulk_g2s(sm + ly.st_sd, L.sd_codes + (size_t)j0 * rbS, (unsigned)nj * rbS, bar_sd);
            bulk_g2s(sm + ly.st_sds, sds.src, sds.bytes, bar_sd);
        }
    }
#pragma unroll 1
    for (int i = t; i < NE; i += kT) dsc[i] = __ldg(L.dexps_scale + i);
    __syncthreads();
    /* The dependent kernel reads the selection before its own wait (to start its weight copies early). It can
     * be launched only once every CTA has signalled, so CTA 0 - the one that publishes the selection - signals
     * after the write and a fence (one lane, right there: a CTA's first signal is the one that counts); the
     * others signal here. */
    if (b != 0) pdl_launch();
    pdl_wait();
    STAMP(1, 1);
    if (warp < kRW) {
        /* ---- moe_topk_host (CF:6220-6240): double softmax, order by (p descending, id ascending), clamp, renormalise */
        float mx = -INFINITY; int bad = 0;
#pragma unroll 1
        for (int i = t; i < NE; i += TR) { const float l = __ldcg(a.s.logits + i); lg[i] = l; if (l != l) bad = 1; mx = fmaxf(mx, l); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); bad |= __shfl_xor_sync(0xffffffffu, bad, o); }
        if (lane == 0) wmax[warp] = mx;
        if (bad && lane == 0) atomicExch(a.s.status, SP_KERR_NAN_ROUTER);
        if (t < SP_MAX_NU) { ctl->sel_desc[t] = t < NE ? t : 0; ctl->p_desc[t] = 0.0f; }
        bar_named(1, TR);
        STAMP(1, 5);
        mx = wmax[0];
#pragma unroll
        for (int w = 1; w < kRW; w++) mx = fmaxf(mx, wmax[w]);
        double part = 0.0;
#pragma unroll 1
        for (int i = t; i < NE; i += TR) { const double e = exp((double)lg[i] - (double)mx); ex[i] = e; part += e; }
        part = warp_sum_f64(part);
        if (lane == 0) red[warp] = part;
        bar_named(1, TR);
        double sum = 0.0;
#pragma unroll
        for (int w = 0; w < kRW; w++) sum += red[w];
        const double rsum = 1.0 / sum;
#pragma unroll 1
        for (int i = t; i < NE; i += TR) p[i] = (float)(ex[i] * rsum);
        bar_named(1, TR);
        STAMP(1, 6);
        if (NE <= 128) {
            /* one warp, four candidates per lane in registers, NU rounds of (largest value, then lowest id among
             * its holders): the order moe_topk_host's strict > insertion produces. key = bits(p) + 1 for a usable
             * probability (p >= 0, so the bit pattern orders like the value), 0 for a NaN or an absent candidate */
            if (warp == 0) {
                unsigned key[4];
#pragma unroll
                for (int k = 0; k < 4; k++) { const int i = lane + 32 * k; const float v = i < NE ? p[i] : __int_as_float(0x7fc00000); key[k] = (v == v) ? __float_as_uint(v) + 1u : 0u; }
#pragma unroll 1
                for (int r = 0; r < NU; r++) {
                    unsigned lm = key[0] > key[1] ? key[0] : key[1]; const unsigned l2 = key[2] > key[3] ? key[2] : key[3]; lm = lm > l2 ? lm : l2;
                    const unsigned m = __reduce_max_sync(0xffffffffu, lm);
                    if (m == 0u) break;
                    unsigned cand = 0x7fffffffu;
#pragma unroll
                    for (int k = 3; k >= 0; k--) if (key[k] == m) cand = (unsigned)(lane + 32 * k);
                    const unsigned w = __reduce_min_sync(0xffffffffu, cand);
#pragma unroll
                    for (int k = 0; k < 4; k++) if ((unsigned)(lane + 32 * k) == w) key[k] = 0u;
                    if (lane == 0) { ctl->sel_desc[r] = (int)w; ctl->p_desc[r] = __uint_as_float(m - 1u); }
                }
                __syncwarp();
            }
        } else {
            /* rank of candidate i = how many candidates beat it (larger p, or equal p and lower id) */
#pragma unroll 1
            for (int i = t; i < NE; i += TR) {
                const float pi = p[i]; int r = 0;
#pragma unroll 4
                for (int j = 0; j < NE; j++) { const float pj = p[j]; r += (pj > pi) || (pj == pi && j < i); }
                if (r < NU && pi == pi) { ctl->sel_desc[r] = i; ctl->p_desc[r] = pi; }
            }
            bar_named(1, TR);
        }
        STAMP(1, 7);
        if (warp == 0) {
            float wnorm = 0.0f; int e = 0, slot = 0;
            if (lane < NU) {
                float ws = 0.0f;
#pragma unroll 1
                for (int k = 0; k < NU; k++) ws = __fadd_rn(ws, ctl->p_desc[k]);
                if (ws < 6.103515625e-5f) ws = 6.103515625e-5f;
                e = ctl->sel_desc[lane];
                wnorm = __fdiv_rn(ctl->p_desc[lane], ws);
#pragma unroll 1
                for (int j = 0; j < NU; j++) slot += (ctl->sel_desc[j] < e);
            }
            __syncwarp();
            if (lane < NU) { ctl->sel_asc[slot] = e; ctl->cw[slot] = __fmul_rn(wnorm, dsc[e]); ctl->p_desc[lane] = wnorm; }
            __syncwarp();
            if (b == 0) asm volatile("bar.arrive 3, 64;" ::: "memory");      /* hands the selection to warp 1, which publishes it (below) */
            if (nP > 0) {                                 /* the selection exists: start the first parts of the routed rows at once */
                const int n1 = nP - n0;
                const GuGeo gg{nP, n0, c0, ctl->sel_asc[slot0], n1 > 0 ? ctl->sel_asc[slot0 + 1] : ctl->sel_asc[slot0], 1 << LP, FFE, rbE, sbE};
                gu_issue(sm, ly, ctl, L, gg, 0, nparts < kGuAhead ? nparts : kGuAhead, lane);
            }
        } else if (warp == 1 && b == 0) {
            /* CTA 0 publishes the selection for the next kernel. A warp with nothing else to do takes it, so that the
             * fence does not sit between the warp that feeds the copy engine and its copies; the CTA's signal to the
             * dependent kernel follows every lane's fence. */
            asm volatile("bar.sync 3, 64;" ::: "memory");
            if (lane < NU) {
                a.s.sel_asc[lane] = ctl->sel_asc[lane]; a.s.cw[lane] = ctl->cw[lane];
                if (a.sel_out) a.sel_out[lane] = ctl->sel_desc[lane];
                if (a.wts_out) a.wts_out[lane] = ctl->p_desc[lane];
                __threadfence();
            }
            __syncwarp();
            if (lane == 0) pdl_launch();
        }
    } else {
        /* ---- the routed experts' input (for the pairs below), the shared expert's hidden vector, its down rows */
        const int ts = t - TR, ws = warp - kRW;
#pragma unroll 1
        for (int i = ts; i < E / 16; i += TS) { reinterpret_cast<int4 *>(q_in)[i] = __ldcg(reinterpret_cast<const int4 *>(a.s.in_q) + i); s_in[i] = __ldcg(a.s.in_s + i); c_in[i] = __ldcg(a.s.in_c + i); }
#pragma unroll 1
        for (int bq = ts; bq < (FFS >> 4); bq += TS) quant_from_global(a.s.hd + 16 * bq, reinterpret_cast<int4 *>(q_hd) + bq, s_hd + bq, c_hd + bq);
        bar_named(2, TS);
        ActR<NIT_S> act;
        act_load<NIT_S>(act, q_hd, s_hd, c_hd, n32s, lane);
        constexpr int WS = kW - kRW;
#pragma unroll 1
        for (int j = ws; j < nj; j += 2 * WS) {
            const int j2 = j + WS; const bool two = j2 < nj;
            bar_wait(bar_sd, &ctl->abort, a.s.status);
            const int jb = two ? j2 : j;
            RowW<NIT_S> wa, wb;
            row_fetch<NIT_S>(wa, sm + ly.st_sd + (unsigned)j * rbS, sm + ly.st_sds + sds.delta + (unsigned)j * sbS, n32s, lane);
            row_fetch<NIT_S>(wb, sm + ly.st_sd + (unsigned)jb * rbS, sm + ly.st_sds + sds.delta + (unsigned)jb * sbS, n32s, lane);
            const float fa = row_dot<NIT_S>(wa, act), fb = row_dot<NIT_S>(wb, act);
            float oa, ob;
            tree2(fa, fb, lane, oa, ob);
            if (lane == 0) { a.s.dn[j0 + j] = oa; if (two) a.s.dn[j0 + j2] = ob; }
        }
    }
    __syncthreads();
    STAMP(1, 2);
    if (warp == kW - 1) {
        /* the last warp has the fewest pairs: it first feeds the copy engine - part k goes out when part k - kGuAhead has landed */
        if (nparts > kGuAhead) {
            const int n1 = nP - n0;
            const GuGeo gg{nP, n0, c0, ctl->sel_asc[slot0], n1 > 0 ? ctl->sel_asc[slot0 + 1] : ctl->sel_asc[slot0], 1 << LP, FFE, rbE, sbE};
#pragma unroll 1
            for (int k = kGuAhead; k < nparts; k++) {
                bar_wait(smem_u32(&ctl->bar[1 + k - kGuAhead]), &ctl->abort, a.s.status);
                gu_issue(sm, ly, ctl, L, gg, k, k + 1, lane);
            }
        }
    }
    STAMP(1, 3);
    /* routed gate|up pairs, as their part lands */
    {
        ActR<NIT_E> act;
        act_load<NIT_E>(act, q_in, s_in, c_in, n32, lane);
        /* four pairs (eight rows) per round: their lane partials wait in registers, one butterfly reduces all
         * eight rows, and the lanes 0, 8, 16, 24 apply the GeGLU of the four pairs at the same time */
#pragma unroll 1
        for (int i0 = warp; i0 < nP; i0 += 4 * kW) {
            float f[8];
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int i = i0 + k * kW;
                f[2 * k] = 0.0f; f[2 * k + 1] = 0.0f;
                if (i < nP) {                             /* warp-uniform */
                    bar_wait(smem_u32(&ctl->bar[1]), &ctl->abort, a.s.status);              /* the scale rows travel with part 0 */
                    bar_wait(smem_u32(&ctl->bar[1 + (i >> LP)]), &ctl->abort, a.s.status);
                    const int run = i >= n0, idx = run ? i - n0 : i;
                    RowW<NIT_E> wg, wu;
                    row_fetch<NIT_E>(wg, sm + ly.st_gc + (unsigned)i * rbE, sm + ctl->gs_off[run] + (unsigned)idx * sbE, n32, lane);
                    row_fetch<NIT_E>(wu, sm + ly.st_uc + (unsigned)i * rbE, sm + ctl->us_off[run] + (unsigned)idx * sbE, n32, lane);
                    f[2 * k] = row_dot<NIT_E>(wg, act); f[2 * k + 1] = row_dot<NIT_E>(wu, act);
                }
            }
            const float tot = tree8(f, lane);             /* lane 4r (and its three neighbours) holds row r: gate of pair k in lanes 8k.., up in lanes 8k+4.. */
            const float upv = __shfl_down_sync(0xffffffffu, tot, 4);
            const int k = lane >> 3, i = i0 + k * kW;
            if ((lane & 7) == 0 && i < nP) a.s.h[P0 + i] = gelu_mul(tot, upv);
        }
    }
    if ((a.flags & SP_STAGED_PREFETCH_DN) && nj > 0) {    /* the routed down rows the next kernel will stage: ask L2 for them */
#pragma unroll 1
        for (int sl = warp; sl < NU; sl += kW) {
            const size_t row = (size_t)ctl->sel_asc[sl] * E + j0;
            l2_prefetch(L.dn_codes + row * (FFE / 2), nj * (FFE / 2), lane);
            l2_prefetch(reinterpret_cast<const unsigned char *>(L.dn_bs) + row * (FFE / 16), nj * (FFE / 16), lane);
        }
    }
    STAMP(1, 12);
    __syncthreads();
    STAMP(1, 4);
}

/* ---------------------------------------------------------------- K3: routed down rows + ordered combine */
/* R consecutive units starting at (slot s, row jj), the first `cnt` of them real; advances (s, jj) past them.
 * `act`/`act_slot`: the lane's registers of one slot's quantised activation, reloaded when the slot changes. */
template <int NIT, int R>
__device__ __forceinline__ void down_round(const unsigned char *sm, const Lay3 &ly, Ctl *ctl, int *status, int &s, int &jj, int cnt, int nj, int njm, int SGs,
                                           unsigned rb, unsigned sb, int n32, int blk16, int lane, float *out, ActR<NIT> &act, int &act_slot) {
    float f[R]; int sl[R], jr[R]; RowW<NIT> rw[R];
    {   /* every landing part these units touch */
        int s_last = s, j_last = jj + cnt - 1;
#pragma unroll 1
        while (j_last >= nj) { j_last -= nj; s_last++; }
        int g = 0, lim = SGs;
#pragma unroll 1
        while (s >= lim) { g++; lim += SGs; }
#pragma unroll 1
        for (;; g++, lim += SGs) { bar_wait(smem_u32(&ctl->bar[g]), &ctl->abort, status); if (s_last < lim) break; }
    }
#pragma unroll
    for (int r = 0; r < R; r++) {                         /* all the rows' bytes first */
        sl[r] = s; jr[r] = jj;
        const unsigned cofs = ly.st_c + ((unsigned)s * (unsigned)njm + (unsigned)jj) * rb;
        const unsigned sofs = ly.st_s + (unsigned)s * ly.span_max + ctl->sdelta[s] + (unsigned)jj * sb;
        row_fetch<NIT>(rw[r], sm + cofs, sm + sofs, n32, lane);
        if (r + 1 < cnt) { if (++jj == nj) { jj = 0; s++; } }          /* units past cnt repeat the last real one */
    }
    if (++jj == nj) { jj = 0; s++; }
#pragma unroll
    for (int r = 0; r < R; r++) {
        const int s = sl[r];
        if (s != act_slot) {                              /* warp-uniform */
            act_load<NIT>(act, reinterpret_cast<const signed char *>(sm + ly.q_h) + (unsigned)s * (unsigned)blk16 * 16u,
                          reinterpret_cast<const float *>(sm + ly.s_h) + (unsigned)s * (unsigned)blk16,
                          reinterpret_cast<const int *>(sm + ly.c_h) + (unsigned)s * (unsigned)blk16, n32, lane);
            act_slot = s;
        }
        f[r] = row_dot<NIT>(rw[r], act);
    }
    if (R == 8) {
        float f8[8];
#pragma unroll
        for (int r = 0; r < 8; r++) f8[r] = f[r < R ? r : 0];
        const float k = tree8(f8, lane);
        const int r = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
        int os = 0, oj = 0;
#pragma unroll
        for (int q = 0; q < 8; q++) if (q == r) { os = sl[q < R ? q : 0]; oj = jr[q < R ? q : 0]; }
        if ((lane & 3) == 0 && r < cnt) out[os * njm + oj] = k;
    } else {
        float o0, o1;
        tree2(f[0], f[R > 1 ? 1 : 0], lane, o0, o1);
        if (lane == 0) { out[sl[0] * njm + jr[0]] = o0; if (cnt > 1) out[sl[R > 1 ? 1 : 0] * njm + jr[R > 1 ? 1 : 0]] = o1; }
    }
}

/* ---- the same row dots on the tensor cores: one warp, 16 rows of one slot (rows ti*16 .. ti*16+15 of the CTA's
 * slice), the row's 32-weight chunks four at a time. mma.sync m16n8k32 s8 x s8: the code nibbles moved to the top of
 * a byte are 16 x code; the activation operand of MMA i is non-zero only in the column (chunk, 16-block) its k-slots
 * belong to, so four MMAs leave, in lane (g, q), the two block sums of chunk 4j+q for rows g and g+8. That lane then
 * does what lane (4j+q) % 32 does in row_dot - one accumulator per slot, chunks in ascending order, the same two fmas
 * and one mul - and the slots are added in the shuffle tree's pairing. Rows past the slice repeat its last row and
 * are dropped. Valid while a row has at most 24 chunks (six groups of four). */
__device__ __forceinline__ void mma_s8_acc(int (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_s8_first(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1, int c) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
                 : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(c));
}
__device__ __forceinline__ float magic16_to_float(int c) { return __fmaf_rn(__int_as_float(c), 0.0625f, -786432.0f); }   /* bits 0x4B400000 + 16 S -> float(S) */
constexpr int kMmaGroups = 6;

__device__ __forceinline__ void down_tile_mma(const unsigned char *sm, const Lay3 &ly, Ctl *ctl, int *status, int s, int ti, int nj, int njm, int SGs,
                                              unsigned rb, unsigned sb, int n32, int blk16, int lane, float *out) {
    bar_wait(smem_u32(&ctl->bar[s / SGs]), &ctl->abort, status);
    const int gq = lane >> 2, q = lane & 3;
    const int r0 = ti * 16 + gq, r1 = r0 + 8;
    const int rc0 = r0 < nj ? r0 : nj - 1, rc1 = r1 < nj ? r1 : nj - 1;
    const unsigned char *c0 = sm + ly.st_c + ((unsigned)s * (unsigned)njm + (unsigned)rc0) * rb;
    const unsigned char *c1 = sm + ly.st_c + ((unsigned)s * (unsigned)njm + (unsigned)rc1) * rb;
    const unsigned char *sbase = sm + ly.st_s + (unsigned)s * ly.span_max + ctl->sdelta[s];
    const unsigned char *sc0 = sbase + (unsigned)rc0 * sb, *sc1 = sbase + (unsigned)rc1 * sb;
    const unsigned char *qh = sm + ly.q_h + (unsigned)s * (unsigned)blk16 * 16u;
    const float *sxp = reinterpret_cast<const float *>(sm + ly.s_h) + (unsigned)s * (unsigned)blk16;
    const unsigned char *zero = reinterpret_cast<const unsigned char *>(ctl->zero);
    const bool bvalid = (gq >> 1) == q; const int bh = gq & 1;
    float acc[8][2];
#pragma unroll
    for (int i = 0; i < 8; i++) acc[i][0] = acc[i][1] = 0.0f;
#pragma unroll
    for (int jj = 0; jj < kMmaGroups; jj++) {
        if (4 * jj < n32) {                               /* warp-uniform */
            const int c = 4 * jj + q; const bool cv = c < n32; const int cc = cv ? c : n32 - 1;
            uint4 w0 = *reinterpret_cast<const uint4 *>(c0 + 16 * cc), w1 = *reinterpret_cast<const uint4 *>(c1 + 16 * cc);
            if (!cv) { w0 = make_uint4(0, 0, 0, 0); w1 = w0; }
            const float s0 = h2f(*reinterpret_cast<const unsigned short *>(sc0 + 2 * cc)), s1 = h2f(*reinterpret_cast<const unsigned short *>(sc1 + 2 * cc));
            const unsigned x0[4] = {w0.x, w0.y, w0.z, w0.w}, x1[4] = {w1.x, w1.y, w1.z, w1.w};
            unsigned a[4][4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                a[i][0] = (x0[i] << 4) & 0xF0F0F0F0u; a[i][1] = (x1[i] << 4) & 0xF0F0F0F0u;
                a[i][2] = x0[i] & 0xF0F0F0F0u;        a[i][3] = x1[i] & 0xF0F0F0F0u;
            }
            const uint4 l0 = *reinterpret_cast<const uint4 *>(bvalid && cv && bh == 0 ? qh + c * 32 : zero);
            const uint4 l1 = *reinterpret_cast<const uint4 *>(bvalid && cv && bh == 1 ? qh + c * 32 + 16 : zero);
            int ca[4], cb[4];
            mma_s8_first(ca, a[0][0], a[0][1], a[0][2], a[0][3], l0.x, l0.y, kMagicBits);
            mma_s8_first(cb, a[2][0], a[2][1], a[2][2], a[2][3], l1.x, l1.y, kMagicBits);
            mma_s8_acc(ca, a[1][0], a[1][1], a[1][2], a[1][3], l0.z, l0.w);
            mma_s8_acc(cb, a[3][0], a[3][1], a[3][2], a[3][3], l1.z, l1.w);
            if (cv) {
                const float2 s2 = *reinterpret_cast<const float2 *>(sxp + 2 * c);
                acc[jj][0] = __fmaf_rn(s0, __fmaf_rn(magic16_to_float(ca[0]), s2.x, __fmul_rn(magic16_to_float(cb[1]), s2.y)), acc[jj][0]);
                acc[jj][1] = __fmaf_rn(s1, __fmaf_rn(magic16_to_float(ca[2]), s2.x, __fmul_rn(magic16_to_float(cb[3]), s2.y)), acc[jj][1]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 2; r++) {
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = acc[i][r];
#pragma unroll
        for (int o = 4; o > 0; o >>= 1)
#pragma unroll
            for (int i = 0; i < o; i++) v[i] += v[i + o];         /* slots s+16, s+8, s+4 of the tree sit in this lane */
        float k = v[0];
        k += __shfl_down_sync(0xffffffffu, k, 2);
        k += __shfl_down_sync(0xffffffffu, k, 1);
        const int row = r ? r1 : r0;
        if (q == 0 && row < nj) out[s * njm + row] = k;
    }
}

template <int NIT>
__global__ void __launch_bounds__(kT, 1) k_ds_experts_down(SArgs a) {
    extern __shared__ __align__(128) unsigned char sm[];
    const SpDims d = a.d;
    const int E = d.E, NU = d.NU, FFE = d.FFE;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5, b = blockIdx.x;
    const Lay3 &ly = *reinterpret_cast<const Lay3 *>(a.lay);
    Ctl *ctl = reinterpret_cast<Ctl *>(sm + ly.ctl);
    signed char *q_h = reinterpret_cast<signed char *>(sm + ly.q_h);
    float *s_h = reinterpret_cast<float *>(sm + ly.s_h); int *c_h = reinterpret_cast<int *>(sm + ly.c_h);
    float *out = reinterpret_cast<float *>(sm + ly.out);
    const SpLayerDev &L = a.L;
    const int4 sl0 = __ldg(reinterpret_cast<const int4 *>(a.s.slices) + 3 * b), sl1 = __ldg(reinterpret_cast<const int4 *>(a.s.slices) + 3 * b + 1);
    const int j0 = sl1.x, nj = sl1.y, njm = (int)ly.njm;
    const unsigned rb = (unsigned)FFE >> 1, sb = (unsigned)FFE >> 4;
    const int n32 = FFE >> 5, blk16 = FFE >> 4, nblk = (NU * FFE) >> 4;
    const int SGs = (NU + kDnBars - 1) / kDnBars;         /* expert slots per landing part */
    STAMP(2, 0);
    if (t == 0) {
#pragma unroll 1
        for (int i = 0; i < kDnBars; i++) mbar_init(smem_u32(&ctl->bar[i]), 1);
        ctl->abort = 0;
        ctl->zero[0] = ctl->zero[1] = ctl->zero[2] = ctl->zero[3] = 0;
        fence_barrier_init();
    }
    __syncthreads();
    pdl_launch();
    if (warp == 0) {                                      /* the selection was published and fenced before this kernel could be launched: start this
                                                             CTA's rows of every selected expert now, before waiting for the predecessor's hidden vectors */
        const int e = lane < NU ? __ldcg(a.s.sel_asc + lane) : 0;
        const float w = lane < NU ? __ldcg(a.s.cw + lane) : 0.0f;
        if (lane < NU) { ctl->sel_asc[lane] = e; ctl->cw[lane] = w; }
        if (nj > 0) {
            const unsigned char *bs = reinterpret_cast<const unsigned char *>(L.dn_bs);
            const Span sp = make_span(bs + ((size_t)e * E + j0) * sb, (unsigned)nj * sb);
            if (lane < NU) ctl->sdelta[lane] = sp.delta;
            const unsigned mine = lane < NU ? (unsigned)nj * rb + sp.bytes : 0u;       /* bytes per landing part: the lanes of its slots add up */
            const int g = lane / SGs;
#pragma unroll
            for (int gg = 0; gg < kDnBars; gg++) {
                const unsigned v = __reduce_add_sync(0xffffffffu, g == gg ? mine : 0u);
                if (lane == 0 && v) mbar_expect_tx(smem_u32(&ctl->bar[gg]), v);
            }
            __syncwarp();
            if (lane < NU) {
                const uint32_t bar = smem_u32(&ctl->bar[g]);
                bulk_g2s(sm + ly.st_c + (unsigned)lane * (unsigned)njm * rb, L.dn_codes + ((size_t)e * E + j0) * rb, (unsigned)nj * rb, bar);
                bulk_g2s(sm + ly.st_s + (unsigned)lane * ly.span_max, sp.src, sp.bytes, bar);
            }
        }
    }
    STAMP(2, 5);
    pdl_wait();
    STAMP(2, 1);
    float hv[16];
    if (t < nblk) {
#pragma unroll
        for (int i = 0; i < 4; i++) { const float4 f = __ldcg(reinterpret_cast<const float4 *>(a.s.h + 16 * t) + i); hv[4 * i] = f.x; hv[4 * i + 1] = f.y; hv[4 * i + 2] = f.z; hv[4 * i + 3] = f.w; }
    }
    if (t < nblk) quant_block16_store(hv, reinterpret_cast<int4 *>(q_h) + t, s_h + t, c_h + t);
#pragma unroll 1
    for (int bq = t + kT; bq < nblk; bq += kT) quant_from_global(a.s.h + 16 * bq, reinterpret_cast<int4 *>(q_h) + bq, s_h + bq, c_h + bq);
    STAMP(2, 6);
    __syncthreads();
    STAMP(2, 3);
    if ((a.flags & SP_STAGED_PREFETCH_NEXT) && a.has_next) {   /* the next layer's router rows and shared gate/up pairs of this CTA's slice */
        const SpLayerDev &N = a.Ln;
        const int r0 = sl0.x, nr = sl0.y, p0 = sl0.z, np = sl0.w;
        if (warp == kW - 1) l2_prefetch(N.router_w + (size_t)r0 * E, nr * E * 4, lane);
        if (warp == kW - 2) { l2_prefetch(N.sg_codes + (size_t)p0 * (E / 2), np * (E / 2), lane); l2_prefetch(reinterpret_cast<const unsigned char *>(N.sg_bs) + (size_t)p0 * (E / 16), np * (E / 16), lane); }
        if (warp == kW - 3) { l2_prefetch(N.su_codes + (size_t)p0 * (E / 2), np * (E / 2), lane); l2_prefetch(reinterpret_cast<const unsigned char *>(N.su_bs) + (size_t)p0 * (E / 16), np * (E / 16), lane); }
    }
    /* unit u = slot * nj + row: slot-major, the order the parts land in. Each warp takes an equal share. */
    if (NIT == 1 && n32 <= 4 * kMmaGroups && (a.flags & SP_STAGED_MMA_DN) && nj > 0) {
        /* tile T = slot * tiles_per_slot + ti, slot-major (the order the parts land in), one tile per warp and turn */
        const int tps = (nj + 15) >> 4;
        int s = 0, ti = warp;
#pragma unroll 1
        while (ti >= tps) { ti -= tps; s++; }
#pragma unroll 1
        while (s < NU) {
            down_tile_mma(sm, ly, ctl, a.s.status, s, ti, nj, njm, SGs, rb, sb, n32, blk16, lane, out);
            ti += kW;
#pragma unroll 1
            while (ti >= tps) { ti -= tps; s++; }
        }
    } else {
        const int U = NU * nj;
        const int ua = (warp * U) / kW, ub = ((warp + 1) * U) / kW;
        int u = ua, s = nj > 0 ? ua / nj : 0, jj = ua - s * nj;          /* the one division of this kernel */
        ActR<NIT> act; int act_slot = -1;
        if (NIT == 1) {                                   /* eight rows per round while a row is one chunk per lane (registers) */
#pragma unroll 1
            for (; ub - u >= 5; u += 8) down_round<NIT, NIT == 1 ? 8 : 2>(sm, ly, ctl, a.s.status, s, jj, ub - u < 8 ? ub - u : 8, nj, njm, SGs, rb, sb, n32, blk16, lane, out, act, act_slot);
        }
#pragma unroll 1
        for (; u < ub; u += 2) down_round<NIT, 2>(sm, ly, ctl, a.s.status, s, jj, ub - u < 2 ? ub - u : 2, nj, njm, SGs, rb, sb, n32, blk16, lane, out, act, act_slot);
    }
    __syncthreads();
    STAMP(2, 7);
#pragma unroll 1
    for (int jj = t; jj < nj; jj += kT) {                 /* k_moe_combine_ord, CF:6071-6077 */
        float o[SP_MAX_NU], w[SP_MAX_NU];
#pragma unroll
        for (int k = 0; k < SP_MAX_NU; k++) { o[k] = k < NU ? out[k * njm + jj] : 0.0f; w[k] = k < NU ? ctl->cw[k] : 0.0f; }
        float acc = 0.0f;
#pragma unroll
        for (int k = 0; k < SP_MAX_NU; k++) if (k < NU) acc = __fadd_rn(acc, __fmul_rn(w[k], o[k]));
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

constexpr int kKEn = (3072 + kT - 1) / kT, kKEw = (4096 + kT - 1) / kT;      /* [E] elements per thread, E <= 3072 / 4096 */
static_assert(4 * kGuAhead + 4 <= 32 && kGuAhead <= kGuBars && 1 + kGuBars <= 12 && kT % 128 == 0 && kT >= 256 && kT <= 1024, "thread count");
/* the Gemma-4-26B-A4B class of geometries gets instances sized for it; everything else the widest ones */
bool narrow(const SpDims &d) { return d.E <= 3072 && d.FFS <= 3072 && d.FFE <= 1024; }

}  // namespace

bool sp_staged_fits(const SpDims &d, int sms, size_t smem_optin) {
    if (d.E > kKEw * kT) return false;
    return lay1(d, sms).total <= smem_optin && lay2(d, sms).total <= smem_optin && lay3(d, sms).total <= smem_optin;
}

/* The share of every phase CTA b of `sms` takes, 12 ints per CTA: router rows r0,nr | shared gate/up pairs
 * p0,np | output rows j0,nj | routed pairs P0,nP | expert slot and column of the first routed pair | 0,0 */
void sp_staged_slices(const SpDims &d, int sms, int *out) {
    const long long NP = (long long)d.NU * d.FFE;
    for (int b = 0; b < sms; b++) {
        int *o = out + 12 * b;
        o[0] = (int)((long long)b * d.NE / sms); o[1] = (int)((long long)(b + 1) * d.NE / sms) - o[0];
        o[2] = (int)((long long)b * d.FFS / sms); o[3] = (int)((long long)(b + 1) * d.FFS / sms) - o[2];
        o[4] = (int)((long long)b * d.E / sms); o[5] = (int)((long long)(b + 1) * d.E / sms) - o[4];
        o[6] = (int)(b * NP / sms); o[7] = (int)((b + 1) * NP / sms) - o[6];
        o[8] = o[6] / d.FFE; o[9] = o[6] - o[8] * d.FFE; o[10] = o[11] = 0;
    }
}

/* per device: the kernels need more than the default 48 KB of dynamic shared memory */
cudaError_t sp_staged_prepare(const SpDims &d, int sms) {
    const int s1 = (int)lay1(d, sms).total, s2 = (int)lay2(d, sms).total, s3 = (int)lay3(d, sms).total;
    cudaError_t e;
    if (narrow(d)) {
        if ((e = cudaFuncSetAttribute(k_ds_router_shared<kKEn, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, s1)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(k_ds_experts_up<3, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, s2)) != cudaSuccess) return e;
        if ((e = cudaFuncSetAttribute(k_ds_experts_down<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, s3)) != cudaSuccess) return e;
    } else {
        if ((e = cudaFuncSetAttribute(k_ds_router_shared<kKEw, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, s1)) != cudaSuccess) return e;
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
    const Lay1 L1 = lay1(d, grid); const Lay2 L2 = lay2(d, grid); const Lay3 L3 = lay3(d, grid);
    const size_t sm1 = L1.total, sm2 = L2.total, sm3 = L3.total;
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
        static_assert(sizeof(Lay1) <= sizeof(a.lay) && sizeof(Lay2) <= sizeof(a.lay) && sizeof(Lay3) <= sizeof(a.lay), "layout does not fit the argument block");
        memcpy(a.lay, &L1, sizeof L1);
        e = nw ? launch_pdl(k_ds_router_shared<kKEn, 3>, grid, sm1, st, pdl && li > 0, a) : launch_pdl(k_ds_router_shared<kKEw, 4>, grid, sm1, st, pdl && li > 0, a);
        (*nlaunch)++;
        memcpy(a.lay, &L2, sizeof L2);
        if (e == cudaSuccess) { e = nw ? launch_pdl(k_ds_experts_up<3, 3>, grid, sm2, st, pdl, a) : launch_pdl(k_ds_experts_up<4, 4>, grid, sm2, st, pdl, a); (*nlaunch)++; }
        memcpy(a.lay, &L3, sizeof L3);
        if (e == cudaSuccess) { e = nw ? launch_pdl(k_ds_experts_down<1>, grid, sm3, st, pdl, a) : launch_pdl(k_ds_experts_down<4>, grid, sm3, st, pdl, a); (*nlaunch)++; }
    }
    if (e == cudaSuccess) { e = sp_graph_launch_finish(d, layers_host[lf + nl - 1], sc, sc.xbuf[(nl - 1) & 1], y_out, st, pdl); (*nlaunch)++; }
    return e;
}
