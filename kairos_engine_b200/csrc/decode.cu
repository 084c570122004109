/* decode.cu — the M=1 decode path of the MoE feed-forward stack as ONE persistent kernel.
 *
 * Replaces, for n_tok == 1, the ~20 launches + one host round trip per layer of
 * g4_ffn_apply (CF:8314-9050; PRE/MID/TAIL phases CF:8338-8339): k_rmsnorm, gemv_w_packed x3
 * (shared expert), k_gelu_mul, k_moe_router_prep, router SGEMM, D2H + moe_topk_host,
 * k_quant_act_int8, k_gemv_q4b_dp4a_grp x2, k_moe_gelu_split_batch, k_moe_combine_ord and the
 * recombine norms. CF = src/backends/cuda/cuda_forward.cu of nihilistau/kairos-engine.
 *
 * One CTA per SM, launched cooperatively so all CTAs are co-resident. Each CTA has 16 consumer
 * warps and one producer warp.
 *
 *   Weights: every CTA owns a fixed slice of each phase's rows. The producer warp streams that
 *   slice through a ring of 16 KB shared-memory slots with bulk async copies (cp.async.bulk,
 *   completion on an mbarrier per slot), in consumption order, as far ahead as the ring allows:
 *   next layer's routing-independent rows (router, shared expert) are in flight while this
 *   layer's experts are still being consumed. Routed-expert rows are issued the moment the
 *   consumers publish the top-NU selection.
 *
 *   Activations between CTAs (logits, shared-expert hidden, expert hidden, outputs) travel as
 *   8-byte {value, epoch} words that readers poll: data and flag arrive together, so there is no
 *   separate grid barrier. The residual x lives in every CTA's shared memory across layers.
 *
 * Per layer:
 *   A (local)  sum x^2 -> ffn_norm / pre_ffw2 / router-prep vectors, int8-quantised in smem
 *   B (grid)   router rows (fp32) + shared-expert gate/up row pairs -> logits, hd = gelu(g)*u
 *   C (local)  softmax/top-NU/renorm (moe_topk_host semantics), quantise hd
 *   D (grid)   shared-expert down rows + routed gate|up row pairs of the NU selected experts
 *   E (local)  quantise the NU expert activations h
 *   F (grid)   routed down rows; each CTA owns output rows j for ALL experts, so the ordered
 *              combine acc = acc + w*out (ascending expert id) happens inside the CTA
 *   G (local)  post_ffw1 / post_ffw2 norms, branch sum, post_ffw norm, residual add -> x
 *
 * Arithmetic is the reference's decode arithmetic (int8 per-16 activation quant, exact int32
 * dots per 16, fp32 scale/accumulate in the order of k_gemv_q4b_dp4a_v2: chunk c in lane c%32,
 * then the shuffle tree). Every wait is bounded; a wait that runs out records an error word,
 * after which all waits fall through and the kernel runs to its end.
 */
#include "common.cuh"
#include "decode.cuh"

#ifdef SP_DECODE_STAMPS
__device__ long long g_sp_stamps[64 * 8];
#define STAMP(li, k) do { if (blockIdx.x == 0 && threadIdx.x == 0 && (li) < 64) { long long t_; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_)); g_sp_stamps[(li) * 8 + (k)] = t_; } } while (0)
extern "C" int sp_debug_read_stamps(long long *out) { return (int)cudaMemcpyFromSymbol(out, g_sp_stamps, sizeof(long long) * 64 * 8); }
#else
#define STAMP(li, k) do { } while (0)
#endif

namespace {

constexpr int kCons = 512;                 /* consumer threads */
constexpr int kCW = kCons / 32;            /* consumer warps */
constexpr int kThreads = kCons + 32;       /* + one producer warp */
constexpr int kSlot = 16384;               /* ring slot bytes */
constexpr int kMaxSlots = 12;
constexpr int KE = 8;                      /* E <= 4096: at most 8 elements per consumer thread */
constexpr unsigned kSpinLimit = 1u << 22;  /* polls before a wait gives up (order of a second) */

/* ---------------------------------------------------------------- PTX helpers */
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.shared::cta.b64 st, [%0]; }" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, unsigned bytes) {
    asm volatile("{ .reg .b64 st; mbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1; }" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, unsigned parity) {
    unsigned ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cons_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCons) : "memory"); }
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

/* ---------------------------------------------------------------- shared state */
struct Ctl {                      /* small control block in shared memory */
    uint64_t full[kMaxSlots];
    uint64_t empty[kMaxSlots];
    uint64_t sel_ready;
    int abort;                    /* a wait ran out: every later wait falls through */
    int sel_asc[SP_MAX_NU];
    float cw[SP_MAX_NU];
    int sel_desc[SP_MAX_NU];
    float p_desc[SP_MAX_NU];
};

struct Act {                      /* one quantised activation vector in shared memory */
    const int4 *q;                /* [in/16] blocks of 16 int8, de-interleaved (common.cuh) */
    const float *sx;              /* [in/16] block scales */
    const int *corr;              /* [in/16] 8 * sum(q) per block */
};

struct Smem {
    Ctl *ctl;
    float *x, *va, *vb;           /* [E] residual, two work vectors */
    signed char *q_nx, *q_in, *q_hd, *q_h;
    float *s_nx, *s_in, *s_hd, *s_h;
    int *c_nx, *c_in, *c_hd, *c_h;
    double *red;                  /* [256] reductions */
    double *ex;                   /* [NE] exp values */
    float *p, *lg, *dsc;          /* [NE] probabilities, logits, per-expert down scales */
    float *out;                   /* [NU][rows_f_max] */
    unsigned char *ring;
};

__host__ __device__ inline size_t al16(size_t v) { return (v + 15) & ~(size_t)15; }

/* one layout function for the device carve and the host size query */
template <class F>
__host__ __device__ inline size_t smem_layout(const SpDims &d, int rows_f_max, F place) {
    size_t o = 0;
    auto take = [&](int id, size_t bytes) { place(id, o); o = al16(o + bytes); };
    take(0, sizeof(Ctl));
    take(1, 4 * (size_t)d.E); take(2, 4 * (size_t)d.E); take(3, 4 * (size_t)d.E);
    take(4, d.E); take(5, d.E); take(6, d.FFS); take(7, (size_t)d.NU * d.FFE);
    take(8, 4 * (size_t)(d.E / 16)); take(9, 4 * (size_t)(d.E / 16)); take(10, 4 * (size_t)(d.FFS / 16)); take(11, 4 * (size_t)d.NU * (d.FFE / 16));
    take(12, 4 * (size_t)(d.E / 16)); take(13, 4 * (size_t)(d.E / 16)); take(14, 4 * (size_t)(d.FFS / 16)); take(15, 4 * (size_t)d.NU * (d.FFE / 16));
    take(16, 8 * 256); take(17, 8 * (size_t)d.NE);
    take(18, 4 * (size_t)d.NE); take(19, 4 * (size_t)d.NE); take(20, 4 * (size_t)d.NE);
    take(21, 4 * (size_t)d.NU * rows_f_max);
    o = (o + 127) & ~(size_t)127;
    place(22, o);                                    /* ring starts here */
    return o;
}

__device__ Smem carve(unsigned char *base, const SpDims &d, int rows_f_max) {
    Smem s;
    unsigned char *ptr[23];
    smem_layout(d, rows_f_max, [&](int id, size_t off) { ptr[id] = base + off; });
    s.ctl = (Ctl *)ptr[0];
    s.x = (float *)ptr[1]; s.va = (float *)ptr[2]; s.vb = (float *)ptr[3];
    s.q_nx = (signed char *)ptr[4]; s.q_in = (signed char *)ptr[5]; s.q_hd = (signed char *)ptr[6]; s.q_h = (signed char *)ptr[7];
    s.s_nx = (float *)ptr[8]; s.s_in = (float *)ptr[9]; s.s_hd = (float *)ptr[10]; s.s_h = (float *)ptr[11];
    s.c_nx = (int *)ptr[12]; s.c_in = (int *)ptr[13]; s.c_hd = (int *)ptr[14]; s.c_h = (int *)ptr[15];
    s.red = (double *)ptr[16]; s.ex = (double *)ptr[17];
    s.p = (float *)ptr[18]; s.lg = (float *)ptr[19]; s.dsc = (float *)ptr[20];
    s.out = (float *)ptr[21];
    s.ring = ptr[22];
    return s;
}

/* ---------------------------------------------------------------- this CTA's share of each phase */
struct Geo {
    int rbE, sbE, rbS, sbS, rbF, sbF;     /* bytes per row: codes (in/2), block scales (in/16) */
    int PB;                               /* row pairs (in = E) per ring slot */
    int RS;                               /* shared-down rows (in = FFS) per slot */
    int RF, XF;                           /* routed-down rows per slot part, experts per slot */
    int r0, nr;                           /* router rows */
    int p0, np;                           /* shared gate/up pairs */
    int j0, nj;                           /* output rows (shared down, routed down) */
    int P0, nP;                           /* routed pairs in [0, NU*FFE) */
};
/* room for n scale rows whatever the 16-byte phase of their first byte */
__device__ __forceinline__ int sr_bytes(int n, int sb) { return (n * sb + 15 + 15) & ~15; }
__device__ Geo make_geo(const SpDims &d, int b, int G) {
    Geo g;
    g.rbE = d.E / 2; g.sbE = d.E / 16; g.rbS = d.FFS / 2; g.sbS = d.FFS / 16; g.rbF = d.FFE / 2; g.sbF = d.FFE / 16;
    g.PB = (kSlot - 64) / (2 * (g.rbE + g.sbE));
    g.RS = (kSlot - 32) / (g.rbS + g.sbS);
    g.r0 = (int)((long long)b * d.NE / G); g.nr = (int)((long long)(b + 1) * d.NE / G) - g.r0;
    g.p0 = (int)((long long)b * d.FFS / G); g.np = (int)((long long)(b + 1) * d.FFS / G) - g.p0;
    g.j0 = (int)((long long)b * d.E / G); g.nj = (int)((long long)(b + 1) * d.E / G) - g.j0;
    const int NP = d.NU * d.FFE;
    g.P0 = (int)((long long)b * NP / G); g.nP = (int)((long long)(b + 1) * NP / G) - g.P0;
    const int rfmax = (kSlot - 32) / (g.rbF + g.sbF);
    g.RF = g.nj < rfmax ? g.nj : rfmax;
    if (g.RF < 1) g.RF = 1;
    const int blk = g.RF * g.rbF + sr_bytes(g.RF, g.sbF);
    g.XF = (g.RF == g.nj && 2 * blk <= kSlot && d.NU >= 2) ? 2 : 1;
    return g;
}

/* chunk walkers: the producer and every consumer warp step through the same sequence */
struct PairWalk {                 /* items [pos, end()) never cross a multiple of `period` */
    int pos, last, period, per, cid;
    __device__ PairWalk(int p0, int n, int period_, int per_, int cid_) : pos(p0), last(p0 + n), period(period_), per(per_), cid(cid_) {}
    __device__ bool valid() const { return pos < last; }
    __device__ int end() const { int e = pos + per; const int eb = (pos / period + 1) * period; e = e < eb ? e : eb; return e < last ? e : last; }
    __device__ void next() { pos = end(); cid++; }
};
struct FWalk {                    /* units u = slot*nj + jj; a chunk = XF experts x all rows, or 1 expert x RF rows */
    int u, last, nj, RF, XF, NU, cid;
    __device__ FWalk(const Geo &g, int NU_, int cid_) : u(0), last(NU_ * g.nj), nj(g.nj), RF(g.RF), XF(g.XF), NU(NU_), cid(cid_) {}
    __device__ bool valid() const { return u < last; }
    __device__ int end() const {
        const int s = u / nj;
        if (RF == nj) { int xs = NU - s; xs = xs < XF ? xs : XF; return (s + xs) * nj; }
        const int jr = u - s * nj; int rf = nj - jr; rf = rf < RF ? rf : RF; return u + rf;
    }
    __device__ void next() { u = end(); cid++; }
};

/* ---------------------------------------------------------------- bounded waits */
__device__ __forceinline__ bool wait_bar(uint64_t *bar, unsigned parity, Ctl *ctl, int *status) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*(volatile int *)&ctl->abort) return false;
    for (unsigned spins = 0; spins < kSpinLimit; spins++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 63) == 63 && *(volatile int *)&ctl->abort) return false;
    }
    *(volatile int *)&ctl->abort = 1;
    atomicExch(status, SP_KERR_BARRIER_TIMEOUT);
    return false;
}
/* {value, epoch} word another CTA publishes; polls until the epoch matches */
__device__ __forceinline__ float ll_read(const unsigned long long *p, unsigned epoch, Ctl *ctl, int *status) {
    for (unsigned spins = 0; spins < kSpinLimit; spins++) {
        const unsigned long long v = ld_relaxed_u64(p);
        if ((unsigned)(v >> 32) == epoch) return __uint_as_float((unsigned)v);
        if ((spins & 63) == 63 && *(volatile int *)&ctl->abort) return 0.0f;
    }
    *(volatile int *)&ctl->abort = 1;
    atomicExch(status, SP_KERR_BARRIER_TIMEOUT);
    return 0.0f;
}
__device__ __forceinline__ void ll_write(unsigned long long *p, float v, unsigned epoch) {
    st_relaxed_u64(p, ((unsigned long long)epoch << 32) | (unsigned long long)__float_as_uint(v));
}

/* ---------------------------------------------------------------- consumer-side math */
/* sum of squares in the reference's order (k_rmsnorm, CF:503-511): 256 strided double
 * partials, then sh[t] += sh[t+o] for o = 128 .. 1. All consumer threads must call. */
__device__ double block_sumsq(const float *v, int n, double *sh) {
    const int t = threadIdx.x;
    if (t < 256) { double s = 0.0; for (int i = t; i < n; i += 256) { const double a = v[i]; s += a * a; } sh[t] = s; }
    cons_sync();
    if (t < 128) sh[t] += sh[t + 128];
    cons_sync();
    if (t < 64) sh[t] += sh[t + 64];
    cons_sync();
    if (t < 32) {
        double a = sh[t] + sh[t + 32];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_down_sync(0xffffffffu, a, o);
        if (t == 0) sh[0] = a;
    }
    cons_sync();
    const double r = sh[0];
    cons_sync();
    return r;
}
__device__ __forceinline__ float rms_scale_from(double ss, int n, float eps) {
    const float ms = (float)(ss / (double)n);
    return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
}
__device__ __forceinline__ float warp_tree(float v) {      /* CF:1711: lane 0 holds the row sum */
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}
/* Q4B row (codes and f16 block scales in shared memory) . int8 activation, in the order of
 * k_gemv_q4b_dp4a_v2 (CF:1697-1711): chunk c accumulates in lane c%32 in increasing c. */
__device__ __forceinline__ float row_dot(const unsigned char *codes, const unsigned char *scales, int n32, int lane, const Act &a) {
    float facc = 0.0f;
    for (int c = lane; c < n32; c += 32) {
        const int4 w = *reinterpret_cast<const int4 *>(codes + 16 * c);
        const unsigned short sc = *reinterpret_cast<const unsigned short *>(scales + 2 * c);
        const int2 corr = *reinterpret_cast<const int2 *>(a.corr + 2 * c);
        const float2 sx = *reinterpret_cast<const float2 *>(a.sx + 2 * c);
        int a0, a1;
        q4b_chunk_dot(w, a.q[2 * c], a.q[2 * c + 1], corr.x, corr.y, a0, a1);
        const float t = __fmaf_rn((float)a0, sx.x, __fmul_rn((float)a1, sx.y));
        facc = __fmaf_rn(h2f(sc), t, facc);
    }
    return warp_tree(facc);
}
/* gate and up rows against the same activation: the activation block is read once */
__device__ __forceinline__ float pair_dot_gelu(const unsigned char *gc, const unsigned char *gs, const unsigned char *uc, const unsigned char *us,
                                               int n32, int lane, const Act &a) {
    float fg = 0.0f, fu = 0.0f;
    for (int c = lane; c < n32; c += 32) {
        const int4 wg = *reinterpret_cast<const int4 *>(gc + 16 * c);
        const int4 wu = *reinterpret_cast<const int4 *>(uc + 16 * c);
        const unsigned short sg = *reinterpret_cast<const unsigned short *>(gs + 2 * c);
        const unsigned short su = *reinterpret_cast<const unsigned short *>(us + 2 * c);
        const int2 corr = *reinterpret_cast<const int2 *>(a.corr + 2 * c);
        const float2 sx = *reinterpret_cast<const float2 *>(a.sx + 2 * c);
        const int4 qa = a.q[2 * c], qb = a.q[2 * c + 1];
        int a0, a1;
        q4b_chunk_dot(wg, qa, qb, corr.x, corr.y, a0, a1);
        fg = __fmaf_rn(h2f(sg), __fmaf_rn((float)a0, sx.x, __fmul_rn((float)a1, sx.y)), fg);
        q4b_chunk_dot(wu, qa, qb, corr.x, corr.y, a0, a1);
        fu = __fmaf_rn(h2f(su), __fmaf_rn((float)a0, sx.x, __fmul_rn((float)a1, sx.y)), fu);
    }
    const float g = warp_tree(fg), u = warp_tree(fu);
    return gelu_mul(g, u);                                   /* meaningful in lane 0 */
}
/* router row in fp32, fixed order: lane l takes the float4 groups q = l, l+32, ... with
 * acc = fma(w, x, acc) over the four elements in order, then the shuffle tree. */
__device__ __forceinline__ float router_row(const float *wrow, const float *rin, int E, int lane) {
    float acc = 0.0f;
    for (int q = lane; q < (E >> 2); q += 32) {
        const float4 w = *reinterpret_cast<const float4 *>(wrow + 4 * q);
        const float4 xv = *reinterpret_cast<const float4 *>(rin + 4 * q);
        acc = __fmaf_rn(w.x, xv.x, acc); acc = __fmaf_rn(w.y, xv.y, acc);
        acc = __fmaf_rn(w.z, xv.z, acc); acc = __fmaf_rn(w.w, xv.w, acc);
    }
    return warp_tree(acc);
}
/* quantise a vector (read through `get`) into de-interleaved int8 blocks in shared memory */
template <class F>
__device__ __forceinline__ void quant_vec(int n, signed char *q, float *sx, int *corr, F get) {
    for (int base = 0; base < n; base += kCons) {
        const int i = base + (int)threadIdx.x;
        const bool valid = i < n;
        const float v = valid ? get(i) : 0.0f;
        const int b = i >> 4;
        quant_elem16(v, valid, q + 16 * b, sx + b, corr + b);
    }
}

/* moe_topk_host (CF:6220-6240) on the device, run redundantly by every CTA. s.lg holds the
 * logits, s.dsc the per-expert down scales. */
__device__ void topk_block(const SpDims &d, Smem &s, int *status) {
    const int NE = d.NE, NU = d.NU, t = threadIdx.x;
    Ctl *ctl = s.ctl;
    float *wmaxf = reinterpret_cast<float *>(s.red);
    float mx = -INFINITY; int bad = 0;
    for (int i = t; i < NE; i += kCons) { const float l = s.lg[i]; if (l != l) bad = 1; mx = fmaxf(mx, l); }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o)); bad |= __shfl_xor_sync(0xffffffffu, bad, o); }
    if ((t & 31) == 0) wmaxf[t >> 5] = mx;
    if (bad && (t & 31) == 0) atomicExch(status, SP_KERR_NAN_ROUTER);
    cons_sync();
    mx = wmaxf[0];
#pragma unroll
    for (int w = 1; w < kCW; w++) mx = fmaxf(mx, wmaxf[w]);
    cons_sync();
    /* exp in double, summed in double in a fixed order (strided partials, shuffle tree, warps in order) */
    double part = 0.0;
    for (int i = t; i < NE; i += kCons) { const double e = exp((double)s.lg[i] - (double)mx); s.ex[i] = e; part += e; }
    part = warp_sum_f64(part);
    if ((t & 31) == 0) s.red[t >> 5] = part;
    cons_sync();
    double sum = 0.0;
#pragma unroll
    for (int w = 0; w < kCW; w++) sum += s.red[w];
    for (int i = t; i < NE; i += kCons) s.p[i] = (float)(s.ex[i] / sum);
    if (t < SP_MAX_NU) { ctl->sel_desc[t] = t < NE ? t : 0; ctl->p_desc[t] = 0.0f; }
    cons_sync();
    /* insertion with strict > == rank by (p desc, id asc) */
    for (int i = t; i < NE; i += kCons) {
        const float pi = s.p[i]; int r = 0;
        for (int j = 0; j < NE; j++) { const float pj = s.p[j]; r += (pj > pi) || (pj == pi && j < i); }
        if (r < NU && pi == pi) { ctl->sel_desc[r] = i; ctl->p_desc[r] = pi; }
    }
    cons_sync();
    float wnorm = 0.0f;
    if (t < NU) {
        float wsum = 0.0f;
        for (int k = 0; k < NU; k++) wsum = __fadd_rn(wsum, ctl->p_desc[k]);
        if (wsum < 6.103515625e-5f) wsum = 6.103515625e-5f;
        const int e = ctl->sel_desc[t];
        wnorm = __fdiv_rn(ctl->p_desc[t], wsum);
        int slot = 0;
        for (int j = 0; j < NU; j++) slot += (ctl->sel_desc[j] < e);
        ctl->sel_asc[slot] = e;
        ctl->cw[slot] = __fmul_rn(wnorm, s.dsc[e]);        /* w * dexps_scale[e], CF:8709 */
    }
    cons_sync();
    if (t < NU) ctl->p_desc[t] = wnorm;                    /* renormalised, descending order */
    cons_sync();
}

/* ---------------------------------------------------------------- the producer warp's lane */
struct Producer {
    Ctl *ctl; unsigned char *ring; int ns; int cid; int *status; bool ok;
    __device__ unsigned char *acquire() {
        const int slot = cid % ns;
        if (cid >= ns && ok) ok = wait_bar(&ctl->empty[slot], (unsigned)((cid / ns - 1) & 1), ctl, status);
        return ring + (size_t)slot * kSlot;
    }
    __device__ uint64_t *bar() { return &ctl->full[cid % ns]; }
    /* nbytes of scale rows starting at `src` (any alignment): the enclosing 16-byte-aligned span */
    __device__ unsigned scale_span(const unsigned char *src, int nbytes, const unsigned char *&asrc) {
        const unsigned delta = (unsigned)((uintptr_t)src & 15);
        asrc = src - delta;
        return (delta + (unsigned)nbytes + 15u) & ~15u;
    }
    __device__ void pairs(const unsigned char *gc, const unsigned char *gs, const unsigned char *uc, const unsigned char *us, int n, int rb, int sb) {
        unsigned char *dst = acquire();
        if (ok) {
            const unsigned char *ags, *aus;
            const unsigned bgs = scale_span(gs, n * sb, ags), bus = scale_span(us, n * sb, aus);
            const unsigned cb = (unsigned)(n * rb), sr = (unsigned)sr_bytes(n, sb);
            mbar_expect_tx(bar(), 2 * cb + bgs + bus);
            bulk_g2s(dst, gc, cb, bar());
            bulk_g2s(dst + cb, uc, cb, bar());
            bulk_g2s(dst + 2 * cb, ags, bgs, bar());
            bulk_g2s(dst + 2 * cb + sr, aus, bus, bar());
        }
        cid++;
    }
    __device__ void rows(const unsigned char *c, const unsigned char *sc, int n, int rb, int sb) {
        unsigned char *dst = acquire();
        if (ok) {
            const unsigned char *as;
            const unsigned bs = scale_span(sc, n * sb, as), cb = (unsigned)(n * rb);
            mbar_expect_tx(bar(), cb + bs);
            bulk_g2s(dst, c, cb, bar());
            bulk_g2s(dst + cb, as, bs, bar());
        }
        cid++;
    }
    __device__ void rows2(const unsigned char *c0, const unsigned char *s0, const unsigned char *c1, const unsigned char *s1, int n, int rb, int sb) {
        unsigned char *dst = acquire();
        if (ok) {
            const unsigned char *a0, *a1;
            const unsigned b0 = scale_span(s0, n * sb, a0), b1 = scale_span(s1, n * sb, a1), cb = (unsigned)(n * rb);
            const unsigned blk = cb + (unsigned)sr_bytes(n, sb);
            mbar_expect_tx(bar(), 2 * cb + b0 + b1);
            bulk_g2s(dst, c0, cb, bar());
            bulk_g2s(dst + cb, a0, b0, bar());
            bulk_g2s(dst + blk, c1, cb, bar());
            bulk_g2s(dst + blk + cb, a1, b1, bar());
        }
        cid++;
    }
    __device__ void flat(const void *src, unsigned bytes) {
        unsigned char *dst = acquire();
        if (ok) { mbar_expect_tx(bar(), bytes); bulk_g2s(dst, src, bytes, bar()); }
        cid++;
    }
};

__device__ void producer_main(const SpDecodeArgs &a, const Geo &g, Smem &s, int ns) {
    const SpDims &d = a.d;
    Producer P{s.ctl, s.ring, ns, 0, a.status, true};
    for (int li = 0; li < a.n_layers; li++) {
        const SpLayerDev L = a.layers[a.layer_first + li];
        /* B: router rows, then shared-expert gate/up pairs */
        for (int r = 0; r < g.nr; r++) P.flat(L.router_w + (size_t)(g.r0 + r) * d.E, (unsigned)d.E * 4u);
        for (PairWalk w(g.p0, g.np, 1 << 30, g.PB, 0); w.valid(); w.next()) {
            const size_t c = (size_t)w.pos; const int n = w.end() - w.pos;
            P.pairs(L.sg_codes + c * g.rbE, (const unsigned char *)L.sg_bs + c * g.sbE,
                    L.su_codes + c * g.rbE, (const unsigned char *)L.su_bs + c * g.sbE, n, g.rbE, g.sbE);
        }
        /* D, routing-independent part: shared-expert down rows */
        for (PairWalk w(g.j0, g.nj, 1 << 30, g.RS, 0); w.valid(); w.next()) {
            const size_t j = (size_t)w.pos;
            P.rows(L.sd_codes + j * g.rbS, (const unsigned char *)L.sd_bs + j * g.sbS, w.end() - w.pos, g.rbS, g.sbS);
        }
        /* the selection of this layer */
        if (P.ok) P.ok = wait_bar(&s.ctl->sel_ready, (unsigned)(li & 1), s.ctl, a.status);
        int sel[SP_MAX_NU];
#pragma unroll
        for (int k = 0; k < SP_MAX_NU; k++) sel[k] = k < d.NU ? *(volatile int *)&s.ctl->sel_asc[k] : 0;
        /* D: routed gate|up pairs */
        for (PairWalk w(g.P0, g.nP, d.FFE, g.PB, 0); w.valid(); w.next()) {
            const int slot = w.pos / d.FFE, c = w.pos - slot * d.FFE, n = w.end() - w.pos;
            int e = 0;
#pragma unroll
            for (int k = 0; k < SP_MAX_NU; k++) if (k == slot) e = sel[k];
            const size_t grow = (size_t)e * 2 * d.FFE + c, urow = grow + d.FFE;
            P.pairs(L.gu_codes + grow * g.rbE, (const unsigned char *)L.gu_bs + grow * g.sbE,
                    L.gu_codes + urow * g.rbE, (const unsigned char *)L.gu_bs + urow * g.sbE, n, g.rbE, g.sbE);
        }
        /* F: routed down rows */
        for (FWalk w(g, d.NU, 0); w.valid(); w.next()) {
            const int slot = w.u / g.nj, jr = w.u - slot * g.nj;
            int e0 = 0, e1 = 0;
#pragma unroll
            for (int k = 0; k < SP_MAX_NU; k++) { if (k == slot) e0 = sel[k]; if (k == slot + 1) e1 = sel[k]; }
            const size_t row0 = (size_t)e0 * d.E + g.j0 + jr;
            if (g.RF == g.nj && w.end() - w.u == 2 * g.nj) {
                const size_t row1 = (size_t)e1 * d.E + g.j0;
                P.rows2(L.dn_codes + row0 * g.rbF, (const unsigned char *)L.dn_bs + row0 * g.sbF,
                        L.dn_codes + row1 * g.rbF, (const unsigned char *)L.dn_bs + row1 * g.sbF, g.nj, g.rbF, g.sbF);
            } else {
                P.rows(L.dn_codes + row0 * g.rbF, (const unsigned char *)L.dn_bs + row0 * g.sbF, w.end() - w.u, g.rbF, g.sbF);
            }
        }
    }
    /* leave only when every copy this lane started has landed (they all have, unless a wait ran out) */
    const int first = P.cid > ns ? P.cid - ns : 0;
    for (int c = first; c < P.cid; c++) {
        uint64_t *bar = &s.ctl->full[c % ns];
        const unsigned parity = (unsigned)((c / ns) & 1);
        for (unsigned spins = 0; spins < kSpinLimit; spins++) if (mbar_try_wait(bar, parity)) break;
    }
}

/* ---------------------------------------------------------------- consumers: ring access */
struct Consumer {
    Ctl *ctl; unsigned char *ring; int ns; int *status; int lane;
    __device__ const unsigned char *wait(int cid) {
        wait_bar(&ctl->full[cid % ns], (unsigned)((cid / ns) & 1), ctl, status);
        return ring + (size_t)(cid % ns) * kSlot;
    }
    __device__ void release(int cid) { __syncwarp(); if (lane == 0) mbar_arrive(&ctl->empty[cid % ns]); }
};

__global__ void __launch_bounds__(kThreads, 1) k_moe_decode_stack(SpDecodeArgs a) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const SpDims d = a.d;
    const int G = gridDim.x, b = blockIdx.x, t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int E = d.E, NE = d.NE, NU = d.NU, FFE = d.FFE, FFS = d.FFS;
    const int rows_f_max = (E + G - 1) / G + 1;
    Smem s = carve(smem_raw, d, rows_f_max);
    const Geo g = make_geo(d, b, G);
    const int ns = a.n_slots;
    Ctl *ctl = s.ctl;

    if (t == 0) {
        for (int i = 0; i < ns; i++) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->empty[i], kCW); }
        mbar_init(&ctl->sel_ready, 1);
        ctl->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == kCW) {                                   /* ---------------- producer warp */
        if (lane == 0) producer_main(a, g, s, ns);
        return;
    }

    /* ---------------------------------------------------------------- consumers */
    Consumer C{ctl, s.ring, ns, a.status, lane};
    int cid = 0;
    for (int i = t; i < E; i += kCons) s.x[i] = a.x_in[i];
    /* norm / scale vectors of the element-wise steps ride in registers: element i = t + 512*k */
    float wn[KE], wp[KE], rs[KE], w1[KE], w2[KE], w3[KE];
    {
        const SpLayerDev &L0 = a.layers[a.layer_first];
#pragma unroll
        for (int k = 0; k < KE; k++) {
            const int i = t + kCons * k;
            wn[k] = wp[k] = rs[k] = w1[k] = w2[k] = w3[k] = 0.0f;
            if (i < E) { wn[k] = __ldg(L0.ffn_norm + i); wp[k] = __ldg(L0.pre_ffw2 + i); rs[k] = __ldg(L0.router_scale + i); }
        }
    }
    cons_sync();

    for (int li = 0; li < a.n_layers; li++) {
        const SpLayerDev &L = a.layers[a.layer_first + li];
        const unsigned epoch = a.epoch_base + (unsigned)li + 1u;
        STAMP(li, 0);
        /* ---------------- A: norms of x ---------------- */
        {
            const float scale = rms_scale_from(block_sumsq(s.x, E, s.red), E, d.eps);
#pragma unroll
            for (int k = 0; k < KE; k++) {
                const int i = t + kCons * k;
                if (kCons * k < E) {                                    /* uniform per CTA: shuffles stay converged */
                    const bool valid = i < E;
                    const float xs = valid ? __fmul_rn(s.x[i], scale) : 0.0f;
                    const int bq = i >> 4;
                    quant_elem16(valid ? __fmul_rn(xs, wn[k]) : 0.0f, valid, s.q_nx + 16 * bq, s.s_nx + bq, s.c_nx + bq);
                    quant_elem16(valid ? __fmul_rn(xs, wp[k]) : 0.0f, valid, s.q_in + 16 * bq, s.s_in + bq, s.c_in + bq);
                    if (valid) s.va[i] = __fmul_rn(__fmul_rn(xs, d.inv_sqrt_e), rs[k]);   /* CF:5952-5953 */
                }
            }
            for (int i = t; i < NE; i += kCons) s.dsc[i] = __ldg(L.dexps_scale + i);
            cons_sync();
        }
        STAMP(li, 1);
        /* ---------------- B: router rows + shared gate/up pairs ---------------- */
        {
            const int n32 = E >> 5;
            const Act act{reinterpret_cast<const int4 *>(s.q_nx), s.s_nx, s.c_nx};
            for (int r = 0; r < g.nr; r++) {                            /* one slot per router row */
                if (warp == (r % kCW)) {
                    const float *wrow = reinterpret_cast<const float *>(C.wait(cid + r));
                    float l = router_row(wrow, s.va, E, lane);
                    if (lane == 0) { if (L.router_bias) l = __fadd_rn(l, __ldg(L.router_bias + g.r0 + r)); ll_write(a.x_logits + g.r0 + r, l, epoch); }
                }
                C.release(cid + r);
            }
            cid += g.nr;
            PairWalk w(g.p0, g.np, 1 << 30, g.PB, cid);
            for (int p = g.p0 + ((warp + kCW - (g.nr % kCW)) % kCW); p < g.p0 + g.np; p += kCW) {
                while (p >= w.end()) { C.release(w.cid); w.next(); }
                const unsigned char *base = C.wait(w.cid);
                const int n = w.end() - w.pos, idx = p - w.pos;
                const size_t c0 = (size_t)w.pos;
                const unsigned cb = (unsigned)(n * g.rbE), sr = (unsigned)sr_bytes(n, g.sbE);
                const unsigned dg = (unsigned)((uintptr_t)((const unsigned char *)L.sg_bs + c0 * g.sbE) & 15);
                const unsigned du = (unsigned)((uintptr_t)((const unsigned char *)L.su_bs + c0 * g.sbE) & 15);
                const float h = pair_dot_gelu(base + (size_t)idx * g.rbE, base + 2 * cb + dg + (size_t)idx * g.sbE,
                                              base + cb + (size_t)idx * g.rbE, base + 2 * cb + sr + du + (size_t)idx * g.sbE, n32, lane, act);
                if (lane == 0) ll_write(a.x_hd + p, h, epoch);
            }
            while (w.valid()) { C.release(w.cid); w.next(); }
            cid = w.cid;
        }
        STAMP(li, 2);
        /* ---------------- C: top-k, quantise hd ---------------- */
        for (int i = t; i < NE; i += kCons) s.lg[i] = ll_read(a.x_logits + i, epoch, ctl, a.status);
        cons_sync();
        STAMP(li, 3);
        topk_block(d, s, a.status);
        if (t == 0) mbar_arrive(&ctl->sel_ready);                       /* the producer may now fetch the routed rows */
        if (b == 0 && t < NU) {
            if (a.sel_out) a.sel_out[(size_t)li * NU + t] = ctl->sel_desc[t];
            if (a.wts_out) a.wts_out[(size_t)li * NU + t] = ctl->p_desc[t];
        }
        quant_vec(FFS, s.q_hd, s.s_hd, s.c_hd, [&](int i) { return ll_read(a.x_hd + i, epoch, ctl, a.status); });
        cons_sync();
        STAMP(li, 4);
        /* ---------------- D: shared down rows + routed gate|up pairs ---------------- */
        {
            const int n32 = E >> 5, n32s = FFS >> 5;
            const Act act_in{reinterpret_cast<const int4 *>(s.q_in), s.s_in, s.c_in};
            const Act act_hd{reinterpret_cast<const int4 *>(s.q_hd), s.s_hd, s.c_hd};
            {
                PairWalk w(g.j0, g.nj, 1 << 30, g.RS, cid);
                for (int j = g.j0 + warp; j < g.j0 + g.nj; j += kCW) {
                    while (j >= w.end()) { C.release(w.cid); w.next(); }
                    const unsigned char *base = C.wait(w.cid);
                    const int n = w.end() - w.pos, idx = j - w.pos;
                    const unsigned dl = (unsigned)((uintptr_t)((const unsigned char *)L.sd_bs + (size_t)w.pos * g.sbS) & 15);
                    const float o = row_dot(base + (size_t)idx * g.rbS, base + (size_t)n * g.rbS + dl + (size_t)idx * g.sbS, n32s, lane, act_hd);
                    if (lane == 0) ll_write(a.x_dn + j, o, epoch);
                }
                while (w.valid()) { C.release(w.cid); w.next(); }
                cid = w.cid;
            }
            {
                PairWalk w(g.P0, g.nP, FFE, g.PB, cid);
                for (int pu = g.P0 + warp; pu < g.P0 + g.nP; pu += kCW) {
                    while (pu >= w.end()) { C.release(w.cid); w.next(); }
                    const unsigned char *base = C.wait(w.cid);
                    const int n = w.end() - w.pos, idx = pu - w.pos;
                    const int slot = w.pos / FFE, c = w.pos - slot * FFE;
                    const size_t grow = (size_t)ctl->sel_asc[slot] * 2 * FFE + c, urow = grow + FFE;
                    const unsigned cb = (unsigned)(n * g.rbE), sr = (unsigned)sr_bytes(n, g.sbE);
                    const unsigned dg = (unsigned)((uintptr_t)((const unsigned char *)L.gu_bs + grow * g.sbE) & 15);
                    const unsigned du = (unsigned)((uintptr_t)((const unsigned char *)L.gu_bs + urow * g.sbE) & 15);
                    const float h = pair_dot_gelu(base + (size_t)idx * g.rbE, base + 2 * cb + dg + (size_t)idx * g.sbE,
                                                  base + cb + (size_t)idx * g.rbE, base + 2 * cb + sr + du + (size_t)idx * g.sbE, n32, lane, act_in);
                    if (lane == 0) ll_write(a.x_h + pu, h, epoch);
                }
                while (w.valid()) { C.release(w.cid); w.next(); }
                cid = w.cid;
            }
        }
        STAMP(li, 5);
        /* the element-wise vectors of G (this layer) and A (next layer): fetched now, used after F */
        {
            const bool more = li + 1 < a.n_layers;
            const SpLayerDev &Ln = a.layers[a.layer_first + li + (more ? 1 : 0)];
#pragma unroll
            for (int k = 0; k < KE; k++) {
                const int i = t + kCons * k;
                if (i < E) {
                    w1[k] = __ldg(L.post_ffw1 + i); w2[k] = __ldg(L.post_ffw2 + i); w3[k] = __ldg(L.post_ffw + i);
                    if (more) { wn[k] = __ldg(Ln.ffn_norm + i); wp[k] = __ldg(Ln.pre_ffw2 + i); rs[k] = __ldg(Ln.router_scale + i); }
                }
            }
        }
        /* ---------------- E: quantise the expert activations ---------------- */
        quant_vec(NU * FFE, s.q_h, s.s_h, s.c_h, [&](int i) { return ll_read(a.x_h + i, epoch, ctl, a.status); });
        cons_sync();
        STAMP(li, 6);
        /* ---------------- F: routed down rows + ordered combine ---------------- */
        {
            const int n32 = FFE >> 5, blk16 = FFE >> 4;
            FWalk w(g, NU, cid);
            for (int u = warp; u < NU * g.nj; u += kCW) {
                while (u >= w.end()) { C.release(w.cid); w.next(); }
                const unsigned char *base = C.wait(w.cid);
                const int slot = u / g.nj, jj = u - slot * g.nj;
                const int s0 = w.u / g.nj, jr0 = w.u - s0 * g.nj;
                const bool whole = g.RF == g.nj;
                const int rows = whole ? g.nj : (w.end() - w.u);
                const unsigned cb = (unsigned)(rows * g.rbF);
                const unsigned blk = cb + (unsigned)sr_bytes(rows, g.sbF);
                const unsigned char *xb = base + (size_t)(slot - s0) * blk;
                const size_t row_first = (size_t)ctl->sel_asc[slot] * E + g.j0 + (whole ? 0 : jr0);
                const unsigned dl = (unsigned)((uintptr_t)((const unsigned char *)L.dn_bs + row_first * g.sbF) & 15);
                const int idx = whole ? jj : (jj - jr0);
                const Act act{reinterpret_cast<const int4 *>(s.q_h) + (size_t)slot * blk16, s.s_h + (size_t)slot * blk16, s.c_h + (size_t)slot * blk16};
                const float o = row_dot(xb + (size_t)idx * g.rbF, xb + cb + dl + (size_t)idx * g.sbF, n32, lane, act);
                if (lane == 0) s.out[slot * rows_f_max + jj] = o;
            }
            while (w.valid()) { C.release(w.cid); w.next(); }
            cid = w.cid;
            cons_sync();
            for (int jj = t; jj < g.nj; jj += kCons) {                   /* k_moe_combine_ord, CF:6071-6077 */
                float acc = 0.0f;
                for (int k = 0; k < NU; k++) acc = __fadd_rn(acc, __fmul_rn(ctl->cw[k], s.out[k * rows_f_max + jj]));
                ll_write(a.x_acc + g.j0 + jj, acc, epoch);
            }
        }
        STAMP(li, 7);
        /* ---------------- G: recombine (CF:9014-9019) ---------------- */
        {
            for (int i = t; i < E; i += kCons) { s.va[i] = ll_read(a.x_dn + i, epoch, ctl, a.status); s.vb[i] = ll_read(a.x_acc + i, epoch, ctl, a.status); }
            cons_sync();
            const float sc1 = rms_scale_from(block_sumsq(s.va, E, s.red), E, d.eps);
            const float sc2 = rms_scale_from(block_sumsq(s.vb, E, s.red), E, d.eps);
#pragma unroll
            for (int k = 0; k < KE; k++) {
                const int i = t + kCons * k;
                if (i < E) {
                    const float mlp = __fmul_rn(__fmul_rn(s.va[i], sc1), w1[k]);
                    const float t1 = __fmul_rn(__fmul_rn(s.vb[i], sc2), w2[k]);
                    s.va[i] = __fadd_rn(mlp, t1);
                }
            }
            cons_sync();
            const float sc3 = rms_scale_from(block_sumsq(s.va, E, s.red), E, d.eps);
#pragma unroll
            for (int k = 0; k < KE; k++) {
                const int i = t + kCons * k;
                if (i < E) s.x[i] = __fadd_rn(s.x[i], __fmul_rn(__fmul_rn(s.va[i], sc3), w3[k]));
            }
            cons_sync();
        }
    }
    if (b == 0) for (int i = t; i < E; i += kCons) a.y_out[i] = s.x[i];
}

}  // namespace

int sp_decode_slots(const SpDims &d, int grid, size_t smem_limit, size_t *smem_bytes) {
    const int rows_f_max = (d.E + grid - 1) / grid + 1;
    const size_t fixed = smem_layout(d, rows_f_max, [](int, size_t) {});
    if (fixed + 2 * (size_t)kSlot > smem_limit) { *smem_bytes = 0; return 0; }
    size_t ns = (smem_limit - fixed) / kSlot;
    if (ns > (size_t)kMaxSlots) ns = kMaxSlots;
    *smem_bytes = fixed + ns * kSlot;
    return (int)ns;
}
int sp_decode_threads() { return kThreads; }

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
