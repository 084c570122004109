/* common.cuh — shared definitions of libsp_moe_b200 (sm_100a only).
 *
 * Reference citations: CF = src/backends/cuda/cuda_forward.cu of nihilistau/kairos-engine.
 */
#pragma once
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stddef.h>

#define SP_MAX_NU 8          /* G4G_MAX, CF:5989 */

struct SpDims {
    int E, NE, NU, FFE, FFS;
    float eps;
    float inv_sqrt_e;        /* 1/sqrtf(E), computed on the host as the reference does (CF:8403) */
};

/* Device view of one layer inside the resident arena. Same layouts as the reference's host
 * tensors (sp_model.h:50-53); expert e is pointer arithmetic (moe_expert_view, CF:6184-6193). */
struct SpLayerDev {
    const float *router_w, *router_scale, *router_bias;
    const float *ffn_norm, *post_ffw1, *pre_ffw2, *post_ffw2, *post_ffw, *dexps_scale;
    const uint8_t *gu_codes; const uint16_t *gu_bs;
    const uint8_t *dn_codes; const uint16_t *dn_bs;
    const uint8_t *sg_codes; const uint16_t *sg_bs;
    const uint8_t *su_codes; const uint16_t *su_bs;
    const uint8_t *sd_codes; const uint16_t *sd_bs;
};

/* error words a kernel can record (read by sp_moe_status) */
enum { SP_KERR_NONE = 0, SP_KERR_NAN_ROUTER = 1, SP_KERR_BARRIER_TIMEOUT = 2, SP_KERR_OVERFLOW = 3 };

/* ---------------------------------------------------------------- loads */
/* streamed-once weight bytes: read-only path, do not keep in L1 */
__device__ __forceinline__ int4 ld_stream16(const void *p) {
    int4 v;
    asm("ld.global.nc.L1::no_allocate.L2::128B.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ unsigned short ld_stream_u16(const void *p) {
    unsigned short v;
    asm("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ float4 ld_stream_f4(const void *p) {
    float4 v;
    asm("ld.global.nc.L1::no_allocate.L2::128B.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}
/* data another CTA wrote during this kernel: must come from L2, never a stale L1 line */
__device__ __forceinline__ float ld_cg_f32(const float *p) { return __ldcg(p); }

__device__ __forceinline__ float h2f(unsigned short h) { return __half2float(__ushort_as_half(h)); }

/* ---------------------------------------------------------------- Q4B x int8 chunk dot
 * One 16-byte chunk = 32 weights; byte k = weight 2k (low nibble) | weight 2k+1 (high nibble),
 * code = (nib ^ 8) - 8 (CF:1459-1461). With t = word ^ 0x88888888 each nibble holds code + 8,
 * so even weights are (t & 0x0F0F0F0F), odd weights ((t >> 4) & 0x0F0F0F0F) as unsigned bytes,
 * and sum(code*q) = dp4a(u, q) - 8*sum(q). The activation block is therefore kept in shared
 * memory de-interleaved per 8 (4 even-index int8, then 4 odd-index int8) with the per-16 sum
 * of q beside it. The integer result equals the reference's sp_unpack8 + __dp4a sequence
 * (CF:1648-1654, 1700-1708) exactly: integer addition is order-free. */
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
/* w: 16 B of codes; q: 32 de-interleaved int8 as two int4 (first 16 weights, last 16 weights) */
__device__ __forceinline__ void q4b_chunk_dot(const int4 &w, const int4 &qa, const int4 &qb,
                                              int corr0, int corr1, int &a0, int &a1) {
    /* low nibbles: (t & 0x0F0F0F0F) = code + 8; high nibbles are taken in place,
     * (t & 0xF0F0F0F0) = 16 * (code + 8), and the exact factor 16 is shifted out of the sum */
    const unsigned t0 = (unsigned)w.x ^ 0x88888888u, t1 = (unsigned)w.y ^ 0x88888888u;
    const unsigned t2 = (unsigned)w.z ^ 0x88888888u, t3 = (unsigned)w.w ^ 0x88888888u;
    const int l0 = dp4a_us(t1 & 0x0F0F0F0Fu, qa.z, dp4a_us(t0 & 0x0F0F0F0Fu, qa.x, -corr0));
    const int h0 = dp4a_us(t1 & 0xF0F0F0F0u, qa.w, dp4a_us(t0 & 0xF0F0F0F0u, qa.y, 0));
    const int l1 = dp4a_us(t3 & 0x0F0F0F0Fu, qb.z, dp4a_us(t2 & 0x0F0F0F0Fu, qb.x, -corr1));
    const int h1 = dp4a_us(t3 & 0xF0F0F0F0u, qb.w, dp4a_us(t2 & 0xF0F0F0F0u, qb.y, 0));
    a0 = l0 + (h0 >> 4); a1 = l1 + (h1 >> 4);
}

/* ---------------------------------------------------------------- tanhf, bit-reproducible
 * The reference calls CUDA's tanhf (CF:1370, 6150): a MUFU-based 2-ulp routine. A last-bit
 * difference there flips int8 activation codes a few layers later, so this library uses a fixed
 * sequence of correctly-rounded operations instead (max error 1.52 ulp against the real tanh),
 * which a CPU can replay bit for bit. |y| < 0.55: y + y*z*P(z); else 1 - 2/(exp(2|y|)+1). */
__device__ __forceinline__ float sp_tanhf(float y) {
    const float ay = fabsf(y);
    if (ay != ay) return y;
    if (ay < 0.55f) {
        const float z = __fmul_rn(y, y);
        float p = 0x1.39f73ep-9f;
        p = __fmaf_rn(p, z, -0x1.13b14ap-7f);
        p = __fmaf_rn(p, z, 0x1.64e2f4p-6f);
        p = __fmaf_rn(p, z, -0x1.ba0982p-5f);
        p = __fmaf_rn(p, z, 0x1.1110dcp-3f);
        p = __fmaf_rn(p, z, -0x1.555554p-2f);
        return __fmaf_rn(__fmul_rn(y, z), p, y);
    }
    if (ay >= 9.01f) return copysignf(1.0f, y);
    const float t = __fmul_rn(ay, 2.0f);
    const float n = rintf(__fmul_rn(t, 0x1.715476p+0f));
    float r = __fmaf_rn(n, -0x1.62e4p-1f, t);
    r = __fmaf_rn(n, -0x1.7f7d1cp-20f, r);
    float q = 0x1.a1892cp-13f;
    q = __fmaf_rn(q, r, 0x1.6d9918p-10f);
    q = __fmaf_rn(q, r, 0x1.1110ap-7f);
    q = __fmaf_rn(q, r, 0x1.55547cp-5f);
    q = __fmaf_rn(q, r, 0x1.555556p-3f);
    q = __fmaf_rn(q, r, 0x1p-1f);
    const float e = __fmaf_rn(__fmul_rn(r, r), q, __fadd_rn(r, 1.0f));
    const float E = __uint_as_float(__float_as_uint(e) + ((unsigned)((int)n) << 23));   /* e * 2^n, exact */
    const float v = __fsub_rn(1.0f, __fdiv_rn(2.0f, __fadd_rn(E, 1.0f)));
    return copysignf(v, y);
}

/* ---------------------------------------------------------------- GELU-tanh gate (CF:1364-1373, 6143-6152)
 * Explicit operation order (the one the reference documents for its compiled kernel,
 * moe_cpu_expert.c:312-318) so the compiler cannot pick another contraction. */
__device__ __forceinline__ float gelu_mul(float x, float up) {
    float r = __fmul_rn(x, 0.044715f);
    r = __fmul_rn(x, r);
    r = __fmaf_rn(x, r, x);
    const float hx = __fmul_rn(x, 0.5f);
    const float y = __fmul_rn(r, 0.7978845608028654f);
    const float th = sp_tanhf(y);
    return __fmul_rn(__fmul_rn(hx, __fadd_rn(th, 1.0f)), up);
}

/* ---------------------------------------------------------------- activation quantiser (CF:1564-1585)
 * One call quantises ONE 16-element block held in registers and writes it de-interleaved:
 * dst[0..3] = q0,q2,q4,q6 | dst[4..7] = q1,q3,q5,q7 | dst[8..11] = q8,q10,.. | dst[12..15] = q9,q11,..
 * Returns the block scale; *qsum = 8 * sum(q) (the dp4a offset correction). */
__device__ __forceinline__ float quant_block16(const float *v, signed char *dst, int *corr) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i++) { const float a = fabsf(v[i]); if (a > m) m = a; }
    const float scale = m > 0.0f ? __fmul_rn(m, 1.0f / 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    int s = 0;
    int q[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        int t = __float2int_rn(__fmul_rn(v[i], inv));
        t = t > 127 ? 127 : t; t = t < -127 ? -127 : t;
        q[i] = t; s += t;
    }
#pragma unroll
    for (int g = 0; g < 2; g++) {
#pragma unroll
        for (int i = 0; i < 4; i++) {
            dst[g * 8 + i]     = (signed char)q[g * 8 + 2 * i];
            dst[g * 8 + 4 + i] = (signed char)q[g * 8 + 2 * i + 1];
        }
    }
    *corr = 8 * s;
    return scale;
}

/* Same quantiser for a block held in registers, stored with one 16-byte write. */
__device__ __forceinline__ void quant_block16_store(const float (&v)[16], int4 *dst, float *sx, int *corr) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; i++) a[i] = fabsf(v[i]);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1)
#pragma unroll
        for (int i = 0; i < o; i++) a[i] = fmaxf(a[i], a[i + o]);
    const float m = a[0];
    const float scale = m > 0.0f ? __fmul_rn(m, 1.0f / 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    int q[16];
#pragma unroll
    for (int i = 0; i < 16; i++) {
        int t = __float2int_rn(__fmul_rn(v[i], inv));
        t = t > 127 ? 127 : t; t = t < -127 ? -127 : t;
        q[i] = t;
    }
    int s = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) s += q[i];
    int4 w;
    w.x = (q[0] & 0xFF) | ((q[2] & 0xFF) << 8) | ((q[4] & 0xFF) << 16) | ((q[6] & 0xFF) << 24);
    w.y = (q[1] & 0xFF) | ((q[3] & 0xFF) << 8) | ((q[5] & 0xFF) << 16) | ((q[7] & 0xFF) << 24);
    w.z = (q[8] & 0xFF) | ((q[10] & 0xFF) << 8) | ((q[12] & 0xFF) << 16) | ((q[14] & 0xFF) << 24);
    w.w = (q[9] & 0xFF) | ((q[11] & 0xFF) << 8) | ((q[13] & 0xFF) << 16) | ((q[15] & 0xFF) << 24);
    *dst = w; *sx = scale; *corr = 8 * s;
}

/* Same quantiser, one element per thread: the 16 lanes of a half-warp hold one block. Every
 * lane of the warp must call (shuffles use the full mask); `valid` gates only the stores.
 * dst/sx/corr point at the block's own slots. */
__device__ __forceinline__ void quant_elem16(float v, bool valid, signed char *dst_block, float *sx_b, int *corr_b) {
    const int k = threadIdx.x & 15;
    float m = fabsf(v);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    const float scale = m > 0.0f ? __fmul_rn(m, 1.0f / 127.0f) : 1.0f;
    const float inv = __fdiv_rn(1.0f, scale);
    int q = __float2int_rn(__fmul_rn(v, inv));
    q = q > 127 ? 127 : q; q = q < -127 ? -127 : q;
    int s = q;
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (valid) {
        const int r = k & 7;
        dst_block[(k & 8) + ((r & 1) << 2) + (r >> 1)] = (signed char)q;
        if (k == 0) { *sx_b = scale; *corr_b = 8 * s; }
    }
}

/* ---------------------------------------------------------------- block-wide f64 sum of squares (CF:497-514)
 * The reference sums in double with 256 strided threads and a halving tree. This keeps the
 * double accumulation and a fixed order (thread-strided partials, warp shuffles, then warps in
 * order); ms is rounded to float once, so the result matches unless the double sums differ in
 * their last bits across a float rounding boundary. */
__device__ __forceinline__ double warp_sum_f64(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}
