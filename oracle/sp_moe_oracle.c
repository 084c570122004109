/* sp_moe_oracle.c — CPU restatement of the kairos-engine Gemma-4 MoE feed-forward layer.
 *
 * TEST INFRASTRUCTURE ONLY: the checker for the CUDA library and the benchmark's timed CPU
 * baseline. See sp_moe_oracle.h for the pinning status of each piece.
 * CF = src/backends/cuda/cuda_forward.cu in the nihilistau/kairos-engine tree.
 *
 * Arithmetic is written with explicit fmaf()/separate statements wherever the reference's
 * CUDA code relies on a particular contraction, and the file is compiled with
 * -ffp-contract=off so the compiler adds none of its own.
 */
#include "sp_moe_oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_threads = 0;
void orc_set_threads(int n) { g_threads = n;
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}

/* ---------- f16 <-> f32 (IEEE binary16, round-to-nearest-even) ---------- */
float orc_half_to_float(uint16_t h) {
    const uint32_t s = (uint32_t)(h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu, u;
    if (e == 0) {
        if (m == 0) u = s;
        else { e = 127 - 15 + 1; while (!(m & 0x400u)) { m <<= 1; e--; } m &= 0x3FFu; u = s | (e << 23) | (m << 13); }
    } else if (e == 31) u = s | 0x7F800000u | (m << 13);
    else u = s | ((e + 127 - 15) << 23) | (m << 13);
    float f; memcpy(&f, &u, 4); return f;
}
uint16_t orc_float_to_half(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    const uint16_t s = (uint16_t)((u >> 16) & 0x8000u);
    const uint32_t a = u & 0x7FFFFFFFu;
    if (a >= 0x7F800000u) return (uint16_t)(s | 0x7C00u | ((a > 0x7F800000u) ? 0x200u : 0));
    if (a >= 0x477FF000u) return (uint16_t)(s | 0x7C00u);              /* rounds to inf */
    if (a < 0x33000001u) return s;                                     /* rounds to zero */
    int e = (int)(a >> 23) - 127;
    uint32_t m = (a & 0x7FFFFFu) | 0x800000u;
    int shift; uint32_t he;
    if (e < -14) { shift = 13 + (-14 - e); he = 0; } else { shift = 13; he = (uint32_t)(e + 15); }
    uint32_t q = m >> shift, rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q++;
    uint32_t r = (he == 0) ? q : ((he << 10) + (q - 0x400u));
    return (uint16_t)(s | r);
}

/* ---------- k_rmsnorm, CF:497-514 ----------
 * 256 "threads": thread t sums x[t], x[t+256], ... in double; then a halving tree over the
 * 256 partials; ms = (float)(ss/n); scale = 1/sqrtf(ms+eps); out = x*scale*w. */
static float rms_scale(const float *x, int n, float eps) {
    double sh[256];
    for (int t = 0; t < 256; t++) { double s = 0.0; for (int i = t; i < n; i += 256) { double v = x[i]; s += v * v; } sh[t] = s; }
    for (int o = 128; o > 0; o >>= 1) for (int t = 0; t < o; t++) sh[t] += sh[t + o];
    const float ms = (float)(sh[0] / (double)n);
    return 1.0f / sqrtf(ms + eps);
}
void orc_rmsnorm(const float *x, const float *w, int n, float eps, float *out) {
    const float scale = rms_scale(x, n, eps);
    for (int i = 0; i < n; i++) { float t = x[i] * scale; out[i] = t * w[i]; }
}

/* ---------- k_moe_router_prep, CF:5938-5954 ----------
 * out[i] = x[i] * scale * (1/sqrtf(E)) * rscale[i], multiplied left to right. */
void orc_router_prep(const float *x, const float *rscale, int n, float eps, float *out) {
    const float scale = rms_scale(x, n, eps);
    const float inv_sqrt_e = 1.0f / sqrtf((float)n);
    for (int i = 0; i < n; i++) { float t = x[i] * scale; t = t * inv_sqrt_e; out[i] = t * rscale[i]; }
}

/* ---------- router logit, CF:8405 -> cublasSgemm (CF:13302-13319) ----------
 * The reference computes fp32 logits with cuBLAS, whose summation order is unspecified. Any
 * fixed fp32 order is a faithful restatement; this one is the order the CUDA library uses so
 * expert ids can be compared bit for bit: 32 lanes, lane l walks the float4 groups
 * q = l, l+32, l+64, ... with acc = fma(w, x, acc) over the 4 elements of each group in
 * order; then lane[l] += lane[l+o] for o = 16, 8, 4, 2, 1; lane 0 is the result. */
float orc_router_dot(const float *wrow, const float *rin, int E) {
    float lane[32];
    const int nq = E >> 2;
    for (int l = 0; l < 32; l++) {
        float acc = 0.0f;
        for (int q = l; q < nq; q += 32)
            for (int i = 0; i < 4; i++) acc = fmaf(wrow[4 * q + i], rin[4 * q + i], acc);
        lane[l] = acc;
    }
    for (int o = 16; o > 0; o >>= 1) for (int l = 0; l < o; l++) lane[l] = lane[l] + lane[l + o];
    return lane[0];
}
double orc_router_dot_f64(const float *wrow, const float *rin, int E) {
    double s = 0.0; for (int i = 0; i < E; i++) s += (double)wrow[i] * (double)rin[i]; return s;
}

/* ---------- moe_topk_host, CF:6220-6240 ---------- */
int orc_topk(const float *logits, int NE, int NU, int *idx, float *wt) {
    float mx = logits[0];
    for (int i = 1; i < NE; i++) if (logits[i] > mx) mx = logits[i];
    double sum = 0.0;
    for (int i = 0; i < NE; i++) sum += exp((double)logits[i] - (double)mx);
    for (int k = 0; k < NU; k++) { idx[k] = -1; wt[k] = -1.0f; }
    for (int i = 0; i < NE; i++) {
        const float p = (float)(exp((double)logits[i] - (double)mx) / sum);
        for (int k = 0; k < NU; k++) {
            if (p > wt[k]) {                                   /* strict >: ties keep the lower id */
                for (int j = NU - 1; j > k; j--) { wt[j] = wt[j - 1]; idx[j] = idx[j - 1]; }
                wt[k] = p; idx[k] = i; break;
            }
        }
    }
    for (int k = 0; k < NU; k++) if (idx[k] < 0) return -1;    /* NaN row, CF:8596-8620 */
    float wsum = 0.0f;
    for (int k = 0; k < NU; k++) wsum += wt[k];
    if (wsum < 6.103515625e-5f) wsum = 6.103515625e-5f;
    for (int k = 0; k < NU; k++) wt[k] /= wsum;
    return 0;
}

/* ---------- k_quant_act_int8, CF:1564-1585 (CPU twin moe_cpu_expert.c:259-273) ---------- */
void orc_quant_act_int8(const float *x, int in, int8_t *qx, float *sx) {
    const int nblk = in >> 4;
    for (int b = 0; b < nblk; b++) {
        float m = 0.0f;
        for (int i = 0; i < 16; i++) { float a = fabsf(x[b * 16 + i]); if (a > m) m = a; }
        const float scale = m > 0.0f ? m * (1.0f / 127.0f) : 1.0f;
        sx[b] = scale;
        const float inv = 1.0f / scale;
        for (int i = 0; i < 16; i++) {
            int q = (int)nearbyintf(x[b * 16 + i] * inv);
            if (q > 127) q = 127; if (q < -127) q = -127;
            qx[b * 16 + i] = (int8_t)q;
        }
    }
}

static inline int nib_code(const uint8_t *row, int i) {
    const uint8_t b = row[i >> 1];
    const int nib = (i & 1) ? (b >> 4) : (b & 0xF);
    return (nib ^ 8) - 8;                                      /* CF:1459-1461 */
}

/* ---------- k_gemv_q4b_dp4a_v2, CF:1688-1713 (CPU twin moe_cpu_expert.c:127-172) ----------
 * Row j, 32-weight chunk c: a0 = sum_{k<16} code*q, a1 = sum_{16<=k<32} code*q (exact ints);
 * t = fma(a0, sx[2c], a1*sx[2c+1]); lane[c%32] = fma(wbsc_c, t, lane[c%32]) in increasing c;
 * then lane[l] = lane[l+o] + lane[l] for o = 16..1 (moe_cpu_expert.h:14-18). */
void orc_gemv_q4b_a(const uint8_t *codes, const uint16_t *bs, int in, int rows,
                    const int8_t *qx, const float *sx, float *y) {
    const int rb = in / 2, nb = in / 32;
#pragma omp parallel for schedule(static) if (rows >= 64)
    for (int j = 0; j < rows; j++) {
        const uint8_t *row = codes + (size_t)j * rb;
        const uint16_t *rbs = bs + (size_t)j * nb;
        float lane[32];
        for (int l = 0; l < 32; l++) lane[l] = 0.0f;
        for (int c = 0; c < nb; c++) {
            int a0 = 0, a1 = 0;
            const uint8_t *p = row + c * 16;
            const int8_t *q = qx + c * 32;
            for (int k = 0; k < 8; k++)  { const uint8_t b = p[k]; a0 += (((b & 0xF) ^ 8) - 8) * q[2 * k] + (((b >> 4) ^ 8) - 8) * q[2 * k + 1]; }
            for (int k = 8; k < 16; k++) { const uint8_t b = p[k]; a1 += (((b & 0xF) ^ 8) - 8) * q[2 * k] + (((b >> 4) ^ 8) - 8) * q[2 * k + 1]; }
            const float m1 = (float)a1 * sx[2 * c + 1];
            const float t = fmaf((float)a0, sx[2 * c], m1);
            lane[c & 31] = fmaf(orc_half_to_float(rbs[c]), t, lane[c & 31]);
        }
        for (int o = 16; o > 0; o >>= 1) for (int l = 0; l < o; l++) lane[l] = lane[l + o] + lane[l];
        y[j] = lane[0];
    }
}

/* ---------- flavour B: k_dequant_arena_q4b (CF:1452-1464) + SGEMM (CF:13302-13319) ----------
 * w = code * f32(f16 scale) is exact in f32. The reference's SGEMM order is unspecified, so
 * the dot is taken in double and rounded once: the real-number answer every fp32 or
 * fp16-operand/fp32-accumulate GEMM approximates. */
void orc_gemv_q4b_b(const uint8_t *codes, const uint16_t *bs, int in, int rows,
                    const float *x, float *y) {
    const int rb = in / 2, nb = in / 32;
#pragma omp parallel for schedule(static) if (rows >= 64)
    for (int j = 0; j < rows; j++) {
        const uint8_t *row = codes + (size_t)j * rb;
        const uint16_t *rbs = bs + (size_t)j * nb;
        double acc = 0.0;
        for (int c = 0; c < nb; c++) {
            const float s = orc_half_to_float(rbs[c]);
            double blk = 0.0;
            for (int k = 0; k < 32; k++) { const float wv = (float)nib_code(row, c * 32 + k) * s; blk += (double)wv * (double)x[c * 32 + k]; }
            acc += blk;
        }
        y[j] = (float)acc;
    }
}

/* ---------- tanhf as a fixed sequence of correctly-rounded IEEE operations ----------
 * The reference calls CUDA's tanhf (k_gelu_mul CF:1370, k_moe_gelu_split_batch CF:6150), a
 * MUFU-based routine documented to 2 ulp that no CPU reproduces bit for bit
 * (moe_cpu_expert.h:19-27); its own CPU path used libm's tanhf instead (moe_cpu_expert.c:249).
 * Both are approximations of the same function, and a last-bit difference there flips int8
 * activation codes a few layers later. So the checker and the CUDA library share THIS routine:
 * only fma / mul / add / div / round-to-integer, each correctly rounded on both machines, hence
 * bit-identical results. Measured against the real tanh: max error 1.52 ulp (tests pin it to
 * <= 2 ulp against libm). |y| < 0.55: y + y*z*P(z), z = y*y. Otherwise 1 - 2/(exp(2|y|)+1) with
 * exp by Cody-Waite reduction and a degree-7 polynomial; |y| >= 9.01 gives +-1. */
float orc_tanhf(float y) {
    const float ay = fabsf(y);
    if (ay != ay) return y;
    if (ay < 0.55f) {
        const float z = y * y;
        float p = 0x1.39f73ep-9f;
        p = fmaf(p, z, -0x1.13b14ap-7f);
        p = fmaf(p, z, 0x1.64e2f4p-6f);
        p = fmaf(p, z, -0x1.ba0982p-5f);
        p = fmaf(p, z, 0x1.1110dcp-3f);
        p = fmaf(p, z, -0x1.555554p-2f);
        const float yz = y * z;
        return fmaf(yz, p, y);
    }
    if (ay >= 9.01f) return copysignf(1.0f, y);
    const float t = ay * 2.0f;
    const float n = nearbyintf(t * 0x1.715476p+0f);
    float r = fmaf(n, -0x1.62e4p-1f, t);
    r = fmaf(n, -0x1.7f7d1cp-20f, r);
    float q = 0x1.a1892cp-13f;
    q = fmaf(q, r, 0x1.6d9918p-10f);
    q = fmaf(q, r, 0x1.1110ap-7f);
    q = fmaf(q, r, 0x1.55547cp-5f);
    q = fmaf(q, r, 0x1.555556p-3f);
    q = fmaf(q, r, 0x1p-1f);
    const float rr = r * r;
    const float r1 = r + 1.0f;
    const float e = fmaf(rr, q, r1);
    uint32_t u; memcpy(&u, &e, 4);
    u += (uint32_t)((int32_t)n) << 23;                           /* e * 2^n, exact */
    float E; memcpy(&E, &u, 4);
    const float d = E + 1.0f;
    const float v = 1.0f - 2.0f / d;
    return copysignf(v, y);
}

/* ---------- k_gelu_mul / k_moe_gelu_split, CF:1364-1373, 6143-6165 ----------
 * Source form: 0.5f*x*(1+tanhf(k*(x+0.044715f*x*x*x)))*up, in the operation order the
 * reference documents for its compiled kernel (moe_cpu_expert.c:312-318): r = x*0.044715;
 * r = x*r; r = fma(x, r, x); y = r*k; th = tanh(y); out = ((x*0.5)*(th+1))*up. */
float orc_gelu_mul(float x, float up) {
    float r = x * 0.044715f;
    r = x * r;
    r = fmaf(x, r, x);
    const float h = x * 0.5f;
    const float yv = r * 0.7978845608028654f;
    const float th = orc_tanhf(yv);
    float o = h * (th + 1.0f);
    return o * up;
}

/* Optional backend for the two flavour-A primitives: when set (to the reference's own
 * sp_moe_cpu_quant / sp_moe_cpu_gemv from oracle/_ref, moe_cpu_expert.c:259-294) the layer below
 * runs its quantisation and GEMVs through the reference's code, bit-identical to the restatement. */
static orc_quant_fn g_quant_fn = 0;
static orc_gemv_fn g_gemv_fn = 0;
void orc_set_backend(orc_quant_fn q, orc_gemv_fn g) { g_quant_fn = q; g_gemv_fn = g; }
static void quant_a(const float *x, int in, int8_t *qx, float *sx) {
    if (g_quant_fn && g_quant_fn(x, in, qx, sx) == 0) return;
    orc_quant_act_int8(x, in, qx, sx);
}
static void gemv_a(const uint8_t *codes, const uint16_t *bs, int in, int rows, const int8_t *qx, const float *sx, float *y) {
    if (g_gemv_fn && g_gemv_fn(codes, bs, in, rows, qx, sx, y) == 0) return;
    orc_gemv_q4b_a(codes, bs, in, rows, qx, sx, y);
}

/* matmul through the AMMD macro (CF:8322-8324): flavour A = quant + dp4a GEMV, B = dequant GEMM */
static void matvec(int flavour, const uint8_t *codes, const uint16_t *bs, int in, int rows,
                   const float *x, float *y, int8_t *qx, float *sx) {
    if (flavour == ORC_FLAVOUR_A) { quant_a(x, in, qx, sx); gemv_a(codes, bs, in, rows, qx, sx, y); }
    else orc_gemv_q4b_b(codes, bs, in, rows, x, y);
}

/* ---------- the layer: g4_ffn_apply with moe_on=1, CF:8314-9050 ---------- */
int orc_layer_forward(const orc_cfg *c, const orc_layer *w, int flavour, int M,
                      const float *x, float *y, int *sel, float *wts, float *logits_out, double *margin) {
    const int E = c->E, NE = c->NE, NU = c->NU, FFE = c->FFE, FFS = c->FFS;
    const float eps = c->eps;
    const int maxin = E > FFS ? E : FFS;
    float *nx = malloc(sizeof(float) * E), *g = malloc(sizeof(float) * FFS), *u = malloc(sizeof(float) * FFS);
    float *dn = malloc(sizeof(float) * E), *mlp = malloc(sizeof(float) * E), *rin = malloc(sizeof(float) * E);
    float *lg = malloc(sizeof(float) * NE), *in = malloc(sizeof(float) * E), *acc = malloc(sizeof(float) * E);
    float *gu = malloc(sizeof(float) * 2 * FFE), *h = malloc(sizeof(float) * FFE), *eo = malloc(sizeof(float) * (size_t)NU * E);
    float *t1 = malloc(sizeof(float) * E), *wt = malloc(sizeof(float) * NU), *cw = malloc(sizeof(float) * NU);
    int8_t *qx = malloc(maxin), *qin = malloc(E); float *sx = malloc(sizeof(float) * (maxin / 16 + 1)), *sin_ = malloc(sizeof(float) * (E / 16 + 1));
    int *idx = malloc(sizeof(int) * NU), *ord = malloc(sizeof(int) * NU);
    double *ld = malloc(sizeof(double) * NE);
    int rc = 0;
    for (int t = 0; t < M && rc == 0; t++) {
        const float *xt = x + (size_t)t * E;
        float *yt = y + (size_t)t * E;
        /* dense (shared-expert) branch, CF:8344-8360, 8396 */
        orc_rmsnorm(xt, w->ffn_norm, E, eps, nx);
        if (flavour == ORC_FLAVOUR_A) {                      /* quantised once per GEMV in the reference; same codes */
            quant_a(nx, E, qx, sx);
            gemv_a(w->sg_codes, w->sg_bs, E, FFS, qx, sx, g);
            gemv_a(w->su_codes, w->su_bs, E, FFS, qx, sx, u);
        } else {
            orc_gemv_q4b_b(w->sg_codes, w->sg_bs, E, FFS, nx, g);
            orc_gemv_q4b_b(w->su_codes, w->su_bs, E, FFS, nx, u);
        }
        for (int i = 0; i < FFS; i++) g[i] = orc_gelu_mul(g[i], u[i]);
        matvec(flavour, w->sd_codes, w->sd_bs, FFS, E, g, dn, qx, sx);
        orc_rmsnorm(dn, w->post_ffw1, E, eps, mlp);
        /* router on the RAW residual with its own weightless norm, CF:8402-8405 */
        orc_router_prep(xt, w->router_scale, E, eps, rin);
        for (int e = 0; e < NE; e++) {
            float l = orc_router_dot(w->router_w + (size_t)e * E, rin, E);
            if (w->router_bias) l = l + w->router_bias[e];
            lg[e] = l;
        }
        if (logits_out) memcpy(logits_out + (size_t)t * NE, lg, sizeof(float) * NE);
        if (orc_topk(lg, NE, NU, idx, wt)) { rc = -1; break; }
        if (sel) memcpy(sel + (size_t)t * NU, idx, sizeof(int) * NU);
        if (wts) memcpy(wts + (size_t)t * NU, wt, sizeof(float) * NU);
        if (margin) {
            for (int e = 0; e < NE; e++) ld[e] = orc_router_dot_f64(w->router_w + (size_t)e * E, rin, E) + (w->router_bias ? (double)w->router_bias[e] : 0.0);
            double lo_sel = 1e300, hi_rest = -1e300;
            for (int e = 0; e < NE; e++) { int in_sel = 0; for (int k = 0; k < NU; k++) in_sel |= (idx[k] == e);
                if (in_sel) { if (ld[e] < lo_sel) lo_sel = ld[e]; } else if (ld[e] > hi_rest) hi_rest = ld[e]; }
            margin[t] = lo_sel - hi_rest;
        }
        /* expert input and zeroed accumulator, CF:8425-8426 */
        orc_rmsnorm(xt, w->pre_ffw2, E, eps, in);
        for (int i = 0; i < E; i++) acc[i] = 0.0f;
        /* experts in ASCENDING id (expert-major walk, CF:8664-8743, 8925-8965) */
        for (int k = 0; k < NU; k++) ord[k] = k;
        for (int a = 1; a < NU; a++) { int v = ord[a], b = a - 1; while (b >= 0 && idx[ord[b]] > idx[v]) { ord[b + 1] = ord[b]; b--; } ord[b + 1] = v; }
        if (flavour == ORC_FLAVOUR_A) quant_a(in, E, qin, sin_);
        for (int s = 0; s < NU; s++) {
            const int k = ord[s], e = idx[k];
            const uint8_t *gc = w->gu_codes + (size_t)e * 2 * FFE * (E / 2);
            const uint16_t *gs = w->gu_bs + (size_t)e * 2 * FFE * (E / 32);
            const uint8_t *dc = w->dn_codes + (size_t)e * E * (FFE / 2);
            const uint16_t *ds = w->dn_bs + (size_t)e * E * (FFE / 32);
            if (flavour == ORC_FLAVOUR_A) gemv_a(gc, gs, E, 2 * FFE, qin, sin_, gu);
            else orc_gemv_q4b_b(gc, gs, E, 2 * FFE, in, gu);
            for (int i = 0; i < FFE; i++) h[i] = orc_gelu_mul(gu[i], gu[FFE + i]);
            matvec(flavour, dc, ds, FFE, E, h, eo + (size_t)s * E, qx, sx);
            cw[s] = wt[k] * w->dexps_scale[e];                 /* CF:8709 */
        }
        /* k_moe_combine_ord (CF:6071-6077): acc = fadd(acc, fmul(w, out)), ascending id */
        for (int i = 0; i < E; i++) { float a = acc[i];
            for (int s = 0; s < NU; s++) { const float p = cw[s] * eo[(size_t)s * E + i]; a = a + p; }
            acc[i] = a; }
        /* recombine, CF:9014-9019 */
        orc_rmsnorm(acc, w->post_ffw2, E, eps, t1);
        for (int i = 0; i < E; i++) mlp[i] = mlp[i] + t1[i];
        orc_rmsnorm(mlp, w->post_ffw, E, eps, t1);
        for (int i = 0; i < E; i++) yt[i] = xt[i] + t1[i];
    }
    free(nx); free(g); free(u); free(dn); free(mlp); free(rin); free(lg); free(in); free(acc); free(gu); free(h); free(eo);
    free(t1); free(wt); free(cw); free(qx); free(qin); free(sx); free(sin_); free(idx); free(ord); free(ld);
    return rc;
}

/* ---------- gemma4_moe_ffn_q4b_cuda semantics, CF:13821-13977 ----------
 * ONE weightless rmsnorm (float sum of squares, rsqrt); experts consume the normed hidden;
 * router input = that * (1/sqrt(E) * scale[i]); logits f32 warp-strided dot (dg_k_gemv_f32,
 * CF:13655-13665); softmax with float expf and double sum; greedy top-k (strict >, ties to the
 * lower id); renorm without clamp; experts accumulate in descending-p order with yo += w*de. */
int orc_standalone_q4b(int E, int NE, int NU, int FF, float eps,
                       const float *gate_inp, const float *gate_inp_scale,
                       const uint8_t *gu_codes, const uint16_t *gu_bscale,
                       const uint8_t *dn_codes, const uint16_t *dn_bscale,
                       const float *hidden, float *out, int *sel_out) {
    if ((E & 31) || (FF & 31)) return 1;
    float *xn = malloc(sizeof(float) * E), *tmp = malloc(sizeof(float) * E), *lg = malloc(sizeof(float) * NE);
    float *gu = malloc(sizeof(float) * 2 * FF), *h = malloc(sizeof(float) * FF), *de = malloc(sizeof(float) * E);
    int8_t *qx = malloc(E > FF ? E : FF); float *sx = malloc(sizeof(float) * ((E > FF ? E : FF) / 16 + 1));
    char *used = calloc(NE, 1); int *idx = malloc(sizeof(int) * NU); float *wt = malloc(sizeof(float) * NU);
    /* dg_k_rmsnorm_vec (CF:13632-13644): block of bd threads, float partials, halving tree */
    { int bd = 256; while (bd > E && bd > 32) bd >>= 1;
      float sh[256];
      for (int t = 0; t < bd; t++) { float a = 0.0f; for (int i = t; i < E; i += bd) a = fmaf(hidden[i], hidden[i], a); sh[t] = a; }
      for (int s = bd >> 1; s > 0; s >>= 1) for (int t = 0; t < s; t++) sh[t] += sh[t + s];
      const float inv = 1.0f / sqrtf(sh[0] / (float)E + eps);
      for (int i = 0; i < E; i++) xn[i] = hidden[i] * inv; }
    { const float rs = 1.0f / sqrtf((float)E);
      for (int i = 0; i < E; i++) tmp[i] = xn[i] * (rs * gate_inp_scale[i]); }       /* CF:13647-13650 */
    for (int o = 0; o < NE; o++) {                                                    /* CF:13655-13665 */
        float lane[32];
        for (int l = 0; l < 32; l++) { float a = 0.0f; for (int i = l; i < E; i += 32) a = fmaf(gate_inp[(size_t)o * E + i], tmp[i], a); lane[l] = a; }
        for (int s = 16; s > 0; s >>= 1) for (int l = 0; l < s; l++) lane[l] += lane[l + s];
        lg[o] = lane[0];
    }
    { float mx = lg[0]; for (int i = 1; i < NE; i++) if (lg[i] > mx) mx = lg[i];      /* CF:13912-13917 */
      double se = 0.0; for (int i = 0; i < NE; i++) { lg[i] = expf(lg[i] - mx); se += lg[i]; }
      for (int i = 0; i < NE; i++) lg[i] = (float)(lg[i] / se); }
    float wsum = 0.0f;
    for (int k = 0; k < NU; k++) { int best = -1; float bv = -1.0f;
        for (int i = 0; i < NE; i++) if (!used[i] && lg[i] > bv) { bv = lg[i]; best = i; }
        if (best < 0) { free(xn); free(tmp); free(lg); free(gu); free(h); free(de); free(qx); free(sx); free(used); free(idx); free(wt); return 1; }
        used[best] = 1; idx[k] = best; wt[k] = bv; wsum += bv; }
    for (int k = 0; k < NU; k++) wt[k] = (wt[k] / wsum) * 1.0f;
    if (sel_out) for (int k = 0; k < NU; k++) sel_out[k] = idx[k];
    for (int i = 0; i < E; i++) out[i] = 0.0f;
    for (int k = 0; k < NU; k++) {
        const int e = idx[k];
        orc_quant_act_int8(xn, E, qx, sx);
        orc_gemv_q4b_a(gu_codes + (size_t)e * 2 * FF * (E / 2), gu_bscale + (size_t)e * 2 * FF * (E / 32), E, 2 * FF, qx, sx, gu);
        for (int i = 0; i < FF; i++) h[i] = orc_gelu_mul(gu[i], gu[FF + i]);
        orc_quant_act_int8(h, FF, qx, sx);
        orc_gemv_q4b_a(dn_codes + (size_t)e * E * (FF / 2), dn_bscale + (size_t)e * E * (FF / 32), FF, E, qx, sx, de);
        for (int i = 0; i < E; i++) out[i] = fmaf(wt[k], de[i], out[i]);             /* dg_k_axpy, CF:13682-13685 */
    }
    free(xn); free(tmp); free(lg); free(gu); free(h); free(de); free(qx); free(sx); free(used); free(idx); free(wt);
    return 0;
}

/* ---------- Q4B block quantiser: documented recipe, PARITY UNPINNED ----------
 * sp_model.h:50-53, CF:1680-1687: per-32 block; the f16 scale is stored FIRST and the codes are
 * derived against the stored scale ("store-then-derive"), so w_hat = code * f16scale exactly;
 * codes in [-7, 7]; byte k of a row = weight 2k (low nibble) | weight 2k+1 (high nibble),
 * nibble = code & 0xF (4-bit two's complement). */
void orc_q4b_quantize(const float *w, int64_t rows, int cols, uint8_t *codes, uint16_t *bs) {
    const int nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < rows; j++) {
        const float *wr = w + j * cols;
        uint8_t *cr = codes + j * (cols / 2);
        for (int b = 0; b < nb; b++) {
            float m = 0.0f;
            for (int k = 0; k < 32; k++) { float a = fabsf(wr[b * 32 + k]); if (a > m) m = a; }
            const uint16_t hs = orc_float_to_half(m / 7.0f);
            bs[j * nb + b] = hs;
            const float s = orc_half_to_float(hs);
            for (int k = 0; k < 32; k += 2) {
                int q0 = 0, q1 = 0;
                if (s > 0.0f) {
                    q0 = (int)nearbyintf(wr[b * 32 + k] / s); q1 = (int)nearbyintf(wr[b * 32 + k + 1] / s);
                    if (q0 > 7) q0 = 7; if (q0 < -7) q0 = -7; if (q1 > 7) q1 = 7; if (q1 < -7) q1 = -7;
                }
                cr[(b * 32 + k) >> 1] = (uint8_t)((q0 & 0xF) | ((q1 & 0xF) << 4));
            }
        }
    }
}
void orc_q4b_dequantize(const uint8_t *codes, const uint16_t *bs, int64_t rows, int cols, float *w) {
    const int nb = cols / 32;
    for (int64_t j = 0; j < rows; j++)
        for (int i = 0; i < cols; i++)
            w[j * cols + i] = (float)nib_code(codes + j * (cols / 2), i) * orc_half_to_float(bs[j * nb + (i >> 5)]);
}

/* ---------- integer GEMM with per-row x per-col scales (ptx_mma.cuh:115-222; epilogue
 * ptx_mma_tile_common.cuh:157-176): C[m][n] = f16( float(sum_k A[m][k]*B[n][k]) * sa[m] * sb[n] ).
 * A is [M][K], B is [N][K] (the tiled kernels' layout), both already unpacked to int8. ---------- */
void orc_int_gemm_scaled(const int8_t *A, const int8_t *B, int M, int N, int K,
                         const float *scale_a, const float *scale_b, uint16_t *C_f16) {
#pragma omp parallel for schedule(static)
    for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            int32_t acc = 0;
            for (int k = 0; k < K; k++) acc += (int32_t)A[(size_t)m * K + k] * (int32_t)B[(size_t)n * K + k];
            float v = (float)acc * scale_a[m];
            v = v * scale_b[n];
            C_f16[(size_t)m * N + n] = orc_float_to_half(v);
        }
}
