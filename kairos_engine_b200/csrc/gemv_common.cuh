/* gemv_common.cuh — the two single-vector kernels the stand-alone entry points share (the reference's
 * gemv_w_packed pair for OK_Q4B, CF:13566-13599 of src/backends/cuda/cuda_forward.cu): the int8 per-16
 * activation quantiser and the Q4B x int8 GEMV, one warp per output row. */
#pragma once
#include "common.cuh"

/* k_quant_act_int8 (CF:1564-1585) into the de-interleaved layout q4b_chunk_dot expects */
static __global__ void k_quant_act(const float *x, int n, signed char *q, float *sx, int *corr) {
    for (int b = blockIdx.x * blockDim.x + threadIdx.x; b < (n >> 4); b += gridDim.x * blockDim.x) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = x[16 * b + i];
        sx[b] = quant_block16(v, q + 16 * b, corr + b);
    }
}
/* k_gemv_q4b_dp4a_v2 (CF:1688-1713): warp per row, chunk c in lane c%32, shuffle tree */
static __global__ void k_gemv_q4b(const uint8_t *codes, const uint16_t *bs, int in, int out,
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
