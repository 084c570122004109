/* quant.cu — Q4B block quantiser / dequantiser on device memory.
 *
 * Format (include/sp_engine/sp_model.h:50-53; CF:1448-1464, 1680-1687 of
 * src/backends/cuda/cuda_forward.cu): per-32 block, the f16 scale is stored first and the codes
 * are derived against the STORED scale, so w_hat = code * f16scale exactly; codes in [-7, 7];
 * byte k of a row = weight 2k (low nibble) | weight 2k+1 (high nibble), 4-bit two's complement.
 * The reference's own quantiser lives in a submodule outside its tree; only this documented
 * recipe is followed. The dequantiser is k_dequant_arena_q4b (CF:1452-1464).
 */
#include "common.cuh"
#include "../../include/sp_engine/moe_backend.h"

namespace {
/* one thread per 32-weight block: 128 B in, 16 B codes + one f16 out */
__global__ void k_q4b_quantize(const float *__restrict__ w, long long nblk, uint4 *__restrict__ codes, unsigned short *__restrict__ bs) {
    const long long b = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblk) return;
    const float4 *src = reinterpret_cast<const float4 *>(w + 32 * b);
    float v[32];
#pragma unroll
    for (int i = 0; i < 8; i++) { const float4 f = src[i]; v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w; }
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 32; i++) m = fmaxf(m, fabsf(v[i]));
    const __half hs = __float2half_rn(__fdiv_rn(m, 7.0f));
    bs[b] = __half_as_ushort(hs);
    const float s = __half2float(hs);
    unsigned word[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 32; i++) {
        int q = 0;
        if (s > 0.0f) { q = __float2int_rn(__fdiv_rn(v[i], s)); q = q > 7 ? 7 : q; q = q < -7 ? -7 : q; }
        word[i >> 3] |= (unsigned)(q & 0xF) << (4 * (i & 7));
    }
    codes[b] = make_uint4(word[0], word[1], word[2], word[3]);
}
__global__ void k_q4b_dequantize(const unsigned char *__restrict__ codes, const unsigned short *__restrict__ bs, long long n, float *__restrict__ w) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const unsigned char byte = codes[i >> 1];
    const int nib = (i & 1) ? (byte >> 4) : (byte & 0xF);
    w[i] = (float)((nib ^ 8) - 8) * h2f(bs[i >> 5]);
}
__global__ void k_gelu_mul_dev(const float *__restrict__ g, const float *__restrict__ up, long long n, float *__restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = gelu_mul(g[i], up[i]);
}
}  // namespace

extern "C" int sp_moe_q4b_quantize_dev(const float *w_dev, int64_t rows, int cols, uint8_t *codes_dev, uint16_t *bs_dev, void *stream) {
    if (!w_dev || !codes_dev || !bs_dev || rows <= 0 || cols <= 0 || (cols & 31)) { sp_set_error("sp_moe_q4b_quantize_dev: bad argument (cols must be a multiple of 32)"); return SP_MOE_EBADARG; }
    const long long nblk = rows * (long long)(cols / 32);
    k_q4b_quantize<<<(unsigned)((nblk + 127) / 128), 128, 0, (cudaStream_t)stream>>>(w_dev, nblk, reinterpret_cast<uint4 *>(codes_dev), bs_dev);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { sp_set_error(cudaGetErrorString(e)); return SP_MOE_ECUDA; }
    return SP_MOE_OK;
}
extern "C" int sp_moe_q4b_dequantize_dev(const uint8_t *codes_dev, const uint16_t *bs_dev, int64_t rows, int cols, float *w_dev, void *stream) {
    if (!w_dev || !codes_dev || !bs_dev || rows <= 0 || cols <= 0 || (cols & 31)) { sp_set_error("sp_moe_q4b_dequantize_dev: bad argument (cols must be a multiple of 32)"); return SP_MOE_EBADARG; }
    const long long n = rows * (long long)cols;
    k_q4b_dequantize<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(codes_dev, bs_dev, n, w_dev);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { sp_set_error(cudaGetErrorString(e)); return SP_MOE_ECUDA; }
    return SP_MOE_OK;
}
extern "C" int sp_moe_gelu_mul_dev(const float *g_dev, const float *up_dev, int64_t n, float *out_dev, void *stream) {
    if (!g_dev || !up_dev || !out_dev || n <= 0) { sp_set_error("sp_moe_gelu_mul_dev: bad argument"); return SP_MOE_EBADARG; }
    k_gelu_mul_dev<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(g_dev, up_dev, n, out_dev);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { sp_set_error(cudaGetErrorString(e)); return SP_MOE_ECUDA; }
    return SP_MOE_OK;
}
