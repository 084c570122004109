/* int_gemm_tc.cu — the reference's quantised PTX-MMA GEMM on tcgen05:
 *     C[m][n] (f16) = f16( float(sum_k A[m][k] * B[n][k]) * scale_a[m] * scale_b[n] )
 * int8 (or packed signed int4) operands, int32 accumulate, per-row x per-column fp32 scales.
 * Replaces sp_frob_matmul_q8_mma_tile / sp_frob_matmul_q4_mma_* (src/backends/cuda/ptx_mma.cuh:
 * 115-222, 268-353; ptx_mma_tile_int8.cuh:92-110; epilogue ptx_mma_tile_common.cuh:157-176), which
 * tile mma.sync m8n8k16 / m8n8k32 per warp. Here: tcgen05.mma kind::i8 (128 x 256 x 32 per
 * instruction), both operands by TMA into 128-byte-swizzled K-major tiles, int32 accumulators in
 * tensor memory (two sets: the epilogue of one tile overlaps the main loop of the next), the same
 * epilogue arithmetic and operation order, so results are bit-identical to the reference's.
 * A is [M][K], B is [N][K] (the tiled kernels' layout); K a multiple of 16.
 * Warp roles: 0-3 epilogue, 4 TMA, 5 MMA issue + TMEM allocation. Every wait is bounded.
 */
#include <mutex>
#include "tc_common.cuh"
#include "../../include/sp_engine/moe_backend.h"

namespace {
using namespace sp_tc;

constexpr int kTM = 128, kTN = 256, kBKB = 128, kStages = 4, kThreads = 192, kMaxDevices = 64;
constexpr uint32_t kABytes = kTM * 128, kBBytes = kTN * 128, kStageBytes = kABytes + kBBytes;   /* 16 KB + 32 KB */
constexpr uint32_t kBarOff = kStages * kStageBytes, kSmemBytes = kBarOff + 192 + 1024;

struct IgMaps { CUtensorMap a, b; };

__global__ void __launch_bounds__(kThreads, 1) k_i8_gemm(const __grid_constant__ IgMaps maps, const float *scale_a, const float *scale_b,
                                                         __half *C, int M, int K, int N, int *status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = sbase + kBarOff;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 32u + 8u * s; };
    auto tfull = [&](int b) { return bar0 + 64u + 8u * b; };
    auto tempty = [&](int b) { return bar0 + 80u + 8u * b; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kBarOff + 96);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + kBarOff + 100);
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) { mbar_init(full(s), 1); mbar_init(empty(s), 1); }
        for (int b = 0; b < 2; b++) { mbar_init(tfull(b), 1); mbar_init(tempty(b), 4); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void *)tmem_slot)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    const int tn = (N + kTN - 1) / kTN, total = ((M + kTM - 1) / kTM) * tn, KB = (K + kBKB - 1) / kBKB;
    bool failed = false;

    if (warp == 4) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int w = blockIdx.x; w < total && !failed; w += gridDim.x) {
                const int m0 = (w / tn) * kTM, n0 = (w % tn) * kTN;
                for (int kb = 0; kb < KB; kb++, it++) {
                    const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
                    if (!mbar_wait(empty(s), ph ^ 1, abort_flag)) { failed = true; break; }
                    mbar_expect_tx(full(s), kStageBytes);               /* rows or k beyond the matrices arrive as zeros */
                    const uint32_t dst = sbase + s * kStageBytes;
                    tma_load_2d(dst, &maps.a, kb * kBKB, m0, full(s));
                    tma_load_2d(dst + kABytes, &maps.b, kb * kBKB, n0, full(s));
                }
            }
            if (failed || *abort_flag) __nanosleep(100000);
        }
    } else if (warp == 5) {
        if (lane == 0) {
            /* s8 x s8 -> s32: c_format 2, a/b_format 1 (signed 8-bit), K-major both, N = 256, M = 128 */
            const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
            uint32_t it = 0, lt = 0;
            for (int w = blockIdx.x; w < total && !failed; w += gridDim.x, lt++) {
                const int b = lt & 1; const uint32_t bph = (lt >> 1) & 1;
                if (!mbar_wait(tempty(b), bph ^ 1, abort_flag)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d0 = tmem + (uint32_t)(b * 256);
                for (int kb = 0; kb < KB; kb++, it++) {
                    const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
                    if (!mbar_wait(full(s), ph, abort_flag)) { failed = true; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t st = sbase + s * kStageBytes;
#pragma unroll
                    for (int ks = 0; ks < kBKB / 32; ks++)
                        umma_i8(d0, make_desc(st + ks * 32), make_desc(st + kABytes + ks * 32), idesc, (kb | ks) ? 1u : 0u);
                    umma_commit(empty(s));
                }
                if (!failed) umma_commit(tfull(b));
            }
        }
    } else {
        /* epilogue (ptx_mma_tile_common.cuh:157-176): f16(float(acc) * sa[row] * sb[col]), left to right */
        const int i = warp * 32 + lane;
        const bool vec = (N & 7) == 0;
        uint32_t lt = 0;
        for (int w = blockIdx.x; w < total && !failed; w += gridDim.x, lt++) {
            const int m0 = (w / tn) * kTM, n0 = (w % tn) * kTN;
            const int b = lt & 1; const uint32_t bph = (lt >> 1) & 1;
            if (!mbar_wait(tfull(b), bph, abort_flag)) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t0 = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(b * 256);
            const int m = m0 + i; const bool rv = m < M;
            const float sa = rv ? __ldg(scale_a + m) : 0.0f;
            __half *crow = C + (size_t)(rv ? m : 0) * N;
            for (int c0 = 0; c0 < kTN; c0 += 16) {
                const int nb = n0 + c0;
                if (nb >= N) break;                                      /* warp-uniform */
                uint32_t v[16];
                tmem_ld16(t0 + c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (rv) {
                    __half o[16];
#pragma unroll
                    for (int n = 0; n < 16; n++) {
                        const float sb = nb + n < N ? __ldg(scale_b + nb + n) : 0.0f;
                        o[n] = __float2half_rn(__fmul_rn(__fmul_rn(__int2float_rn((int)v[n]), sa), sb));
                    }
                    if (vec && nb + 16 <= N) {
                        *reinterpret_cast<uint4 *>(crow + nb) = *reinterpret_cast<const uint4 *>(o);
                        *reinterpret_cast<uint4 *>(crow + nb + 8) = *reinterpret_cast<const uint4 *>(o + 8);
                    } else {
#pragma unroll
                        for (int n = 0; n < 16; n++) if (nb + n < N) crow[nb + n] = o[n];
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty(b));
        }
    }
    if (failed && lane == 0) atomicExch(status, SP_KERR_BARRIER_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        if (*abort_flag) __nanosleep(100000);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

/* packed signed int4 (low nibble = even index, nib >= 8 -> nib - 16; ptx_mma.cuh:375-385) -> int8 */
__global__ void __launch_bounds__(256) k_unpack_s4(const uint8_t *src, int8_t *dst, size_t n_bytes) {
    for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n_bytes; i += (size_t)gridDim.x * 256) {
        const unsigned b = src[i];
        const int lo = (int)(b & 0xFu), hi = (int)(b >> 4);
        reinterpret_cast<char2 *>(dst)[i] = make_char2((char)(lo >= 8 ? lo - 16 : lo), (char)(hi >= 8 ? hi - 16 : hi));
    }
}

int ig_fail(int code, const char *msg) { sp_set_error(msg); return code; }

cudaError_t make_u8_map(EncodeTiledFn fn, CUtensorMap *m, const void *ptr, int K, int rows, int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K};
    const cuuint32_t box[2] = {(cuuint32_t)kBKB, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

int run_q8(const int8_t *A, const int8_t *B, const float *sa, const float *sb, uint16_t *C, int M, int K, int N, cudaStream_t st, const char *who, int **status_out = nullptr) {
    if (!A || !B || !sa || !sb || !C) return ig_fail(SP_MOE_EBADARG, "quantised GEMM: NULL argument");
    if (M <= 0 || N <= 0 || K <= 0 || (K & 15)) return ig_fail(SP_MOE_EBADARG, "quantised GEMM: M, N, K must be positive and K a multiple of 16");
    if (((uintptr_t)A | (uintptr_t)B) & 15) return ig_fail(SP_MOE_EBADARG, "quantised GEMM: operand pointers must be 16-byte aligned");
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return ig_fail(SP_MOE_ECUDA, "quantised GEMM: no CUDA device");
    EncodeTiledFn fn = nullptr;
    if (encode_tiled_fn(&fn) != cudaSuccess) return ig_fail(SP_MOE_EUNSUPPORTED, "quantised GEMM: cuTensorMapEncodeTiled is not available");
    IgMaps maps;
    if (make_u8_map(fn, &maps.a, A, K, M, kTM) != cudaSuccess || make_u8_map(fn, &maps.b, B, K, N, kTN) != cudaSuccess)
        return ig_fail(SP_MOE_EBADARG, "quantised GEMM: could not describe the operands to the TMA unit");
    static std::mutex mu;                                 /* one error word and one attribute call per device, at first use there */
    static int *status_of[kMaxDevices] = {};
    if (dev < 0 || dev >= kMaxDevices) return ig_fail(SP_MOE_EUNSUPPORTED, "quantised GEMM: device ordinal out of range");
    int *status = nullptr;
    {
        std::lock_guard<std::mutex> lk(mu);
        if (!status_of[dev]) {
            int *p = nullptr;
            if (cudaFuncSetAttribute(k_i8_gemm, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes) != cudaSuccess) return ig_fail(SP_MOE_ECUDA, "quantised GEMM: shared-memory attribute");
            if (cudaMalloc((void **)&p, 256) != cudaSuccess || cudaMemset(p, 0, 256) != cudaSuccess) { if (p) cudaFree(p); return ig_fail(SP_MOE_ECUDA, "quantised GEMM: status word allocation failed"); }
            status_of[dev] = p;
        }
        status = status_of[dev];
    }
    const int tiles = ((M + kTM - 1) / kTM) * ((N + kTN - 1) / kTN);
    k_i8_gemm<<<tiles < sms ? tiles : sms, kThreads, kSmemBytes, st>>>(maps, sa, sb, reinterpret_cast<__half *>(C), M, K, N, status);
    (void)who;
    if (cudaGetLastError() != cudaSuccess) return ig_fail(SP_MOE_ECUDA, "quantised GEMM: kernel launch failed");
    if (status_out) *status_out = status;
    return SP_MOE_OK;
}

/* After the stream has drained: a bounded wait that ran out inside the kernel left a non-zero word. */
int read_status(int *status) {
    int v = 0;
    if (cudaMemcpy(&v, status, sizeof v, cudaMemcpyDeviceToHost) != cudaSuccess) return ig_fail(SP_MOE_ECUDA, "quantised GEMM: status read failed");
    if (v) { cudaMemset(status, 0, sizeof v); return ig_fail(SP_MOE_ECUDA, "quantised GEMM: a bounded wait inside the kernel ran out"); }
    return SP_MOE_OK;
}

}  // namespace

extern "C" int sp_frob_matmul_q8_dev(const int8_t *A_dev, const int8_t *B_dev, const float *scale_a_dev, const float *scale_b_dev,
                                     uint16_t *C_f16_dev, int M, int K, int N, void *stream) {
    return run_q8(A_dev, B_dev, scale_a_dev, scale_b_dev, C_f16_dev, M, K, N, (cudaStream_t)stream, "sp_frob_matmul_q8_dev");
}

extern "C" int sp_frob_matmul_q4_dev(const uint8_t *A_q4_dev, const uint8_t *B_q4_dev, const float *scale_a_dev, const float *scale_b_dev,
                                     uint16_t *C_f16_dev, int M, int K, int N, void *stream) {
    if (!A_q4_dev || !B_q4_dev) return ig_fail(SP_MOE_EBADARG, "sp_frob_matmul_q4_dev: NULL argument");
    if (M <= 0 || N <= 0 || K <= 0 || (K & 15)) return ig_fail(SP_MOE_EBADARG, "sp_frob_matmul_q4_dev: M, N, K must be positive and K a multiple of 16");
    cudaStream_t st = (cudaStream_t)stream;
    int8_t *a8 = nullptr, *b8 = nullptr;
    if (cudaMalloc((void **)&a8, (size_t)M * K) != cudaSuccess || cudaMalloc((void **)&b8, (size_t)N * K) != cudaSuccess) {
        if (a8) cudaFree(a8);
        cudaGetLastError();
        return ig_fail(SP_MOE_EBACKEND_OOM, "sp_frob_matmul_q4_dev: scratch allocation failed");
    }
    k_unpack_s4<<<1024, 256, 0, st>>>(A_q4_dev, a8, (size_t)M * K / 2);
    k_unpack_s4<<<1024, 256, 0, st>>>(B_q4_dev, b8, (size_t)N * K / 2);
    int *status = nullptr;
    int rc = run_q8(a8, b8, scale_a_dev, scale_b_dev, C_f16_dev, M, K, N, st, "sp_frob_matmul_q4_dev", &status);
    const cudaError_t se = cudaStreamSynchronize(st);      /* the scratch is freed below, so the stream is drained here anyway */
    cudaFree(a8); cudaFree(b8);
    if (rc == SP_MOE_OK && se != cudaSuccess) rc = ig_fail(SP_MOE_ECUDA, "sp_frob_matmul_q4_dev: the stream reported an error");
    if (rc == SP_MOE_OK) rc = read_status(status);
    return rc;
}
