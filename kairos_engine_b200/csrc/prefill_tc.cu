/* prefill_tc.cu — the prefill GEMMs of the MoE feed-forward layer on the 5th-generation tensor
 * cores (tcgen05.mma, accumulators in tensor memory), sm_100a only.
 *
 * Replaces the reference's prefill matmul for Q4B tensors (gemm_w, CF:13488-13518 of
 * src/backends/cuda/cuda_forward.cu: dequantise the whole tensor to a scratch matrix, then
 * cuBLAS) and its expert-major loop (gather / GEMM / GELU split / GEMM / scatter, CF:8925-8965)
 * with one grouped kernel per GEMM that dequantises Q4B tiles on the fly.
 *
 * Arithmetic. The reference multiplies w = code * f16 scale (exact in fp32, CF:1452-1464) by fp32
 * activations. fp16 operands alone cannot hold that (a 4-bit code times an 11-bit scale needs 14
 * bits; an fp32 activation 24), so both operands are split into two fp16 terms,
 *     w = w_hi + w_lo  (exact: w_hi = fp16(code*scale), w_lo = fma(code, scale, -w_hi)),
 *     x = x_hi + x_lo  (x_hi = fp16(x), x_lo = fp16(x - x_hi); |x - x_hi - x_lo| <= 2^-22 |x|),
 * and D += w_hi*x_hi + w_lo*x_hi + w_hi*x_lo accumulates in fp32 in tensor memory (the dropped
 * w_lo*x_lo term is below 2^-22 relative). That is three MMAs per k-step.
 *
 * Tile: 128 activation rows (the MMA's M: one TMEM lane per row) x 256 weight rows (its N: one
 * TMEM column per weight row), K in stages of 64. One 128x256x16 MMA reads 12 KB of operands from
 * shared memory per 128 tensor-core cycles; two 128x128x16 ones would read 16 KB, and shared-memory
 * bandwidth (operand reads + the unpack warps' writes + TMA) is what bounds this kernel.
 *   gate|up GEMM : columns [0,128) = 128 gate rows, columns [128,256) = the matching 128 up rows, so
 *                  the epilogue thread that owns a TMEM lane (one activation row) holds g and u of
 *                  the same outputs and writes gelu(g)*u directly, already split into fp16 hi/lo
 *                  for the next GEMM, 16 bytes at a time;
 *   down GEMM    : columns = weight rows [j0, j0+256), fp32 out, 16 bytes at a time.
 * Activation tiles come in by TMA (2-D tiled copy, 128-byte swizzle) from row lists sorted by
 * expert; weight tiles are unpacked by eight warps into the same swizzled layout. Inside every
 * group of 8 k the order is 0,4,1,5,2,6,3,7 on BOTH operands (the natural order of the nibble
 * unpack), which a dot product does not see.
 * Warp roles (14 warps): 0-3 epilogue (TMEM lane quadrant = warp), 4 TMA, 5 MMA issue + TMEM
 * allocation, 6-13 weight unpack. Two shared-memory stages, two accumulator sets (512 TMEM columns)
 * so the epilogue of one tile overlaps the main loop of the next. Every wait is bounded.
 */
#include <vector>
#include "prefill_tc.cuh"
#include "tc_common.cuh"

namespace {
using namespace sp_tc;

constexpr int kTileN = 128, kBK = 64, kStages = 2;
constexpr int kThreads = 448;
constexpr uint32_t kAHalf = 256 * 128, kBHalf = kTileN * 128;
constexpr uint32_t kStageBytes = 2 * kAHalf + 2 * kBHalf;             /* 98304 */
constexpr uint32_t kBarOff = kStages * kStageBytes;
constexpr uint32_t kSmemBytes = kBarOff + 128 + 1024;                 /* + alignment slack */

struct TcMaps { CUtensorMap hi, lo; };

struct TcArgs {
    const uint8_t *codes[2]; const uint16_t *bs[2];   /* weight tensor feeding accumulator 0 / 1 */
    long long group_rows;          /* rows per group (expert) in the tensor */
    int acc1_off;                  /* pair: row offset of accumulator 1's rows inside the group */
    int rows;                      /* valid output rows (pair: per accumulator) */
    int K;
    const int *tiles;              /* {group, first row, valid rows} per activation tile */
    const int *n_tiles;
    int m_tiles;
    __half *out_hi, *out_lo; int out_k;               /* pair: geglu output rows, split + permuted */
    float *out_f; int out_stride; const int *rowmap;  /* plain: out_f[(rowmap ? rowmap[r] : r) * stride + j] */
    int *status;
};

__device__ __forceinline__ int kpos(int e) { return ((e & 3) << 1) | (e >> 2); }     /* slot of element e inside its group of 8 */

/* one Q4B block (32 weights, one f16 scale) -> four 16-byte chunks of hi and (LO) of lo halves */
template <bool LO>
__device__ __forceinline__ void unpack_block(const int4 &w, unsigned short scale, unsigned char *a_hi, unsigned char *a_lo,
                                             uint32_t rowoff, int r7, int g0) {
    const __half2 s2 = __half2half2(__ushort_as_half(scale));
    const __half2 k1032 = __half2half2(__ushort_as_half((unsigned short)0x6408));
    const uint32_t words[4] = {(uint32_t)w.x, (uint32_t)w.y, (uint32_t)w.z, (uint32_t)w.w};
#pragma unroll
    for (int q = 0; q < 4; q++) {
        const uint32_t t = words[q] ^ 0x88888888u;
        uint32_t hi[4], lo[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t bits = ((t >> (4 * j)) & 0x000F000Fu) | 0x64006400u;        /* halves 1024 + (code + 8): elements j, j + 4 */
            const __half2 c = __hsub2(*reinterpret_cast<const __half2 *>(&bits), k1032);
            const __half2 h = __hmul2(c, s2);
            hi[j] = *reinterpret_cast<const uint32_t *>(&h);
            if (LO) { const __half2 l = __hfma2(c, s2, __hneg2(h)); lo[j] = *reinterpret_cast<const uint32_t *>(&l); }
        }
        const uint32_t off = rowoff + (uint32_t)(((g0 + q) ^ r7) << 4);
        *reinterpret_cast<uint4 *>(a_hi + off) = make_uint4(hi[0], hi[1], hi[2], hi[3]);
        if (LO) *reinterpret_cast<uint4 *>(a_lo + off) = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    }
}

/* TERMS: 3 = all of w_hi*x_hi + w_lo*x_hi + w_hi*x_lo (exact to 2^-22); 2 = the weight rounded to fp16
 * (w_hi*x_hi + w_hi*x_lo); 1 = fp16 x fp16, the reference's SP_G4_GEMM_F16 mode (CF:13350-13365). */
template <bool PAIR, int TERMS>
__global__ void __launch_bounds__(kThreads, 1) k_tc_gemm(const TcArgs a, const __grid_constant__ TcMaps maps) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char *smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const uint32_t sbase = smem_u32(smem);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t bar0 = sbase + kBarOff;
    auto full = [&](int s) { return bar0 + 8u * s; };
    auto empty = [&](int s) { return bar0 + 16u + 8u * s; };
    auto tfull = [&](int b) { return bar0 + 32u + 8u * b; };
    auto tempty = [&](int b) { return bar0 + 48u + 8u * b; };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + kBarOff + 64);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + kBarOff + 68);

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) { mbar_init(full(s), 9); mbar_init(empty(s), 1); }
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

    const int n_tiles = *a.n_tiles;
    const int total = n_tiles * a.m_tiles;
    const int KB = a.K / kBK;
    bool failed = false;

    if (warp == 4) {
        /* ---------------- activation tiles by TMA */
        if (lane == 0) {
            uint32_t it = 0;
            for (int w = blockIdx.x; w < total && !failed; w += gridDim.x) {
                const int nt = w / a.m_tiles;
                const int row0 = a.tiles[3 * nt + 1];
                for (int kb = 0; kb < KB; kb++, it++) {
                    const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
                    if (!mbar_wait(empty(s), ph ^ 1, abort_flag)) { failed = true; break; }
                    mbar_expect_tx(full(s), TERMS >= 2 ? 2 * kBHalf : kBHalf);
                    const uint32_t dst = sbase + s * kStageBytes + 2 * kAHalf;
                    tma_load_2d(dst, &maps.hi, kb * kBK, row0, full(s));
                    if (TERMS >= 2) tma_load_2d(dst + kBHalf, &maps.lo, kb * kBK, row0, full(s));
                }
            }
            if (failed || *abort_flag) __nanosleep(100000);          /* let copies in flight land before the CTA leaves */
        }
    } else if (warp == 5) {
        /* ---------------- MMA issue */
        if (lane == 0) {
            uint32_t it = 0, lt = 0;
            for (int w = blockIdx.x; w < total && !failed; w += gridDim.x, lt++) {
                const int nt = w / a.m_tiles;
                const uint32_t idesc = (1u << 4) | ((256u >> 3) << 17) | ((128u >> 4) << 24);   /* f16 x f16 -> f32, K-major both, M = 128, N = 256 */
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
                    for (int ks = 0; ks < kBK / 16; ks++) {
                        /* A operand = activation rows (M), B operand = the 256 weight rows (N) */
                        const uint64_t whi = make_desc(st + ks * 32), wlo = make_desc(st + kAHalf + ks * 32);
                        const uint64_t xhi = make_desc(st + 2 * kAHalf + ks * 32), xlo = make_desc(st + 2 * kAHalf + kBHalf + ks * 32);
                        umma_f16(d0, xhi, whi, idesc, (kb | ks) ? 1u : 0u);
                        if (TERMS >= 3) umma_f16(d0, xhi, wlo, idesc, 1u);
                        if (TERMS >= 2) umma_f16(d0, xlo, whi, idesc, 1u);
                    }
                    umma_commit(empty(s));                          /* stage reusable once these MMAs have read it */
                }
                if (!failed) umma_commit(tfull(b));
            }
        }
    } else if (warp >= 6) {
        /* ---------------- weight tiles: Q4B -> fp16 hi/lo, swizzled K-major rows */
        const int r = (warp - 6) * 32 + lane;
        const int acc = r >> 7, i = r & 127, r7 = r & 7;
        const uint32_t rowoff = (uint32_t)r * 128u;
        const size_t rb = (size_t)a.K / 2; const int n32 = a.K / 32;
        uint32_t it = 0;
        for (int w = blockIdx.x; w < total && !failed; w += gridDim.x) {
            const int nt = w / a.m_tiles, mt = w - nt * a.m_tiles;
            const int grp = a.tiles[3 * nt];
            int jj = PAIR ? mt * 128 + i : mt * 256 + r;
            if (jj > a.rows - 1) jj = a.rows - 1;
            const size_t wrow = (size_t)((long long)grp * a.group_rows) + (size_t)(PAIR ? acc * a.acc1_off : 0) + (size_t)jj;
            const int tsel = PAIR ? acc : 0;
            const unsigned char *cp = a.codes[tsel] + wrow * rb;
            const uint16_t *sp = a.bs[tsel] + wrow * n32;
            int4 c0 = ld_stream16(cp), c1 = ld_stream16(cp + 16);
            uint32_t sc = *reinterpret_cast<const uint32_t *>(sp);
            for (int kb = 0; kb < KB; kb++, it++) {
                const int4 w0 = c0, w1 = c1; const uint32_t s2 = sc;
                if (kb + 1 < KB) { c0 = ld_stream16(cp + 32 * (kb + 1)); c1 = ld_stream16(cp + 32 * (kb + 1) + 16); sc = *reinterpret_cast<const uint32_t *>(sp + 2 * (kb + 1)); }
                const int s = it % kStages; const uint32_t ph = (it / kStages) & 1;
                if (!mbar_wait(empty(s), ph ^ 1, abort_flag)) { failed = true; break; }
                unsigned char *ahi = smem + s * kStageBytes, *alo = ahi + kAHalf;
                unpack_block<TERMS >= 3>(w0, (unsigned short)(s2 & 0xFFFFu), ahi, alo, rowoff, r7, 0);
                unpack_block<TERMS >= 3>(w1, (unsigned short)(s2 >> 16), ahi, alo, rowoff, r7, 4);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(full(s));
            }
        }
    } else {
        /* ---------------- epilogue: TMEM -> registers -> global */
        const int i = warp * 32 + lane;                             /* TMEM lane = activation row inside the tile */
        uint32_t lt = 0;
        for (int w = blockIdx.x; w < total && !failed; w += gridDim.x, lt++) {
            const int nt = w / a.m_tiles, mt = w - nt * a.m_tiles;
            const int row0 = a.tiles[3 * nt + 1], nv = a.tiles[3 * nt + 2];
            const int b = lt & 1; const uint32_t bph = (lt >> 1) & 1;
            if (!mbar_wait(tfull(b), bph, abort_flag)) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t t0 = tmem + ((uint32_t)(warp * 32) << 16) + (uint32_t)(b * 256);
            const bool rv = i < nv;
            const int sr = row0 + (rv ? i : 0);
            if (PAIR) {
                __half *ohi = a.out_hi + (size_t)sr * a.out_k, *olo = a.out_lo + (size_t)sr * a.out_k;
                for (int c0 = 0; c0 < 128; c0 += 16) {
                    const int j0 = mt * 128 + c0;
                    if (j0 >= a.rows) break;                             /* warp-uniform */
                    uint32_t g[16], u[16];
                    tmem_ld16(t0 + c0, g);
                    tmem_ld16(t0 + 128 + c0, u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (rv) {
#pragma unroll
                        for (int h8 = 0; h8 < 2; h8++) {
                            if (j0 + 8 * h8 < a.rows) {                  /* rows is a multiple of 8 */
                                __half hh[8], hl[8];
#pragma unroll
                                for (int n = 0; n < 8; n++) {
                                    const float h = gelu_mul(__uint_as_float(g[8 * h8 + n]), __uint_as_float(u[8 * h8 + n]));
                                    const __half x = __float2half_rn(h);
                                    hh[kpos(n)] = x; hl[kpos(n)] = __float2half_rn(__fsub_rn(h, __half2float(x)));
                                }
                                *reinterpret_cast<uint4 *>(ohi + j0 + 8 * h8) = *reinterpret_cast<const uint4 *>(hh);
                                *reinterpret_cast<uint4 *>(olo + j0 + 8 * h8) = *reinterpret_cast<const uint4 *>(hl);
                            }
                        }
                    }
                }
            } else {
                float *orow = a.out_f + (size_t)(a.rowmap ? __ldg(a.rowmap + sr) : sr) * a.out_stride;
                for (int c0 = 0; c0 < 256; c0 += 16) {
                    const int j0 = mt * 256 + c0;
                    if (j0 >= a.rows) break;                             /* warp-uniform */
                    uint32_t v[16];
                    tmem_ld16(t0 + c0, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (rv) {
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            if (j0 + 4 * q < a.rows)                     /* rows is a multiple of 4 */
                                *reinterpret_cast<float4 *>(orow + j0 + 4 * q) =
                                    make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]), __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(tempty(b));
        }
    }
    if (failed && lane == 0) atomicExch(a.status, SP_KERR_BARRIER_TIMEOUT);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        if (*abort_flag) __nanosleep(100000);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

/* ---------------------------------------------------------------- helpers around the GEMM */
/* fp32 rows -> fp16 hi/lo rows, k order 0,4,1,5,2,6,3,7 inside each group of 8; one block per row */
__global__ void __launch_bounds__(256) k_tc_split(const float *src, const int *gather, int K, __half *hi, __half *lo) {
    const size_t r = blockIdx.x;
    const float *x = src + (size_t)(gather ? gather[r] : (int)r) * K;
    for (int c = threadIdx.x; c < K / 8; c += 256) {
        const float4 a = *reinterpret_cast<const float4 *>(x + 8 * c), b = *reinterpret_cast<const float4 *>(x + 8 * c + 4);
        const float v[8] = {a.x, b.x, a.y, b.y, a.z, b.z, a.w, b.w};
        __half h[8], l[8];
#pragma unroll
        for (int k = 0; k < 8; k++) { h[k] = __float2half_rn(v[k]); l[k] = __float2half_rn(__fsub_rn(v[k], __half2float(h[k]))); }
        *reinterpret_cast<uint4 *>(hi + r * K + 8 * c) = *reinterpret_cast<const uint4 *>(h);
        *reinterpret_cast<uint4 *>(lo + r * K + 8 * c) = *reinterpret_cast<const uint4 *>(l);
    }
}
/* block-wide inclusive scan of one int per thread (1024 threads) */
__device__ __forceinline__ int scan1024(int v, int *sh) {
    const int t = threadIdx.x;
    sh[t] = v;
    __syncthreads();
    for (int dlt = 1; dlt < 1024; dlt <<= 1) { const int u = t >= dlt ? sh[t - dlt] : 0; __syncthreads(); sh[t] += u; __syncthreads(); }
    return sh[t];
}
/* activation tiles: each group's rows in the fewest tiles of at most 128 rows, evenly sized. One thread per
 * group (groups <= 1024) counts its tiles, a scan places them, each thread writes its own. Row ranges are
 * clamped to [0, max_rows]: offsets come from the caller (or from counts another GPU sent). */
__global__ void __launch_bounds__(1024) k_tc_plan(const int *offsets, int groups, int fixed_rows, int max_rows, int *tiles, int *n_tiles, int cap) {
    __shared__ int sh[1024];
    const int g = threadIdx.x;
    int first = 0, cnt = 0;
    if (g < groups) {
        first = offsets ? offsets[g] : 0;
        int last = offsets ? offsets[g + 1] : fixed_rows;
        first = first < 0 ? 0 : (first > max_rows ? max_rows : first);
        last = last < first ? first : (last > max_rows ? max_rows : last);
        cnt = last - first;
    }
    const int nt = cnt > 0 ? (cnt + kTileN - 1) / kTileN : 0;
    const int per = nt > 0 ? ((((cnt + nt - 1) / nt) + 15) & ~15) : 0;
    int mine = 0;
    for (int i = 0; i < nt; i++) if (cnt - i * per > 0) mine++;
    const int end = scan1024(mine, sh);
    int n = end - mine;
    for (int i = 0; i < mine && n < cap; i++, n++) {
        const int left = cnt - i * per;
        tiles[3 * n] = g; tiles[3 * n + 1] = first + i * per; tiles[3 * n + 2] = left < per ? left : per;
    }
    if (g == 1023) *n_tiles = end < cap ? end : cap;
}
__global__ void __launch_bounds__(1024) k_tc_scan(const int *count, int groups, int *offsets) {
    __shared__ int sh[1024];
    const int g = threadIdx.x;
    const int end = scan1024(g < groups ? count[g] : 0, sh);
    if (g < groups) offsets[g + 1] = end;
    if (g == 0) offsets[0] = 0;
}
__global__ void __launch_bounds__(256) k_tc_pairs(const int *sel_asc, const int *pairpos, const int *offsets, int n_pairs, int NU, int *gather, int *rowmap) {
    const int p = blockIdx.x * 256 + threadIdx.x;
    if (p >= n_pairs) return;
    const int row = offsets[sel_asc[p]] + pairpos[p];
    gather[row] = p / NU; rowmap[row] = p;
}

}  // namespace

/* ---------------------------------------------------------------- host side */
struct SpTcPlan {
    int Mcap, Rcap, sms;
    unsigned char *base; size_t bytes;
    __half *nx_hi, *nx_lo, *hd_hi, *hd_lo, *in_hi, *in_lo, *h_hi, *h_lo;
    int *tiles_sh, *ntiles_sh, *tiles_r, *ntiles_r, *offsets, *gather, *rowmap;
    int cap_sh, cap_r;
    int terms;                                         /* MMAs per k-step: 3, 2 or 1 */
    TcMaps m_nx, m_hd, m_in, m_h;
};

bool sp_tc_supported(const SpDims &d) { return (d.E % 64 == 0) && (d.FFE % 64 == 0) && (d.FFS % 64 == 0); }

namespace {
cudaError_t make_map(sp_tc::EncodeTiledFn fn, CUtensorMap *m, void *ptr, int K, int rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kTileN};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}
size_t up256(size_t v) { return (v + 255) & ~(size_t)255; }
}  // namespace

cudaError_t sp_tc_create(const SpDims &d, int max_tokens, int max_rows, SpTcPlan **out, size_t *bytes) {
    *out = nullptr; *bytes = 0;
    if (!sp_tc_supported(d)) return cudaSuccess;
    sp_tc::EncodeTiledFn fn = nullptr;
    cudaError_t e = sp_tc::encode_tiled_fn(&fn);
    if (e != cudaSuccess) return e;
    SpTcPlan *p = new SpTcPlan();
    p->Mcap = ((max_tokens + kTileN - 1) / kTileN) * kTileN;
    p->Rcap = (int)((((long long)max_rows + kTileN - 1) / kTileN) * kTileN);
    int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&p->sms, cudaDevAttrMultiProcessorCount, dev);
    p->cap_sh = p->Mcap / kTileN + 2; p->cap_r = p->Rcap / kTileN + d.NE + 2;
    size_t o = 0; auto take = [&](size_t b) { size_t at = o; o = up256(o + b); return at; };
    const size_t E = d.E, FFE = d.FFE, FFS = d.FFS;
    const size_t o_nxh = take(2 * p->Mcap * E), o_nxl = take(2 * p->Mcap * E), o_hdh = take(2 * p->Mcap * FFS), o_hdl = take(2 * p->Mcap * FFS);
    const size_t o_inh = take(2 * p->Rcap * E), o_inl = take(2 * p->Rcap * E), o_hh = take(2 * p->Rcap * FFE), o_hl = take(2 * p->Rcap * FFE);
    const size_t o_tsh = take(12 * (size_t)p->cap_sh), o_nsh = take(4), o_tr = take(12 * (size_t)p->cap_r), o_nr = take(4);
    const size_t o_off = take(4 * ((size_t)d.NE + 1)), o_g = take(4 * (size_t)p->Rcap), o_rm = take(4 * (size_t)p->Rcap);
    p->bytes = o;
    e = cudaMalloc((void **)&p->base, o);
    if (e != cudaSuccess) { delete p; return e; }
    cudaMemset(p->base, 0, o);
    unsigned char *b = p->base;
    p->nx_hi = (__half *)(b + o_nxh); p->nx_lo = (__half *)(b + o_nxl); p->hd_hi = (__half *)(b + o_hdh); p->hd_lo = (__half *)(b + o_hdl);
    p->in_hi = (__half *)(b + o_inh); p->in_lo = (__half *)(b + o_inl); p->h_hi = (__half *)(b + o_hh); p->h_lo = (__half *)(b + o_hl);
    p->tiles_sh = (int *)(b + o_tsh); p->ntiles_sh = (int *)(b + o_nsh); p->tiles_r = (int *)(b + o_tr); p->ntiles_r = (int *)(b + o_nr);
    p->offsets = (int *)(b + o_off); p->gather = (int *)(b + o_g); p->rowmap = (int *)(b + o_rm);
    cudaError_t m = cudaSuccess;
    auto mk = [&](CUtensorMap *t, void *ptr, int K, int rows) { if (m == cudaSuccess) m = make_map(fn, t, ptr, K, rows); };
    mk(&p->m_nx.hi, p->nx_hi, d.E, p->Mcap); mk(&p->m_nx.lo, p->nx_lo, d.E, p->Mcap);
    mk(&p->m_hd.hi, p->hd_hi, d.FFS, p->Mcap); mk(&p->m_hd.lo, p->hd_lo, d.FFS, p->Mcap);
    mk(&p->m_in.hi, p->in_hi, d.E, p->Rcap); mk(&p->m_in.lo, p->in_lo, d.E, p->Rcap);
    mk(&p->m_h.hi, p->h_hi, d.FFE, p->Rcap); mk(&p->m_h.lo, p->h_lo, d.FFE, p->Rcap);
    if (m == cudaSuccess) m = cudaFuncSetAttribute(k_tc_gemm<true, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (m == cudaSuccess) m = cudaFuncSetAttribute(k_tc_gemm<false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (m == cudaSuccess) m = cudaFuncSetAttribute(k_tc_gemm<true, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (m == cudaSuccess) m = cudaFuncSetAttribute(k_tc_gemm<false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (m == cudaSuccess) m = cudaFuncSetAttribute(k_tc_gemm<true, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (m == cudaSuccess) m = cudaFuncSetAttribute(k_tc_gemm<false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    /* house convention: behaviour switches are SP_* variables read once. 3 (default) keeps every product the fp32
     * reference arithmetic sees down to 2^-22; 2 rounds the dequantised weight to fp16; 1 also rounds the activation. */
    const char *tv = getenv("SP_MOE_PREFILL_TERMS");
    p->terms = tv ? atoi(tv) : 3;
    if (p->terms < 1 || p->terms > 3) p->terms = 3;
    if (m != cudaSuccess) { cudaFree(p->base); delete p; return m; }
    *out = p; *bytes = o;
    return cudaSuccess;
}
void sp_tc_destroy(SpTcPlan *p) { if (!p) return; if (p->base) cudaFree(p->base); delete p; }

namespace {
template <bool PAIR>
void launch_gemm(const SpTcPlan *p, const TcArgs &a, const TcMaps &maps, cudaStream_t st, int *nl) {
    if (p->terms == 3) k_tc_gemm<PAIR, 3><<<p->sms, kThreads, kSmemBytes, st>>>(a, maps);
    else if (p->terms == 2) k_tc_gemm<PAIR, 2><<<p->sms, kThreads, kSmemBytes, st>>>(a, maps);
    else k_tc_gemm<PAIR, 1><<<p->sms, kThreads, kSmemBytes, st>>>(a, maps);
    (*nl)++;
}
}  // namespace

cudaError_t sp_tc_shared_expert(SpTcPlan *p, const SpDims &d, const SpLayerDev &L, int M, const float *nx, float *dn,
                                int *status, cudaStream_t st, int *nl, int phase) {
    if (!p || M > p->Mcap) return cudaErrorInvalidValue;
    if (phase != 2) {                                     /* gate/up + GeGLU -> hd (split fp16), kept in the plan's scratch */
        k_tc_split<<<M, 256, 0, st>>>(nx, nullptr, d.E, p->nx_hi, p->nx_lo); (*nl)++;
        k_tc_plan<<<1, 1024, 0, st>>>(nullptr, 1, M, M, p->tiles_sh, p->ntiles_sh, p->cap_sh); (*nl)++;
        TcArgs a{};
        a.codes[0] = L.sg_codes; a.bs[0] = L.sg_bs; a.codes[1] = L.su_codes; a.bs[1] = L.su_bs;
        a.group_rows = 0; a.acc1_off = 0; a.rows = d.FFS; a.K = d.E; a.tiles = p->tiles_sh; a.n_tiles = p->ntiles_sh;
        a.m_tiles = (d.FFS + 127) / 128; a.out_hi = p->hd_hi; a.out_lo = p->hd_lo; a.out_k = d.FFS; a.status = status;
        launch_gemm<true>(p, a, p->m_nx, st, nl);
    }
    if (phase != 1) {                                     /* down: hd -> dn (the tile table of the first phase is still in place) */
        TcArgs b{};
        b.codes[0] = b.codes[1] = L.sd_codes; b.bs[0] = b.bs[1] = L.sd_bs;
        b.group_rows = 0; b.rows = d.E; b.K = d.FFS; b.tiles = p->tiles_sh; b.n_tiles = p->ntiles_sh;
        b.m_tiles = (d.E + 255) / 256; b.out_f = dn; b.out_stride = d.E; b.rowmap = nullptr; b.status = status;
        launch_gemm<false>(p, b, p->m_hd, st, nl);
    }
    return cudaGetLastError();
}

cudaError_t sp_tc_routed(SpTcPlan *p, const SpDims &d, const SpLayerDev &L, int R, const float *src, const int *gather,
                         const int *offsets, const int *rowmap, float *out, int *status, cudaStream_t st, int *nl) {
    if (!p || R > p->Rcap) return cudaErrorInvalidValue;
    if (R == 0) return cudaSuccess;
    k_tc_split<<<R, 256, 0, st>>>(src, gather, d.E, p->in_hi, p->in_lo); (*nl)++;
    k_tc_plan<<<1, 1024, 0, st>>>(offsets, d.NE, 0, R, p->tiles_r, p->ntiles_r, p->cap_r); (*nl)++;
    TcArgs a{};
    a.codes[0] = a.codes[1] = L.gu_codes; a.bs[0] = a.bs[1] = L.gu_bs;
    a.group_rows = 2LL * d.FFE; a.acc1_off = d.FFE; a.rows = d.FFE; a.K = d.E; a.tiles = p->tiles_r; a.n_tiles = p->ntiles_r;
    a.m_tiles = (d.FFE + 127) / 128; a.out_hi = p->h_hi; a.out_lo = p->h_lo; a.out_k = d.FFE; a.status = status;
    launch_gemm<true>(p, a, p->m_in, st, nl);
    TcArgs b{};
    b.codes[0] = b.codes[1] = L.dn_codes; b.bs[0] = b.bs[1] = L.dn_bs;
    b.group_rows = d.E; b.rows = d.E; b.K = d.FFE; b.tiles = p->tiles_r; b.n_tiles = p->ntiles_r;
    b.m_tiles = (d.E + 255) / 256; b.out_f = out; b.out_stride = d.E; b.rowmap = rowmap; b.status = status;
    launch_gemm<false>(p, b, p->m_h, st, nl);
    return cudaGetLastError();
}

cudaError_t sp_tc_sort_pairs(SpTcPlan *p, const SpDims &d, int M, const int *sel_asc, const int *count, const int *pairpos,
                             const int **offsets, const int **gather, const int **rowmap, cudaStream_t st, int *nl) {
    if (!p || (long long)M * d.NU > p->Rcap) return cudaErrorInvalidValue;
    k_tc_scan<<<1, 1024, 0, st>>>(count, d.NE, p->offsets); (*nl)++;
    const int np = M * d.NU;
    k_tc_pairs<<<(np + 255) / 256, 256, 0, st>>>(sel_asc, pairpos, p->offsets, np, d.NU, p->gather, p->rowmap); (*nl)++;
    *offsets = p->offsets; *gather = p->gather; *rowmap = p->rowmap;
    return cudaGetLastError();
}
