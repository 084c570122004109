/* prefill_tc.cuh — launch interface of the tensor-core prefill GEMMs (prefill_tc.cu): grouped
 * Q4B-weight x fp16-split-activation GEMMs on tcgen05 with TMEM accumulators. */
#pragma once
#include "common.cuh"

struct SpTcPlan;     /* buffers, tile tables and TMA descriptors; host object */

/* K dimensions must be multiples of 64 (one 128-byte swizzled shared-memory row of fp16) */
bool sp_tc_supported(const SpDims &d);
cudaError_t sp_tc_create(const SpDims &d, int max_tokens, int max_rows, SpTcPlan **out, size_t *bytes);
void sp_tc_destroy(SpTcPlan *p);

/* shared expert: nx [M][E] f32 (normalised input) -> dn [M][E] f32 = Wd . geglu(Wg nx, Wu nx) */
cudaError_t sp_tc_shared_expert(SpTcPlan *p, const SpDims &d, const SpLayerDev &L, int M, const float *nx, float *dn,
                                int *status, cudaStream_t st, int *nl, int phase = 0);
/* routed experts on R rows sorted by expert (expert e owns rows [offsets[e], offsets[e+1]), device
 * array of NE+1 ints): out[rowmap ? rowmap[r] : r][E] = Wdn[e] . geglu(Wgu[e] . rows[r]).
 * gather != NULL: row r is src[gather[r]] instead of src[r]. R <= max_rows. */
cudaError_t sp_tc_routed(SpTcPlan *p, const SpDims &d, const SpLayerDev &L, int R, const float *src, const int *gather,
                         const int *offsets, const int *rowmap, float *out, int *status, cudaStream_t st, int *nl);
/* single-GPU helper: per-expert counts -> offsets[NE+1]; pair (t, slot) with expert e and list
 * position pos lands on sorted row offsets[e] + pos: gather[row] = t, rowmap[row] = pair.
 * Returns device pointers owned by the plan. */
cudaError_t sp_tc_sort_pairs(SpTcPlan *p, const SpDims &d, int M, const int *sel_asc, const int *count, const int *pairpos,
                             const int **offsets, const int **gather, const int **rowmap, cudaStream_t st, int *nl);
