/* batched.cuh — launch interface of the M > 1 paths (batched.cu): the per-token decode
 * arithmetic for small batches and the dequant-GEMM arithmetic for prefill. */
#pragma once
#include "common.cuh"

#define SP_BATCHED_MAX_SLICES 4

struct SpBatchedScratch {
    void *base;            /* one allocation carved into the buffers the kernels use */
    size_t bytes;
    int max_tokens;
    int max_rows;          /* rows the expert stage accepts (>= max_tokens * NU) */
    struct SpTcPlan *tc;   /* tensor-core prefill plan, NULL when the geometry or the switch rules it out */
};

cudaError_t sp_batched_alloc(const SpDims &d, int max_tokens, int max_rows, SpBatchedScratch *s, size_t *bytes);
void sp_batched_free(SpBatchedScratch *s);
/* Runs layers [lf, lf+nl) on M tokens; enqueues only. *nlaunch = kernels launched.
 * layers_host: HOST array of the layers' device views (they ride as kernel parameters). */
cudaError_t sp_batched_forward(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl, int flavour, int M,
                               const float *x, float *y, int32_t *sel, float *wts,
                               SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch);

/* The same layer cut into the three stages an expert-parallel run needs (one layer at a time;
 * the shared-expert result and the combine weights stay in the scratch between route and finish).
 *   route   : sel_asc[M*NU] (expert ids per token, ascending), cw[M*NU] (combine weights in that
 *             order), rows[M*NU][E] (each pair's input row, sorted by expert), counts[NE] (pairs per
 *             expert), pair_index[M*NU] (where pair t*NU+k sits in rows)
 *   experts : R rows; sorted position p (expert e owns positions [offsets[e], offsets[e+1])) is row
 *             row_index[p] of rows_in and of rows_out (NULL = the rows are already sorted); R <= max_rows
 *   finish  : output of token t's k-th expert (ascending id) = pair_rows[pair_index[t*NU+k]] (NULL = t*NU+k)
 * t0 / slice: the tokens of one layer may be handled as up to SP_BATCHED_MAX_SLICES independent slices (slice i =
 * M tokens starting at token t0 of the handle's max_tokens) that are between route and finish at the same time;
 * route, shared and finish of a slice must name the same (t0, slice). The experts stage is per call. */
cudaError_t sp_batched_ep_route(const SpDims &d, const SpLayerDev &L, int flavour, int M, const float *x, int32_t *sel_asc, float *cw,
                                float *rows, int32_t *counts, int32_t *pair_index, int32_t *sel, float *wts, int defer_shared, int n_ranks, int capacity,
                                SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch, int t0 = 0, int slice = 0);
/* receive side of the padded exchange (route called with a capacity): offsets[NE+1] and row_index[n_ranks*capacity] */
cudaError_t sp_batched_ep_recv_layout(const SpDims &d, const int32_t *counts_all, int n_ranks, int rank, int capacity, int32_t *offsets, int32_t *row_index,
                                      cudaStream_t st, int *nlaunch);
/* the shared expert of the tokens the last route call prepared, when that call deferred it */
/* phase: 0 = the whole shared expert, 1 = gate/up + GeGLU only, 2 = the down rows only (after a phase-1 call for the same tokens) */
cudaError_t sp_batched_ep_shared(const SpDims &d, const SpLayerDev &L, int flavour, int M, SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch, int t0 = 0, int slice = 0, int phase = 0);
cudaError_t sp_batched_ep_experts(const SpDims &d, const SpLayerDev &L, int flavour, int R, const float *rows_in, const int32_t *row_index, const int32_t *offsets,
                                  float *rows_out, SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch,
                                  const int32_t *in_index = nullptr, int n_in = 0);   /* in_index: sorted position -> input row when pairs share input rows */
/* token dispatch (each token's input row travels once per destination rank): sender side after a route call made with
 * rows == NULL, and the receiver's input index after the receive layout */
cudaError_t sp_batched_ep_tokens(const SpDims &d, int M, int n_ranks, int capacity, int cap_tokens, const int32_t *sel_asc, const int32_t *pair_index,
                                 float *tokrows, int32_t *tokidx, int32_t *slot, SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch, int t0 = 0, int slice = 0);
cudaError_t sp_batched_ep_in_index(const int32_t *row_index, const int32_t *tokidx_recv, int n_ranks, int capacity, int cap_tokens, int32_t *in_index,
                                   cudaStream_t st, int *nlaunch);
cudaError_t sp_batched_ep_finish(const SpDims &d, const SpLayerDev &L, int M, const float *x, const float *pair_rows, const int32_t *pair_index, float *y,
                                 SpBatchedScratch *s, cudaStream_t st, int *nlaunch, int t0 = 0, int slice = 0);
