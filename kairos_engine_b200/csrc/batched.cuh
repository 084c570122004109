/* batched.cuh — launch interface of the M > 1 paths (batched.cu): the per-token decode
 * arithmetic for small batches and the dequant-GEMM arithmetic for prefill. */
#pragma once
#include "common.cuh"

struct SpBatchedScratch {
    void *base;            /* one allocation carved into the buffers the kernels use */
    size_t bytes;
    int max_tokens;
};

cudaError_t sp_batched_alloc(const SpDims &d, int max_tokens, SpBatchedScratch *s, size_t *bytes);
void sp_batched_free(SpBatchedScratch *s);
/* Runs layers [lf, lf+nl) on M tokens; enqueues only. *nlaunch = kernels launched.
 * layers_host: HOST array of the layers' device views (they ride as kernel parameters). */
cudaError_t sp_batched_forward(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl, int flavour, int M,
                               const float *x, float *y, int32_t *sel, float *wts,
                               SpBatchedScratch *s, int *status, cudaStream_t st, int *nlaunch);
