/* batched.cu — placeholder until the M > 1 kernels land: reports "not supported". */
#include "batched.cuh"
cudaError_t sp_batched_alloc(const SpDims &, int max_tokens, SpBatchedScratch *s, size_t *bytes) { s->base = nullptr; s->bytes = 0; s->max_tokens = max_tokens; *bytes = 0; return cudaSuccess; }
void sp_batched_free(SpBatchedScratch *s) { if (s && s->base) cudaFree(s->base); if (s) s->base = nullptr; }
cudaError_t sp_batched_forward(const SpDims &, const SpLayerDev *, int, int, int, int, const float *, float *, int32_t *, float *,
                               SpBatchedScratch *, int *, cudaStream_t, int *nlaunch) { *nlaunch = 0; return cudaErrorNotSupported; }
