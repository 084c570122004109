/* decode.cuh — launch interface of the persistent M=1 decode kernel (decode.cu). */
#pragma once
#include "common.cuh"

struct SpDecodeArgs {
    const SpLayerDev *layers;      /* device array of all layers */
    int layer_first, n_layers;
    SpDims d;
    const float *x_in;             /* [E] */
    float *y_out;                  /* [E] */
    int32_t *sel_out;              /* [n_layers][NU] descending-p ids, or NULL */
    float *wts_out;                /* [n_layers][NU], or NULL */
    /* scratch in device memory, written by some CTAs and read by others */
    float *logits;                 /* [NE] */
    float *hd;                     /* [FFS]      shared-expert GeGLU output */
    float *dn;                     /* [E]        shared-expert down output */
    float *h;                      /* [NU][FFE]  routed GeGLU outputs, ascending-id slots */
    float *acc;                    /* [E]        combined routed output */
    unsigned *bar;                 /* monotonically increasing arrival counter */
    int *status;                   /* SP_KERR_* */
    unsigned bar_base;             /* counter value when this launch starts */
};

size_t sp_decode_smem_bytes(const SpDims &d, int grid);
int sp_decode_threads();
int sp_decode_barriers_per_layer();
cudaError_t sp_decode_prepare(size_t smem, int *max_grid);
cudaError_t sp_decode_launch(const SpDecodeArgs &args, int grid, size_t smem, cudaStream_t st);
