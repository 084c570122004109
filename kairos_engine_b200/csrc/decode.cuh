/* decode.cuh — launch interface of the persistent M=1 decode kernel (decode.cu). */
#pragma once
#include "common.cuh"

struct SpDecodeArgs {
    SpLayerDev layer0;             /* device pointers of layer 0 (router_bias always set: see bias_mask) */
    size_t layer_stride;           /* bytes between consecutive layers' slabs */
    unsigned long long bias_mask;  /* bit li: layer layer_first + li has a router bias (n_layers <= 64 per launch) */
    int layer_first, n_layers;
    SpDims d;
    const float *x_in;             /* [E] */
    float *y_out;                  /* [E] */
    int32_t *sel_out;              /* [n_layers][NU] descending-p ids, or NULL */
    float *wts_out;                /* [n_layers][NU], or NULL */
    /* exchange buffers in device memory: 8-byte {f32 value, u32 epoch} words, written by the
     * CTA that owns the element and polled by every CTA; zero-initialised, epochs start at 1 */
    unsigned long long *x_logits;  /* [NE] */
    unsigned long long *x_hd;      /* [FFS]      shared-expert GeGLU output */
    unsigned long long *x_dn;      /* [E]        shared-expert down output */
    unsigned long long *x_h;       /* [NU][FFE]  routed GeGLU outputs, ascending-id slots */
    unsigned long long *x_acc;     /* [E]        combined routed output */
    int *status;                   /* SP_KERR_* */
    unsigned epoch_base;           /* layer li of this launch publishes epoch_base + li + 1 */
    int n_slots;                   /* ring slots that fit the dynamic shared memory */
};

/* ring slots and total dynamic shared memory for these dims under `smem_limit`; 0 if it cannot fit */
int sp_decode_slots(const SpDims &d, int grid, size_t smem_limit, size_t *smem_bytes);
int sp_decode_threads();
cudaError_t sp_decode_prepare(const SpDims &d, size_t smem, int *max_grid);
cudaError_t sp_decode_launch(const SpDecodeArgs &args, int grid, size_t smem, cudaStream_t st);

/* ---- the three-kernels-per-layer decode path (decode_graph.cu) ---- */
struct SpGraphScratch {
    float *logits, *hd, *dn, *h, *acc;          /* [NE] [FFS] [E] [NU*FFE] [E] */
    signed char *in_q; float *in_s; int *in_c;  /* the routed experts' quantised input, [E] / [E/16] */
    int *sel_asc; float *cw;                    /* [NU] */
    int *status;
    float *xbuf[2];                             /* residual between layers, ping-pong */
    const float *prev_post_ffw1, *prev_post_ffw2, *prev_post_ffw;   /* set per launch */
};
size_t sp_graph_scratch_bytes(const SpDims &d);
cudaError_t sp_graph_decode_enqueue(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl, const float *x_in, float *y_out,
                                    int32_t *sel, float *wts, const SpGraphScratch &sc, int sms, cudaStream_t st, bool pdl, int *nlaunch);
