/* decode.cuh — launch interfaces of the M=1 decode paths: three kernels per layer replayed from a
 * CUDA graph, with the weight rows staged through shared memory by the copy engine
 * (decode_staged.cu, the default) or read by the warps directly (decode_graph.cu, any geometry). */
#pragma once
#include "common.cuh"

struct SpGraphScratch {
    float *logits, *hd, *dn, *h, *acc;          /* [NE] [FFS] [E] [NU*FFE] [E] */
    signed char *in_q; float *in_s; int *in_c;  /* the routed experts' quantised input, [E] / [E/16] */
    int *sel_asc; float *cw;                    /* [NU] */
    int *status;
    float *xbuf[2];                             /* residual between layers, ping-pong */
    const float *prev_post_ffw1, *prev_post_ffw2, *prev_post_ffw;   /* set per launch */
    const int *slices;                          /* [grid][12]: each CTA's share of every phase (sp_staged_slices) */
};

/* ---- decode_graph.cu ---- */
/* per device, before the first enqueue: the kernels' dynamic shared-memory limits */
cudaError_t sp_graph_prepare();
cudaError_t sp_graph_decode_enqueue(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl, const float *x_in, float *y_out,
                                    int32_t *sel, float *wts, const SpGraphScratch &sc, int sms, cudaStream_t st, bool pdl, int *nlaunch);
/* recombine of the last layer of a run (one CTA): y = x_prev + post_ffw-normed branch sum */
cudaError_t sp_graph_launch_finish(const SpDims &d, const SpLayerDev &last, const SpGraphScratch &sc, const float *x_prev, float *y_out,
                                   cudaStream_t st, bool pdl);

/* ---- decode_staged.cu ---- */
enum {
    SP_STAGED_PREFETCH_SD = 1,      /* K1 asks L2 for the shared-expert down rows K2 will stage */
    SP_STAGED_PREFETCH_DN = 2,      /* K2 asks L2 for the routed down rows K3 will stage */
    SP_STAGED_PREFETCH_NEXT = 4,    /* K3 asks L2 for the next layer's router rows and shared gate/up rows */
    SP_STAGED_MMA_DN = 8,           /* K3 takes its row dots on mma.sync (16-row tiles) instead of dp4a chains; same bits */
    SP_STAGED_DEFAULT = 15
};
/* true when one CTA's slice of every phase fits `smem_optin` bytes of shared memory on a grid of `sms` CTAs */
bool sp_staged_fits(const SpDims &d, int sms, size_t smem_optin);
cudaError_t sp_staged_prepare(const SpDims &d, int sms);
void sp_staged_slices(const SpDims &d, int sms, int *out /* [sms][12] */);
/* stamps: NULL, or 48 device words that receive CTA 0's globaltimer readings in the last layer of the run:
 * [kernel 0..2][16]: 0 entry, 1 predecessor done, 2 activations ready, 3 first weight row may start, 4 rows done, 5.. finer marks */
cudaError_t sp_staged_decode_enqueue(const SpDims &d, const SpLayerDev *layers_host, int lf, int nl, const float *x_in, float *y_out,
                                     int32_t *sel, float *wts, const SpGraphScratch &sc, int sms, unsigned flags, long long *stamps,
                                     cudaStream_t st, bool pdl, int *nlaunch);
