/* handle.cuh — the library's handle, shared by the translation units that implement its entry points. */
#pragma once
#include "common.cuh"
#include "decode.cuh"
#include "batched.cuh"
#include "../../include/sp_engine/moe_backend.h"
#include <vector>

struct LayerOffsets {           /* byte offsets into the arena */
    size_t router_w, router_scale, router_bias, ffn_norm, post_ffw1, pre_ffw2, post_ffw2, post_ffw, dexps_scale;
    size_t gu_codes, gu_bs, dn_codes, dn_bs, sg_codes, sg_bs, su_codes, su_bs, sd_codes, sd_bs;
    size_t end;
};

struct sp_moe {
    sp_moe_config cfg;
    SpDims d;
    int device;
    unsigned char *arena;       /* all layers, contiguous */
    size_t arena_bytes, layer_bytes;
    LayerOffsets off;           /* offsets inside one layer's slab */
    SpLayerDev *layers_dev;     /* device array [n_layers] */
    std::vector<SpLayerDev> layers_host;
    std::vector<unsigned char> has_bias, uploaded;
    int *status;
    int *status_host;           /* page-locked copy target: one synchronisation reads the error word */
    /* host-pointer entry staging */
    float *x_dev, *y_dev; int32_t *sel_dev; float *wts_dev;
    SpBatchedScratch bs;
    /* three-kernel decode path replayed from CUDA graphs, one per (first layer, layer count) */
    struct DecodeGraph { int lf, nl; bool routing; cudaGraphExec_t exec; int launches; };
    std::vector<DecodeGraph> graphs;
    /* small batches (1 < M <= 64) are launch-bound: the layer run is replayed from a graph per shape */
    struct BatchGraph { int lf, nl, M, flavour; bool routing; cudaGraphExec_t exec; int launches; };
    std::vector<BatchGraph> bgraphs;
    SpGraphScratch gs; unsigned char *gs_base; float *g_x, *g_y; int32_t *g_sel; float *g_wts;
    int decode_impl;            /* 0 = rows staged through shared memory (decode_staged.cu), 1 = rows read directly (decode_graph.cu) */
    unsigned staged_flags;
    int seq_tokens;                       /* decode batches up to this size run token by token through the single-token graph */
    long long *stamps;          /* device time stamps of the last layer of a decode run (SP_MOE_TIMING=1), else NULL */
    long long *stamps_host;
    uint64_t timing_runs; double timing_us[3][4], timing_layer_us;
    int sms;
    cudaStream_t stream;        /* stream of the host-pointer entry */
    cudaStream_t last_stream;
    size_t scratch_bytes;
    uint64_t launches;
    void *ep_state;             /* buffers, streams and events of sp_moe_ep_forward_dev (ep_nccl.cu), created on first use */
    void (*ep_state_free)(void *);
};

