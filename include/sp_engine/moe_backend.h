/* moe_backend.h — C ABI of libsp_moe_b200: the Gemma-4-26B-A4B mixture-of-experts feed-forward
 * layer (router softmax top-NU over NE experts, Q4B expert gate|up GeGLU + down, the always-on
 * shared expert, ordered weighted combine, sandwich norms) as hand-written sm_100a kernels with
 * every expert resident in device memory.
 *
 * It replaces, behind the same conventions, what the kairos-engine CUDA backend does inside
 * src/backends/cuda/cuda_forward.cu (cited below as CF):
 *   g4_ffn_block -> g4_ffn_apply(moe_on=1)           CF:9101-9114, 8314-9050   -> sp_moe_forward*
 *   build_weights (MoE part), moe_cache_init,
 *   moe_resident, moe_expert_view                     CF:2222-2372, 6773-6951, 6184-6193 -> sp_moe_open / sp_moe_upload_layer*
 *   gemma4_moe_ffn_q4b_cuda (standalone operator)     CF:13821-13977           -> same symbol, same signature
 *   sp_cuda_model_release                             CF:16103-16107           -> sp_moe_close
 *
 * Conventions (include/sp_engine/sp_status.h:18-59, CF:187-202): every entry returns int,
 * 0 = success, negative sp_status value on error, with the detail in the thread-local
 * sp_last_error(). Callers own every host buffer they pass; the handle owns all device memory.
 * A handle is not thread-safe (the reference's callers hold a per-session mutex,
 * tools/sp_daemon/src/cuda_kvdecode_dispatch.rs:400-401); different handles may be used
 * concurrently. There is no CPU fallback: without a CUDA device every call fails.
 */
#ifndef SP_ENGINE_MOE_BACKEND_H
#define SP_ENGINE_MOE_BACKEND_H
#include <stdint.h>
#include <stddef.h>
#ifdef __cplusplus
extern "C" {
#endif

/* status values used here; numerically those of include/sp_engine/sp_status.h */
#define SP_MOE_OK            0
#define SP_MOE_ENOMEM      (-1)
#define SP_MOE_EBADARG     (-3)
#define SP_MOE_EBADSTATE   (-4)
#define SP_MOE_EUNSUPPORTED (-5)
#define SP_MOE_ECUDA      (-40)
#define SP_MOE_EBACKEND_OOM (-43)

/* Thread-local error text of the last failing call on this thread (sp_status.h:57-59).
 * Exported WEAK so that, when linked into the daemon, the math core's definitions win. */
const char *sp_last_error(void);
void        sp_set_error(const char *msg);

typedef struct sp_moe sp_moe;          /* opaque; replaces the engine-owned g_w MoE fields, CF:1856-1903 */

/* Arithmetic the forward runs in (the AMMD switch, CF:8322-8324). */
#define SP_MOE_FLAVOUR_DECODE  0   /* int8 per-16 activation quant + exact integer dots (decode, M small) */
#define SP_MOE_FLAVOUR_PREFILL 1   /* exact Q4B dequant, floating-point GEMM (prefill, M large) */

typedef struct {
    int32_t E;           /* hidden size; multiple of 32, <= 4096 */
    int32_t NE;          /* routed experts per layer, <= 1024 */
    int32_t NU;          /* experts used per token, <= 8 (G4G_MAX, CF:5989) */
    int32_t FFE;         /* routed expert FFN width; multiple of 32 */
    int32_t FFS;         /* shared expert FFN width; multiple of 32 */
    int32_t n_layers;
    int32_t max_tokens;  /* largest M a forward call may pass */
    int32_t device;      /* CUDA device ordinal */
    float   eps;
    int32_t max_expert_rows; /* rows one sp_moe_ep_experts_dev call may pass; 0 = max_tokens * NU. An
                                expert-parallel rank can receive up to (tokens of the whole job) * NU */
    int32_t reserved[6]; /* zero */
} sp_moe_config;

/* One layer's weights in the reference's layouts (sp_model.h:50-53, CF:1448-1464, 6179-6193):
 * Q4B codes are row-major, in/2 bytes per row, byte k = weight 2k (low nibble) | weight 2k+1
 * (high nibble), 4-bit two's complement; block scales are f16 bit patterns [rows][in/32].
 * gate|up is ONE fused tensor of NE*2*FFE rows (expert e owns rows [e*2*FFE, (e+1)*2*FFE),
 * gate first, then up); down is NE*E rows of FFE columns. */
typedef struct {
    const float    *router_w;      /* [NE][E] f32, CF:2258-2268 */
    const float    *router_scale;  /* [E]   ffn_gate_inp.scale */
    const float    *router_bias;   /* [NE]  optional, may be NULL (added to the logits) */
    const float    *ffn_norm, *post_ffw1, *pre_ffw2, *post_ffw2, *post_ffw;   /* [E] */
    const float    *dexps_scale;   /* [NE]  ffn_down_exps.scale, CF:1873-1878 */
    const uint8_t  *gu_codes;  const uint16_t *gu_bs;
    const uint8_t  *dn_codes;  const uint16_t *dn_bs;
    const uint8_t  *sg_codes;  const uint16_t *sg_bs;   /* shared gate [FFS][E] */
    const uint8_t  *su_codes;  const uint16_t *su_bs;   /* shared up   [FFS][E] */
    const uint8_t  *sd_codes;  const uint16_t *sd_bs;   /* shared down [E][FFS] */
} sp_moe_layer_weights;

/* gemma4_kv_open's MoE share (CF:9807 -> build_weights CF:2222-2372 -> moe_cache_init
 * CF:6773-6879): allocates one resident arena for all n_layers * NE experts plus scratch. */
int  sp_moe_open(const sp_moe_config *cfg, sp_moe **out);
/* sp_cuda_model_release, CF:16103-16107. NULL-safe. */
int  sp_moe_close(sp_moe *h);
/* Copies one layer into the arena (moe_stage without the cache, CF:9065-9099). The pointers
 * are HOST memory in sp_moe_upload_layer and DEVICE memory in sp_moe_upload_layer_dev. */
int  sp_moe_upload_layer(sp_moe *h, int layer, const sp_moe_layer_weights *w);
int  sp_moe_upload_layer_dev(sp_moe *h, int layer, const sp_moe_layer_weights *w);
/* Fills every layer of the handle from a `.sp-model` file (include/sp_engine/sp_model.h:97-134): the MoE share of
 * build_weights (CF:2222-2372) + moe_cache_init (CF:6773-6879) in one call. The file is memory-mapped and each
 * tensor goes straight from the mapping into the arena. names: NULL for the defaults, or 18 printf templates (one
 * %d = the layer) in the order router_w, router_scale, ffn_norm, post_ffw1, pre_ffw2, post_ffw2, post_ffw,
 * dexps_scale, then codes and block scales of gate|up, down, shared gate, shared up, shared down (defaults:
 * "blk.%d.ffn_gate_inp.weight", ..., "blk.%d.ffn_down.weight.bscale"; a tensor "blk.%d.ffn_gate_inp.bias", when
 * present, becomes the router bias). Checked: magic, layout rules, header CRC-32, each tensor's bounds,
 * alignment, dtype, byte size and name hash; the per-tensor blake3 digest is not (no BLAKE3 in this library). */
int  sp_moe_load_sp_model(sp_moe *h, const char *path, const char *const *names);
/* Replaces only the router's per-expert logit bias of one layer (DEVICE pointer to NE floats, or NULL for
 * no bias); the other tensors stay as uploaded. The reference adds such a bias where the model file carries
 * one (`ffn_gate_inp.bias`, read with the router in build_weights, CF:2258-2268); load-imbalance experiments
 * use it to skew the routing without touching the experts. */
int  sp_moe_set_router_bias_dev(sp_moe *h, int layer, const float *bias_dev);
/* Bytes of device memory the handle holds (arena + scratch). */
size_t sp_moe_device_bytes(const sp_moe *h);

/* g4_ffn_apply (CF:8314-9050) over layers [layer_first, layer_first + n_layers): each layer's
 * output residual feeds the next. x, y: [M][E] f32; sel: [n_layers][M][NU] expert ids in
 * descending probability (moe_topk_host order, CF:6220-6240); wts: the matching renormalised
 * probabilities. sel / wts may be NULL. HOST pointers; copies in, runs, copies out, synchronises. */
int  sp_moe_forward(sp_moe *h, int layer_first, int n_layers, int flavour, int M,
                    const float *x, float *y, int32_t *sel, float *wts);
/* Same with DEVICE pointers on a caller stream (a cudaStream_t passed as void*); enqueues only.
 * A router row with a NaN (the reference's hard error, CF:8596-8620) is reported by the next
 * sp_moe_status call. */
int  sp_moe_forward_dev(sp_moe *h, int layer_first, int n_layers, int flavour, int M,
                        const float *x_dev, float *y_dev, int32_t *sel_dev, float *wts_dev,
                        void *stream);
/* Synchronises the handle's last stream and returns 0 or the error a kernel recorded. */
int  sp_moe_status(sp_moe *h);

/* One layer of g4_ffn_apply cut where (token, expert) pairs would change GPU, for expert-parallel
 * prefill (the reference is single-GPU: its expert-major loop, CF:8925-8965, visits every expert
 * on the one device; here each GPU owns a contiguous block of experts and the caller moves rows
 * between the stages with an all-to-all). DEVICE pointers, enqueue only, one layer in flight per
 * handle (the shared-expert branch and the combine weights wait in the handle between route and
 * finish).
 *   route   : x[M][E] -> sel_asc[M][NU] (each token's experts, ascending id), cw[M][NU] (combine
 *             weight = renormalised probability * down-scale, same order), rows[M*NU][E] (each
 *             pair's input row - x normalised with pre_ffw_norm_2 - sorted by expert, so by owner:
 *             the all-to-all send buffer), counts[NE] (pairs per expert), pair_index[M*NU] (the row
 *             of pair t*NU+k in that buffer, and so in what comes back); sel/wts as in
 *             sp_moe_forward (or NULL). defer_shared != 0 leaves the shared expert out: call
 *             sp_moe_ep_shared_dev (same layer, flavour, M) any time before finish - typically right
 *             after starting the dispatch exchange, so the two overlap. capacity > 0 (with n_ranks
 *             ranks owning NE / n_ranks experts each) pads the buffer: rows for rank r start at row
 *             r * capacity of rows[n_ranks * capacity][E], so the exchange needs no split sizes and
 *             no host read; a rank's block that does not fit is reported by sp_moe_status
 *   recv_layout (padded exchange only): counts_all[n_ranks][NE] (every rank's counts, gathered) ->
 *             offsets[NE+1] and row_index[n_ranks * capacity] for the experts stage, whose n_rows
 *             is then n_ranks * capacity
 *   experts : rows_in[n_rows][E] -> rows_out[n_rows][E] = down(geglu(gate|up(row))) with the weights of
 *             the row's expert. Sorted by expert, position p belongs to expert e when
 *             offsets[e] <= p < offsets[e+1] (offsets: NE+1 ints, device memory) and is row
 *             row_index[p] of rows_in / rows_out; row_index NULL = the rows are already sorted.
 *             n_rows <= max_expert_rows of the config
 *   finish  : token t's k-th expert output (sel_asc order) is row pair_index[t*NU+k] of pair_rows
 *             (pair_index NULL = row t*NU+k) -> y = the layer's output residual
 * A run through the three stages is bit-identical to sp_moe_forward_dev on the same tokens. */
int sp_moe_ep_route_dev(sp_moe *h, int layer, int flavour, int M, const float *x_dev,
                        int32_t *sel_asc_dev, float *cw_dev, float *rows_dev, int32_t *counts_dev,
                        int32_t *pair_index_dev, int32_t *sel_dev, float *wts_dev, int defer_shared,
                        int n_ranks, int capacity, void *stream);
int sp_moe_ep_recv_layout_dev(sp_moe *h, const int32_t *counts_all_dev, int n_ranks, int rank, int capacity,
                              int32_t *offsets_dev, int32_t *row_index_dev, void *stream);
int sp_moe_ep_shared_dev(sp_moe *h, int layer, int flavour, int M, void *stream);
int sp_moe_ep_experts_dev(sp_moe *h, int layer, int flavour, int n_rows, const float *rows_in_dev,
                          const int32_t *row_index_dev, const int32_t *offsets_dev, float *rows_out_dev,
                          void *stream);
int sp_moe_ep_finish_dev(sp_moe *h, int layer, int M, const float *x_dev, const float *pair_rows_dev,
                         const int32_t *pair_index_dev, float *y_dev, void *stream);

/* The whole expert-parallel loop in one call: layers [layer_first, layer_first + n_layers) over n_ranks GPUs (one
 * process each; this rank's tokens x_dev[M][E] in, y_dev[M][E] out, DEVICE pointers), the five stages above driven
 * from inside the library with NCCL doing the count gather and the two exchanges of every layer (ncclAllGather,
 * ncclSend / ncclRecv groups). nccl_comm: an ncclComm_t of the n_ranks processes, passed as void* - the caller's
 * own, or one made with the helpers below. NCCL is looked up at run time (libnccl.so.2), not linked.
 *   capacity_rows > 0 : padded exchange - room per destination rank for the whole call; no host read, the call
 *                       only enqueues (kernels on `stream`, NCCL on an internal stream, events between them) and
 *                       can be captured into a CUDA graph. slices (1..4): the tokens are handled as that many
 *                       independent slices, so one slice's exchanges run under another's expert GEMMs. A block
 *                       that does not fit is reported by sp_moe_status; rerun with capacity_rows = 0.
 *   capacity_rows == 0: exact exchange - split sizes read on the host once per layer (the call synchronises).
 * Needs max_expert_rows of the config >= n_ranks * capacity (padded) or the rows this rank can receive (exact).
 * The first call allocates the exchange buffers (make it before any capture). Bit-identical to sp_moe_forward_dev.
 * Every rank must have opened its handle with the same configuration (the buffers are laid out alike everywhere).
 * In a world of up to four ranks the rows are moved by device-to-device copies into the peers' buffers, which the
 * first call (outside a capture) maps through CUDA IPC - all ranks of one node - with NCCL left to carry the counts
 * and a one-int all-reduce; with more ranks, or where the mapping fails on any rank, by NCCL send/recv pairs
 * (SP_MOE_EP_EXCHANGE=copy|nccl in the environment overrides the choice). In the padded exchange a token's input
 * row travels once per destination rank, with a slot per pair (SP_MOE_EP_DISPATCH=rows: one row per pair). */
int sp_moe_ep_forward_dev(sp_moe *h, void *nccl_comm, int n_ranks, int rank, int layer_first, int n_layers, int flavour,
                          int M, const float *x_dev, float *y_dev, int capacity_rows, int slices, void *stream);
/* rows this rank's experts processed in the last layer of the last sp_moe_ep_forward_dev call */
long long sp_moe_ep_last_rows(const sp_moe *h);
/* Stage times of the LAST layer of the most recent sp_moe_ep_forward_dev call, in milliseconds, from CUDA events:
 * ms6[0] route (norms, router, top-NU, send buffer), [1] count gather + dispatch exchange, [2] end of the dispatch
 * to end of the experts stage (the shared expert runs under the dispatch), [3] combine exchange, [4] finish,
 * [5] the whole layer. Needs SP_MOE_TIMING=1 in the environment when the handle was opened, one token slice and
 * a call made outside a stream capture; otherwise SP_MOE_EBADSTATE. Synchronises. */
int sp_moe_ep_timing(sp_moe *h, float *ms6);
/* Communicator helpers for callers without NCCL headers: 128 opaque bytes from one rank (ncclGetUniqueId), handed to
 * every rank by whatever channel the job has, then one communicator per rank on its current CUDA device. */
int sp_moe_ep_unique_id(void *id128);
int sp_moe_ep_comm_create(const void *id128, int n_ranks, int rank, void **comm_out);
int sp_moe_ep_comm_destroy(void *comm);

/* The reference's standalone single-token operator, verbatim signature (CF:13821-13825).
 * All pointers are HOST memory; allocates, uploads the whole expert set, runs, frees.
 * Its semantics differ from the layer above (one weightless norm, no shared expert, no
 * clamp, descending-probability accumulation; CF:13821-13977). Returns 0, or 1 on error. */
int gemma4_moe_ffn_q4b_cuda(int E, int NE, int NU, int FF, float eps,
                            const float *gate_inp, const float *gate_inp_scale,
                            const unsigned char *gu_codes, const unsigned short *gu_bscale,
                            const unsigned char *dn_codes, const unsigned short *dn_bscale,
                            const float *hidden, float *out, int *sel_out);

/* The reference's MoE plugin hook for SwiGLU models with separate gate / up / down expert tensors
 * (sp_q36gpu_upload_experts + sp_q36gpu_moe, CF:16203-16289; the hook type it is registered under
 * is int (*)(void *ctx, const char *gate_name, const int *idx, const float *wt, int NU,
 * const float *x, int E, int FF, float *y), CF:16444-16454). Experts are uploaded once per layer
 * under a tag (HOST pointers; Q4B codes [NE][FF][E/2] + f16 scales for gate and up, [NE][E][FF/2]
 * + scales for down). sp_moe_ext_moe takes the expert ids and weights the caller's router chose
 * and HOST x / y: y = sum_k wt[k] * down(silu(gate x) * (up x)) in the caller's k order, in the
 * decode arithmetic (gemv_w_packed). Returns 0 = handled, nonzero = not mine (unknown tag, other
 * shape), which is the hook's contract; upload/open return 0 or 1 like the reference's. */
typedef struct sp_moe_ext sp_moe_ext;
int sp_moe_ext_open(int device, sp_moe_ext **out);
int sp_moe_ext_close(sp_moe_ext *h);
int sp_moe_ext_upload_experts(sp_moe_ext *h, const char *tag,
                              const uint8_t *gate_codes, const uint16_t *gate_bs,
                              const uint8_t *up_codes, const uint16_t *up_bs,
                              const uint8_t *down_codes, const uint16_t *down_bs, int NE, int FF, int E);
int sp_moe_ext_moe(void *h, const char *tag, const int *idx, const float *wt, int NU,
                   const float *x, int E, int FF, float *y);

/* The quantised GEMM of src/backends/cuda/ptx_mma.cuh (sp_frob_matmul_q8_mma_tile, ptx_mma_tile_int8.cuh:92-110,
 * and the int4 kernels, ptx_mma.cuh:268-353) on DEVICE memory:
 *   C[m][n] (f16 bits) = f16( float(sum_k A[m][k] * B[n][k]) * scale_a[m] * scale_b[n] ),
 * A [M][K] and B [N][K] int8 (q8) or packed signed int4, two per byte, low nibble first (q4);
 * int32 accumulate; K a multiple of 16, operand pointers 16-byte aligned. Enqueues on `stream`;
 * the q4 entry unpacks into scratch it allocates, so it also synchronises the stream and frees. */
int sp_frob_matmul_q8_dev(const int8_t *A_dev, const int8_t *B_dev, const float *scale_a_dev,
                          const float *scale_b_dev, uint16_t *C_f16_dev, int M, int K, int N, void *stream);
int sp_frob_matmul_q4_dev(const uint8_t *A_q4_dev, const uint8_t *B_q4_dev, const float *scale_a_dev,
                          const float *scale_b_dev, uint16_t *C_f16_dev, int M, int K, int N, void *stream);

/* Q4B block quantiser on DEVICE memory: the recipe of sp_model.h:50-53 / CF:1680-1687 (per-32
 * block, f16 scale stored first, codes derived against the stored scale, codes in [-7,7]).
 * The reference's own quantiser is in a submodule that is not part of its tree; this follows
 * the documented recipe only. w: [rows][cols] f32; codes: [rows][cols/2]; bs: [rows][cols/32]. */
int sp_moe_q4b_quantize_dev(const float *w_dev, int64_t rows, int cols,
                            uint8_t *codes_dev, uint16_t *bs_dev, void *stream);
/* k_dequant_arena_q4b, CF:1452-1464. */
int sp_moe_q4b_dequantize_dev(const uint8_t *codes_dev, const uint16_t *bs_dev, int64_t rows, int cols,
                              float *w_dev, void *stream);

/* gemv_w_packed for OK_Q4B (CF:13566-13599): y[rows] = W . x in the decode arithmetic (int8 per-16
 * activation quant, CF:1564-1585, then the Q4B x int8 GEMV, CF:1688-1713). DEVICE pointers; W is
 * [rows][in/2] codes + f16 [rows][in/32] scales; in a multiple of 32, at most 4096. Allocates its int8
 * scratch for the call, synchronises the stream and frees it. */
int sp_moe_gemv_q4b_dev(const uint8_t *codes_dev, const uint16_t *bs_dev, int in, int rows,
                        const float *x_dev, float *y_dev, void *stream);

/* sp_moe_gemv_q4b_dev without any allocation. NO COUNTERPART IN THE REFERENCE (there the caller of
 * gemv_w_packed owns the int8 scratch). For callers that must not allocate device memory when they
 * call - a serving loop that has committed the whole card to pre-sized arenas, where cudaMalloc can
 * fail and where cudaMalloc / cudaFree stall every stream of the device, or a component that only
 * ever works in buffers its host hands it. The int8 scratch is a fixed array inside the library
 * (6 KB per device that loads it, held until exit), so `in` is limited to 4096; larger values are
 * refused with SP_MOE_EBADARG. The call enqueues on `stream` and returns; it calls no cudaMalloc,
 * cudaFree or other allocating routine. The FIRST call on each device also looks up the array's
 * device address (cudaGetSymbolAddress): make that first call before opening any stream capture.
 * Every call shares the one array and leaves its last contents there: two calls whose kernels can
 * overlap on the GPU (different streams) race on it - keep them on one stream or order them. */
int sp_moe_gemv_q4b_static_dev(const uint8_t *codes_dev, const uint16_t *bs_dev, int in, int rows,
                               const float *x_dev, float *y_dev, void *stream);

/* k_gelu_mul (CF:1364-1373): out[i] = gelu_tanh(g[i]) * up[i] on DEVICE memory, in the library's
 * bit-reproducible arithmetic (the tanh is a fixed sequence of correctly-rounded operations). */
int sp_moe_gelu_mul_dev(const float *g_dev, const float *up_dev, int64_t n, float *out_dev, void *stream);

/* Counters for callers that report them (the reference prints similar lines under SP_MOE_TIMING,
 * CF:9020-9044): kernels launched by this handle since open. */
uint64_t sp_moe_kernel_launches(const sp_moe *h);

/* Phase timing of the single-token decode path: the counterpart of the reference's `[g4-moe] TIMING`
 * accounting (CF:7186-7201, 9020-9044; switched on the same way, SP_MOE_TIMING=1 in the environment
 * when the handle is opened - without it no clock is read and this call returns SP_MOE_EBADSTATE).
 * The reference splits host wall time into sync / route / expert loop / stage; none of those exist
 * here (no host round trip, nothing staged), so the phases are this path's own: for each of the
 * three kernels of a layer, microseconds on the device clock between entry, the predecessor's
 * results being visible, the end of the per-layer prologue (norms / top-NU / quantisation) and the
 * last weight row. Values are of the LAST layer of the most recent M=1 decode call, read from
 * CTA 0; the call synchronises the handle's last stream. With SP_MOE_TIMING=1 the host entry
 * sp_moe_forward also prints one `[g4-moe] TIMING` line to stderr every 300 decoded layers. */
typedef struct {
    float wait_us[3];      /* kernel entry -> predecessor's results visible (0: router + shared gate/up, 1: top-NU + shared down + routed gate|up, 2: routed down + combine) */
    float prologue_us[3];  /* -> activations normalised / selected / quantised in shared memory */
    float rows_us[3];      /* -> last weight row of the CTA's slice done */
    float layer_us;        /* first kernel's entry -> last kernel's last row */
    float raw_us[3][16];   /* every stamp a kernel took, microseconds since the first kernel's entry (0 = not taken) */
} sp_moe_timing;
int sp_moe_decode_timing(sp_moe *h, sp_moe_timing *out);

/* Failure-path probe: runs one CTA that waits on a copy that is never started, with a limit of
 * `polls` polls (1..1048576). The wait gives up, the kernel returns normally and records the same
 * error word a real timed-out wait in the decode kernels records, so the next sp_moe_status call
 * returns SP_MOE_ECUDA with the timeout text, and the handle stays usable. Nothing traps or hangs.
 * (The reference's model for this is the bounded handshake of tools/moe_cpu_bench/handshake_test.cu:14-41.) */
int sp_moe_debug_wait_timeout(sp_moe *h, int polls, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* SP_ENGINE_MOE_BACKEND_H */
