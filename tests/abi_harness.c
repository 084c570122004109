/* abi_harness.c — calls every entry point of include/sp_engine/moe_backend.h from plain C, the way the
 * daemon's C glue (tools/sp_daemon/c_backend_cuda/sp_daemon_cuda_glue.c:247-499) and its Rust
 * `unsafe extern "C"` block would: structs are laid out by the C compiler from the header, device
 * buffers come from the CUDA runtime, nothing of Python is in the process. A ctypes test cannot see a
 * struct-layout or argument-list drift between header and library; this does.
 *
 * Test infrastructure: built and run by tests/test_abi_harness_gpu.py
 *   gcc -O1 -Iinclude -I<cuda>/include tests/abi_harness.c -L<lib dir> -lsp_moe_b200 -L<cuda>/lib64 -lcudart -lm
 * Checks are self-consistency checks (host entry == device entry == staged expert-parallel run, bit for
 * bit; quantise -> dequantise round trip; documented refusals); parity with the CPU checker is the
 * Python tests' job. Prints one line per check and exits 0 only if all passed.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <cuda_runtime_api.h>
#include "sp_engine/moe_backend.h"

static int g_fail = 0, g_checks = 0;
#define CHECK(cond, ...) do { g_checks++; if (!(cond)) { g_fail++; printf("FAIL %s:%d: ", __FILE__, __LINE__); printf(__VA_ARGS__); printf(" [last error: %s]\n", sp_last_error()); } } while (0)
#define CUDA_OK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { printf("FAIL cuda %s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); return 2; } } while (0)

static uint32_t g_seed = 12345u;
static float frand(void) { g_seed = g_seed * 1664525u + 1013904223u; return (float)(g_seed >> 8) / 16777216.0f; }   /* [0,1) */
static float gauss(void) { float s = 0.0f; for (int i = 0; i < 12; i++) s += frand(); return s - 6.0f; }

enum { E = 128, NE = 8, NU = 2, FFE = 32, FFS = 64, NL = 2, MT = 8 };

static void *dev_copy(const void *host, size_t bytes) {
    void *p = NULL;
    if (cudaMalloc(&p, bytes) != cudaSuccess) return NULL;
    if (host && cudaMemcpy(p, host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return NULL;
    return p;
}

/* quantise a random [rows][cols] matrix on the device through the library's own quantiser */
static int make_q4b(int64_t rows, int cols, float std, uint8_t **codes, uint16_t **bs, uint8_t **codes_dev, uint16_t **bs_dev) {
    const size_t n = (size_t)rows * cols;
    float *w = (float *)malloc(n * 4);
    for (size_t i = 0; i < n; i++) w[i] = gauss() * std;
    float *w_dev = (float *)dev_copy(w, n * 4);
    *codes_dev = (uint8_t *)dev_copy(NULL, n / 2); *bs_dev = (uint16_t *)dev_copy(NULL, n / 32 * 2);
    if (!w_dev || !*codes_dev || !*bs_dev) return 1;
    if (sp_moe_q4b_quantize_dev(w_dev, rows, cols, *codes_dev, *bs_dev, NULL)) return 1;
    *codes = (uint8_t *)malloc(n / 2); *bs = (uint16_t *)malloc(n / 32 * 2);
    if (cudaMemcpy(*codes, *codes_dev, n / 2, cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
    if (cudaMemcpy(*bs, *bs_dev, n / 32 * 2, cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
    /* round trip: dequantise and compare with the input within half a quantisation step of the block */
    float *back_dev = (float *)dev_copy(NULL, n * 4), *back = (float *)malloc(n * 4);
    if (!back_dev || sp_moe_q4b_dequantize_dev(*codes_dev, *bs_dev, rows, cols, back_dev, NULL)) return 1;
    if (cudaMemcpy(back, back_dev, n * 4, cudaMemcpyDeviceToHost) != cudaSuccess) return 1;
    double worst = 0.0;
    for (size_t i = 0; i < n; i++) { const double d = fabs((double)back[i] - w[i]); if (d > worst) worst = d; }
    CHECK(worst <= 6.0 * std / 7.0, "Q4B round trip error %.4g", worst);
    cudaFree(w_dev); cudaFree(back_dev); free(w); free(back);
    return 0;
}

int main(void) {
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0) { printf("no CUDA device\n"); return 3; }
    CUDA_OK(cudaSetDevice(0));

    /* ---- error text */
    sp_set_error("harness");
    CHECK(strcmp(sp_last_error(), "harness") == 0, "sp_set_error / sp_last_error");

    /* ---- open: refusals first, then the real handle */
    sp_moe *h = NULL;
    sp_moe_config bad; memset(&bad, 0, sizeof bad);
    bad.E = 100; bad.NE = NE; bad.NU = NU; bad.FFE = FFE; bad.FFS = FFS; bad.n_layers = 1; bad.max_tokens = 1; bad.eps = 1e-6f;
    CHECK(sp_moe_open(&bad, &h) == SP_MOE_EBADARG && h == NULL, "open must refuse E %% 32 != 0");
    CHECK(sp_moe_open(NULL, &h) == SP_MOE_EBADARG, "open must refuse NULL");
    sp_moe_config cfg; memset(&cfg, 0, sizeof cfg);
    cfg.E = E; cfg.NE = NE; cfg.NU = NU; cfg.FFE = FFE; cfg.FFS = FFS; cfg.n_layers = NL; cfg.max_tokens = MT; cfg.device = 0; cfg.eps = 1e-6f;
    CHECK(sp_moe_open(&cfg, &h) == SP_MOE_OK && h != NULL, "sp_moe_open");
    if (!h) return 1;
    CHECK(sp_moe_device_bytes(h) > 0, "sp_moe_device_bytes");

    /* ---- weights: layer 0 through the host entry, layer 1 through the device entry */
    float *x = (float *)malloc(MT * E * 4), *y = (float *)malloc(MT * E * 4), *y2 = (float *)malloc(MT * E * 4);
    for (int i = 0; i < MT * E; i++) x[i] = gauss();
    CHECK(sp_moe_forward(h, 0, NL, SP_MOE_FLAVOUR_DECODE, 1, x, y, NULL, NULL) == SP_MOE_EBADSTATE, "forward before upload must be refused");
    for (int L = 0; L < NL; L++) {
        float router[NE * E], vecs[6][E], dsc[NE], bias[NE];
        for (int i = 0; i < NE * E; i++) router[i] = gauss() * 0.02f;
        for (int k = 0; k < 6; k++) for (int i = 0; i < E; i++) vecs[k][i] = 0.5f + frand();
        for (int i = 0; i < NE; i++) { dsc[i] = 0.5f + frand(); bias[i] = 0.1f * gauss(); }
        uint8_t *c[5], *cd[5]; uint16_t *s[5], *sd[5];
        const int64_t rows[5] = {(int64_t)NE * 2 * FFE, (int64_t)NE * E, FFS, FFS, E};
        const int cols[5] = {E, FFE, E, E, FFS};
        for (int k = 0; k < 5; k++) if (make_q4b(rows[k], cols[k], 0.02f, &c[k], &s[k], &cd[k], &sd[k])) { printf("FAIL: building Q4B tensor %d: %s\n", k, sp_last_error()); return 1; }
        sp_moe_layer_weights w; memset(&w, 0, sizeof w);
        if (L == 0) {
            w.router_w = router; w.router_scale = vecs[0]; w.router_bias = bias; w.ffn_norm = vecs[1]; w.post_ffw1 = vecs[2]; w.pre_ffw2 = vecs[3];
            w.post_ffw2 = vecs[4]; w.post_ffw = vecs[5]; w.dexps_scale = dsc;
            w.gu_codes = c[0]; w.gu_bs = s[0]; w.dn_codes = c[1]; w.dn_bs = s[1]; w.sg_codes = c[2]; w.sg_bs = s[2];
            w.su_codes = c[3]; w.su_bs = s[3]; w.sd_codes = c[4]; w.sd_bs = s[4];
            CHECK(sp_moe_upload_layer(h, L, &w) == SP_MOE_OK, "sp_moe_upload_layer");
            w.gu_codes = NULL;
            CHECK(sp_moe_upload_layer(h, L, &w) == SP_MOE_EBADARG, "upload must refuse a NULL tensor");
        } else {
            w.router_w = (const float *)dev_copy(router, sizeof router); w.router_scale = (const float *)dev_copy(vecs[0], E * 4);
            w.router_bias = NULL; w.ffn_norm = (const float *)dev_copy(vecs[1], E * 4); w.post_ffw1 = (const float *)dev_copy(vecs[2], E * 4);
            w.pre_ffw2 = (const float *)dev_copy(vecs[3], E * 4); w.post_ffw2 = (const float *)dev_copy(vecs[4], E * 4);
            w.post_ffw = (const float *)dev_copy(vecs[5], E * 4); w.dexps_scale = (const float *)dev_copy(dsc, NE * 4);
            w.gu_codes = cd[0]; w.gu_bs = sd[0]; w.dn_codes = cd[1]; w.dn_bs = sd[1]; w.sg_codes = cd[2]; w.sg_bs = sd[2];
            w.su_codes = cd[3]; w.su_bs = sd[3]; w.sd_codes = cd[4]; w.sd_bs = sd[4];
            CHECK(sp_moe_upload_layer_dev(h, L, &w) == SP_MOE_OK, "sp_moe_upload_layer_dev");
        }
    }

    /* ---- forward: host entry, both flavours, M = 1 and M = MT; device entry must agree bit for bit */
    int32_t sel[NL * MT * NU]; float wts[NL * MT * NU];
    float *x_dev = (float *)dev_copy(x, MT * E * 4), *y_dev = (float *)dev_copy(NULL, MT * E * 4);
    int32_t *sel_dev = (int32_t *)dev_copy(NULL, sizeof sel); float *wts_dev = (float *)dev_copy(NULL, sizeof wts);
    cudaStream_t st; CUDA_OK(cudaStreamCreate(&st));
    for (int flavour = 0; flavour < 2; flavour++) for (int M = 1; M <= MT; M += MT - 1) {
        memset(sel, 0xff, sizeof sel);
        CHECK(sp_moe_forward(h, 0, NL, flavour, M, x, y, sel, wts) == SP_MOE_OK, "sp_moe_forward flavour %d M %d", flavour, M);
        int ok = 1;
        for (int i = 0; i < M * E; i++) if (!isfinite(y[i])) ok = 0;
        for (int i = 0; i < NL * M * NU; i++) if (sel[i] < 0 || sel[i] >= NE || !(wts[i] >= 0.0f && wts[i] <= 1.0f)) ok = 0;
        for (int i = 0; i < NL * M; i++) { float s_ = 0.0f; for (int k = 0; k < NU; k++) s_ += wts[i * NU + k]; if (fabsf(s_ - 1.0f) > 1e-5f) ok = 0; }
        CHECK(ok, "forward outputs are finite, ids in range, weights renormalised (flavour %d M %d)", flavour, M);
        CHECK(sp_moe_forward_dev(h, 0, NL, flavour, M, x_dev, y_dev, sel_dev, wts_dev, st) == SP_MOE_OK, "sp_moe_forward_dev");
        CHECK(sp_moe_status(h) == SP_MOE_OK, "sp_moe_status");
        CUDA_OK(cudaMemcpy(y2, y_dev, (size_t)M * E * 4, cudaMemcpyDeviceToHost));
        CHECK(memcmp(y, y2, (size_t)M * E * 4) == 0, "device entry == host entry, bit for bit (flavour %d M %d)", flavour, M);
    }
    CHECK(sp_moe_forward(h, 0, NL, 7, 1, x, y, NULL, NULL) == SP_MOE_EBADARG, "unknown flavour must be refused");
    CHECK(sp_moe_forward(h, 0, NL, 0, MT + 1, x, y, NULL, NULL) == SP_MOE_EBADARG, "M > max_tokens must be refused");
    CHECK(sp_moe_kernel_launches(h) > 0, "sp_moe_kernel_launches");

    /* ---- one layer in stages on one GPU (route -> experts -> finish) == forward_dev on that layer */
    for (int flavour = 0; flavour < 2; flavour++) {
        const int M = MT;
        int32_t *sel_asc = (int32_t *)dev_copy(NULL, M * NU * 4), *counts = (int32_t *)dev_copy(NULL, NE * 4), *pair_index = (int32_t *)dev_copy(NULL, M * NU * 4);
        float *cw = (float *)dev_copy(NULL, M * NU * 4), *rows = (float *)dev_copy(NULL, (size_t)M * NU * E * 4), *rows_out = (float *)dev_copy(NULL, (size_t)M * NU * E * 4);
        float *y_st = (float *)dev_copy(NULL, M * E * 4);
        CHECK(sp_moe_ep_route_dev(h, 0, flavour, M, x_dev, sel_asc, cw, rows, counts, pair_index, NULL, NULL, 1, 0, 0, st) == SP_MOE_OK, "sp_moe_ep_route_dev");
        CHECK(sp_moe_ep_shared_dev(h, 0, flavour, M, st) == SP_MOE_OK, "sp_moe_ep_shared_dev");
        int32_t hc[NE], off[NE + 1];
        CUDA_OK(cudaStreamSynchronize(st));
        CUDA_OK(cudaMemcpy(hc, counts, sizeof hc, cudaMemcpyDeviceToHost));
        off[0] = 0; for (int e = 0; e < NE; e++) off[e + 1] = off[e] + hc[e];
        CHECK(off[NE] == M * NU, "route counts add up to M * NU (%d)", off[NE]);
        int32_t *off_dev = (int32_t *)dev_copy(off, sizeof off);
        CHECK(sp_moe_ep_experts_dev(h, 0, flavour, M * NU, rows, NULL, off_dev, rows_out, st) == SP_MOE_OK, "sp_moe_ep_experts_dev");
        CHECK(sp_moe_ep_finish_dev(h, 0, M, x_dev, rows_out, pair_index, y_st, st) == SP_MOE_OK, "sp_moe_ep_finish_dev");
        CHECK(sp_moe_forward_dev(h, 0, 1, flavour, M, x_dev, y_dev, NULL, NULL, st) == SP_MOE_OK, "forward_dev (one layer)");
        CHECK(sp_moe_status(h) == SP_MOE_OK, "status after the staged run");
        CUDA_OK(cudaMemcpy(y, y_st, M * E * 4, cudaMemcpyDeviceToHost)); CUDA_OK(cudaMemcpy(y2, y_dev, M * E * 4, cudaMemcpyDeviceToHost));
        CHECK(memcmp(y, y2, M * E * 4) == 0, "staged layer == sp_moe_forward_dev, bit for bit (flavour %d)", flavour);
        /* the padded exchange's receive layout, one rank that is also its own source */
        int32_t *roff = (int32_t *)dev_copy(NULL, (NE + 1) * 4), *ridx = (int32_t *)dev_copy(NULL, M * NU * 4);
        CHECK(sp_moe_ep_recv_layout_dev(h, counts, 1, 0, M * NU, roff, ridx, st) == SP_MOE_OK, "sp_moe_ep_recv_layout_dev");
        int32_t hoff[NE + 1];
        CUDA_OK(cudaStreamSynchronize(st));
        CUDA_OK(cudaMemcpy(hoff, roff, sizeof hoff, cudaMemcpyDeviceToHost));
        CHECK(memcmp(hoff, off, sizeof off) == 0, "receive layout offsets == prefix sum of the counts");
        CHECK(sp_moe_ep_recv_layout_dev(h, counts, 3, 0, 4, roff, ridx, st) == SP_MOE_EBADARG, "recv_layout must refuse n_ranks that does not divide NE");
        cudaFree(sel_asc); cudaFree(counts); cudaFree(pair_index); cudaFree(cw); cudaFree(rows); cudaFree(rows_out); cudaFree(y_st); cudaFree(off_dev); cudaFree(roff); cudaFree(ridx);
    }

    /* ---- the expert-parallel loop inside the library, as a world of one rank: its own NCCL communicator,
     * every exchange a send to itself; both exchange kinds must reproduce sp_moe_forward_dev bit for bit.
     * Where libnccl is absent the entries say so and the section is skipped. */
    {
        unsigned char id[128];
        const int rc_id = sp_moe_ep_unique_id(id);
        if (rc_id == SP_MOE_EUNSUPPORTED) printf("note: no NCCL library here, expert-parallel loop not exercised\n");
        else {
            void *comm = NULL;
            CHECK(rc_id == SP_MOE_OK, "sp_moe_ep_unique_id");
            CHECK(sp_moe_ep_comm_create(id, 1, 0, &comm) == SP_MOE_OK && comm != NULL, "sp_moe_ep_comm_create");
            CHECK(sp_moe_ep_comm_create(id, 1, 3, &comm) == SP_MOE_EBADARG, "comm_create must refuse rank >= n_ranks");
            const int M = MT;
            float *y_ep = (float *)dev_copy(NULL, M * E * 4);
            for (int flavour = 0; flavour < 2 && comm; flavour++)
                for (int cap = 0; cap <= M * NU; cap += M * NU) {          /* exact exchange, then padded with room for every pair */
                    CHECK(sp_moe_ep_forward_dev(h, comm, 1, 0, 0, NL, flavour, M, x_dev, y_ep, cap, 1, st) == SP_MOE_OK, "sp_moe_ep_forward_dev (flavour %d, capacity %d)", flavour, cap);
                    CHECK(sp_moe_forward_dev(h, 0, NL, flavour, M, x_dev, y_dev, NULL, NULL, st) == SP_MOE_OK, "forward_dev");
                    CHECK(sp_moe_status(h) == SP_MOE_OK, "status after the expert-parallel loop");
                    CUDA_OK(cudaMemcpy(y, y_ep, M * E * 4, cudaMemcpyDeviceToHost)); CUDA_OK(cudaMemcpy(y2, y_dev, M * E * 4, cudaMemcpyDeviceToHost));
                    CHECK(memcmp(y, y2, M * E * 4) == 0, "library loop on one rank == sp_moe_forward_dev, bit for bit (flavour %d, capacity %d)", flavour, cap);
                    CHECK(sp_moe_ep_last_rows(h) == (cap ? cap : M * NU), "sp_moe_ep_last_rows = %lld", sp_moe_ep_last_rows(h));
                }
            {
                float ms6[6];
                const int rc_t = sp_moe_ep_timing(h, ms6);          /* stage events carry time only when the handle was opened with SP_MOE_TIMING=1 */
                if (getenv("SP_MOE_TIMING")) CHECK(rc_t == SP_MOE_OK && ms6[5] > 0.0f && ms6[0] >= 0.0f && ms6[4] >= 0.0f, "sp_moe_ep_timing (layer %.4f ms)", ms6[5]);
                else CHECK(rc_t == SP_MOE_EBADSTATE, "sp_moe_ep_timing without SP_MOE_TIMING must be refused");
                CHECK(sp_moe_ep_timing(h, NULL) == SP_MOE_EBADARG, "sp_moe_ep_timing must refuse NULL");
            }
            CHECK(sp_moe_ep_forward_dev(h, comm, 3, 0, 0, NL, 0, M, x_dev, y_ep, 0, 1, st) == SP_MOE_EBADARG, "ep_forward must refuse n_ranks that does not divide NE");
            CHECK(sp_moe_ep_forward_dev(h, NULL, 1, 0, 0, NL, 0, M, x_dev, y_ep, 0, 1, st) == SP_MOE_EBADARG, "ep_forward must refuse a NULL communicator");
            if (comm) CHECK(sp_moe_ep_comm_destroy(comm) == SP_MOE_OK, "sp_moe_ep_comm_destroy");
            cudaFree(y_ep);
        }
    }

    /* ---- the file loader and the bias setter: refusals (a real file is the Python tests' job) */
    CHECK(sp_moe_load_sp_model(h, "/nonexistent/model.sp-model", NULL) == SP_MOE_EBADARG && strstr(sp_last_error(), "cannot open") != NULL, "load_sp_model must refuse a missing file");
    CHECK(sp_moe_load_sp_model(h, NULL, NULL) == SP_MOE_EBADARG, "load_sp_model must refuse NULL");
    CHECK(sp_moe_set_router_bias_dev(h, 99, NULL) == SP_MOE_EBADARG, "set_router_bias must refuse a layer out of range");
    CHECK(sp_moe_set_router_bias_dev(h, 1, NULL) == SP_MOE_OK, "sp_moe_set_router_bias_dev");

    /* ---- timing entry (not switched on here) and the failure-path probe */
    sp_moe_timing tm;
    CHECK(sp_moe_decode_timing(h, &tm) == (getenv("SP_MOE_TIMING") ? SP_MOE_OK : SP_MOE_EBADSTATE), "sp_moe_decode_timing without/with SP_MOE_TIMING");
    CHECK(sp_moe_debug_wait_timeout(h, 1000, st) == SP_MOE_OK, "sp_moe_debug_wait_timeout launch");
    CHECK(sp_moe_status(h) == SP_MOE_ECUDA && strstr(sp_last_error(), "wait ran out") != NULL, "a wait that ran out is reported by sp_moe_status");
    CHECK(sp_moe_status(h) == SP_MOE_OK, "the error word is cleared once reported");
    CHECK(sp_moe_forward(h, 0, NL, 0, 1, x, y, NULL, NULL) == SP_MOE_OK, "the handle works after the reported timeout");

    /* ---- single-vector entries */
    {
        uint8_t *c, *cd; uint16_t *s, *sd;
        if (make_q4b(96, E, 0.02f, &c, &s, &cd, &sd)) return 1;
        float *ya = (float *)dev_copy(NULL, 96 * 4), *yb = (float *)dev_copy(NULL, 96 * 4);
        float ha[96], hb[96];
        CHECK(sp_moe_gemv_q4b_dev(cd, sd, E, 96, x_dev, ya, st) == SP_MOE_OK, "sp_moe_gemv_q4b_dev");
        CHECK(sp_moe_gemv_q4b_static_dev(cd, sd, E, 96, x_dev, yb, st) == SP_MOE_OK, "sp_moe_gemv_q4b_static_dev");
        CUDA_OK(cudaStreamSynchronize(st));
        CUDA_OK(cudaMemcpy(ha, ya, sizeof ha, cudaMemcpyDeviceToHost)); CUDA_OK(cudaMemcpy(hb, yb, sizeof hb, cudaMemcpyDeviceToHost));
        CHECK(memcmp(ha, hb, sizeof ha) == 0, "static-scratch GEMV == allocating GEMV");
        CHECK(sp_moe_gemv_q4b_static_dev(cd, sd, 4096 + 32, 1, x_dev, yb, st) == SP_MOE_EBADARG, "static GEMV must refuse in > 4096");
        CHECK(sp_moe_gelu_mul_dev(ya, yb, 96, ya, st) == SP_MOE_OK, "sp_moe_gelu_mul_dev");
        CUDA_OK(cudaStreamSynchronize(st));
        CUDA_OK(cudaMemcpy(hb, ya, sizeof hb, cudaMemcpyDeviceToHost));
        int ok = 1;
        for (int i = 0; i < 96; i++) { const double g = ha[i], ref = 0.5 * g * (1.0 + tanh(0.7978845608028654 * (g + 0.044715 * g * g * g))) * ha[i]; if (fabs(ref - hb[i]) > 1e-5 * (1.0 + fabs(ref))) ok = 0; }
        CHECK(ok, "gelu_mul values");
    }

    /* ---- the standalone operator (host pointers, verbatim reference signature) */
    {
        uint8_t *gc, *gcd, *dc, *dcd; uint16_t *gs, *gsd, *ds, *dsd;
        if (make_q4b((int64_t)NE * 2 * FFE, E, 0.02f, &gc, &gs, &gcd, &gsd) || make_q4b((int64_t)NE * E, FFE, 0.02f, &dc, &ds, &dcd, &dsd)) return 1;
        float gi[NE * E], gsc[E], out[E]; int so[NU];
        for (int i = 0; i < NE * E; i++) gi[i] = gauss() * 0.02f;
        for (int i = 0; i < E; i++) gsc[i] = 1.0f;
        CHECK(gemma4_moe_ffn_q4b_cuda(E, NE, NU, FFE, 1e-6f, gi, gsc, gc, gs, dc, ds, x, out, so) == 0, "gemma4_moe_ffn_q4b_cuda");
        int ok = so[0] != so[1] && so[0] >= 0 && so[0] < NE && so[1] >= 0 && so[1] < NE;
        for (int i = 0; i < E; i++) if (!isfinite(out[i])) ok = 0;
        CHECK(ok, "standalone operator outputs");
        CHECK(gemma4_moe_ffn_q4b_cuda(100, NE, NU, FFE, 1e-6f, gi, gsc, gc, gs, dc, ds, x, out, so) == 1, "standalone operator must refuse E %% 32 != 0");
    }

    /* ---- plugin hook */
    {
        sp_moe_ext *xh = NULL;
        CHECK(sp_moe_ext_open(0, &xh) == 0 && xh, "sp_moe_ext_open");
        uint8_t *c[3], *cd[3]; uint16_t *s[3], *sd[3];
        if (make_q4b((int64_t)NE * FFE, E, 0.02f, &c[0], &s[0], &cd[0], &sd[0]) || make_q4b((int64_t)NE * FFE, E, 0.02f, &c[1], &s[1], &cd[1], &sd[1]) ||
            make_q4b((int64_t)NE * E, FFE, 0.02f, &c[2], &s[2], &cd[2], &sd[2])) return 1;
        CHECK(sp_moe_ext_upload_experts(xh, "blk.0.ffn_gate_exps", c[0], s[0], c[1], s[1], c[2], s[2], NE, FFE, E) == 0, "sp_moe_ext_upload_experts");
        int idx[2] = {3, 5}; float wt[2] = {0.7f, 0.3f}, out[E];
        CHECK(sp_moe_ext_moe(xh, "blk.0.ffn_gate_exps", idx, wt, 2, x, E, FFE, out) == 0, "sp_moe_ext_moe");
        CHECK(sp_moe_ext_moe(xh, "blk.9.other", idx, wt, 2, x, E, FFE, out) != 0, "an unknown tag is 'not mine'");
        CHECK(sp_moe_ext_close(xh) == 0, "sp_moe_ext_close");
    }

    /* ---- quantised GEMM: C = f16(float(A.B^T) * sa * sb), small exact case */
    {
        enum { M = 128, N = 128, K = 64 };
        static int8_t A[M * K], B[N * K]; static float sa[M], sb[N]; static uint16_t Cq[M * N];
        for (int i = 0; i < M * K; i++) A[i] = (int8_t)((int)(frand() * 7) - 3);
        for (int i = 0; i < N * K; i++) B[i] = (int8_t)((int)(frand() * 7) - 3);
        for (int i = 0; i < M; i++) sa[i] = 1.0f;
        for (int i = 0; i < N; i++) sb[i] = 1.0f;
        int8_t *Ad = (int8_t *)dev_copy(A, sizeof A), *Bd = (int8_t *)dev_copy(B, sizeof B);
        float *sad = (float *)dev_copy(sa, sizeof sa), *sbd = (float *)dev_copy(sb, sizeof sb);
        uint16_t *Cd = (uint16_t *)dev_copy(NULL, sizeof Cq);
        CHECK(sp_frob_matmul_q8_dev(Ad, Bd, sad, sbd, Cd, M, K, N, st) == SP_MOE_OK, "sp_frob_matmul_q8_dev");
        CUDA_OK(cudaStreamSynchronize(st));
        CUDA_OK(cudaMemcpy(Cq, Cd, sizeof Cq, cudaMemcpyDeviceToHost));
        int ok = 1;
        for (int m = 0; m < M && ok; m += 17) for (int n = 0; n < N; n += 13) {
            int acc = 0; for (int k = 0; k < K; k++) acc += (int)A[m * K + k] * B[n * K + k];
            /* |acc| <= 576: exactly representable in f16 */
            const uint16_t hbits = Cq[m * N + n]; const int sgn = hbits >> 15, ex = (hbits >> 10) & 31, man = hbits & 1023;
            const float v = (ex == 0 ? ldexpf((float)man, -24) : ldexpf((float)(man | 1024), ex - 25)) * (sgn ? -1.0f : 1.0f);
            if (v != (float)acc) ok = 0;
        }
        CHECK(ok, "int8 GEMM values are exact");
        /* packed int4 operands: the same entry shape */
        static uint8_t A4[M * K / 2], B4[N * K / 2];
        for (int i = 0; i < M * K / 2; i++) A4[i] = (uint8_t)((A[2 * i] & 0xF) | ((A[2 * i + 1] & 0xF) << 4));
        for (int i = 0; i < N * K / 2; i++) B4[i] = (uint8_t)((B[2 * i] & 0xF) | ((B[2 * i + 1] & 0xF) << 4));
        uint8_t *A4d = (uint8_t *)dev_copy(A4, sizeof A4), *B4d = (uint8_t *)dev_copy(B4, sizeof B4);
        uint16_t *C4d = (uint16_t *)dev_copy(NULL, sizeof Cq); static uint16_t C4[M * N];
        CHECK(sp_frob_matmul_q4_dev(A4d, B4d, sad, sbd, C4d, M, K, N, st) == SP_MOE_OK, "sp_frob_matmul_q4_dev");
        CUDA_OK(cudaMemcpy(C4, C4d, sizeof C4, cudaMemcpyDeviceToHost));
        CHECK(memcmp(C4, Cq, sizeof Cq) == 0, "int4 GEMM == int8 GEMM on the same values");
    }

    CHECK(sp_moe_close(h) == SP_MOE_OK, "sp_moe_close");
    CHECK(sp_moe_close(NULL) == SP_MOE_OK, "sp_moe_close(NULL)");
    printf("%s: %d checks, %d failed\n", g_fail ? "FAILED" : "OK", g_checks, g_fail);
    return g_fail ? 1 : 0;
}
