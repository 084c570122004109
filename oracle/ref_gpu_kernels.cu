/* ref_gpu_kernels.cu — the reference's OWN decode kernels on this GPU, as a timing baseline.
 * TEST INFRASTRUCTURE ONLY (built into oracle/_ref by `make -C oracle ref_gpu`; loaded by bench.py's
 * baseline leg and by nothing in the product).
 *
 * tools/moe_cpu_bench/moe_cpu_bench.cu of the reference holds verbatim copies of the three kernels
 * its served decode path runs per routed expert (k_quant_act_int8, k_gemv_q4b_dp4a_v2,
 * k_moe_gelu_split_batch; lines 35-94 there). That file is compiled from where it lies in the
 * reference tree - it is included below, never copied - with its program entry renamed away, and
 * this wrapper launches the kernels exactly as its main does (lines 247-252): one expert =
 * quantise x, gate|up GEMV (2*FFE rows, warp per row, 8 rows per block), GeGLU split, quantise h,
 * down GEMV (E rows). Geometry is the file's own (E = 2816, FFE = 704). */
#define main sp_ref_moe_cpu_bench_program_entry      /* its benchmark program is not wanted, only its kernels */
#include "tools/moe_cpu_bench/moe_cpu_bench.cu"
#undef main

extern "C" int sp_ref_gpu_geometry(int *e, int *ffe) { *e = E; *ffe = FFE; return 0; }

/* Runs n_experts routed experts back to back on `stream` (what one decode token's routed branch does per
 * layer with NU = n_experts), expert k reading the packed tensors at index ids[k] of the given arrays
 * (gate|up: [2*FFE][E/2] codes + [2*FFE][E/32] f16 scales per expert; down: [E][FFE/2] + [E][FFE/32]).
 * row_off_gu / row_off_dn: the byte offset of every row, as the reference's kernels take them. */
extern "C" int sp_ref_gpu_experts(const float *x_dev, const unsigned char *gu_codes, const unsigned short *gu_bs,
                                  const unsigned char *dn_codes, const unsigned short *dn_bs,
                                  const unsigned long long *row_off_gu, const unsigned long long *row_off_dn,
                                  const int *ids, int n_experts, signed char *qx, float *sx, float *gu, float *h, float *out, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    const size_t gub = (size_t)2 * FFE * (E / 2), gusb = (size_t)2 * FFE * (E / 32);
    const size_t dwb = (size_t)E * (FFE / 2), dwsb = (size_t)E * (FFE / 32);
    for (int k = 0; k < n_experts; k++) {
        const size_t e = (size_t)ids[k];
        k_quant_act_int8<<<1, 256, 0, st>>>(x_dev, E, E, qx, sx);
        k_gemv_q4b_dp4a_v2<<<(2 * FFE + 7) / 8, 256, 0, st>>>(gu_codes + e * gub, row_off_gu, gu_bs + e * gusb, E / 32, E, qx, sx, gu, 2 * FFE);
        k_moe_gelu_split_batch<<<(FFE + 255) / 256, 256, 0, st>>>(gu, FFE, 1, h);
        k_quant_act_int8<<<1, 256, 0, st>>>(h, FFE, FFE, qx, sx);
        k_gemv_q4b_dp4a_v2<<<(E + 7) / 8, 256, 0, st>>>(dn_codes + e * dwb, row_off_dn, dn_bs + e * dwsb, FFE / 32, FFE, qx, sx, out + (size_t)k * E, E);
    }
    return (int)cudaGetLastError();
}
