"""Times the quantised GEMM (sp_frob_matmul_q8_dev) alone: `python -m kairos_engine_b200.bench_int_gemm [M N K]`.
bench.py reports the same number in its `int_gemm` object; this entry exists so one kernel can be profiled
without the rest of the bench around it."""
import sys

import torch

from .engine import int_gemm_scaled


def main():
    M, N, K = (int(v) for v in sys.argv[1:4]) if len(sys.argv) >= 4 else (8192, 8192, 8192)
    g = torch.Generator(device="cuda").manual_seed(11)
    A = torch.randint(-128, 128, (M, K), dtype=torch.int8, device="cuda", generator=g)
    B = torch.randint(-128, 128, (N, K), dtype=torch.int8, device="cuda", generator=g)
    sa = torch.rand(M, device="cuda", generator=g) * 1e-3
    sb = torch.rand(N, device="cuda", generator=g) * 1e-3
    for _ in range(3):
        int_gemm_scaled(A, B, sa, sb)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(10):
        int_gemm_scaled(A, B, sa, sb)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 10
    print(f"int8 GEMM {M}x{N}x{K}: {ms:.3f} ms, {2.0 * M * N * K / ms / 1e9:.1f} TOPS")


if __name__ == "__main__":
    main()
