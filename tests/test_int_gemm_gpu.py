"""The quantised GEMM (int8 / packed int4 operands, int32 accumulate, per-row x per-column scales) on
tcgen05 kind::i8, bit for bit against the CPU checker's restatement of the reference's scalar
reference (src/backends/cuda/ptx_mma.cuh:375-405; epilogue ptx_mma_tile_common.cuh:157-176)."""
import numpy as np
import pytest

import orc

pytestmark = pytest.mark.gpu


def _case(M, N, K, seed):
    r = np.random.default_rng(seed)
    A = r.integers(-128, 128, (M, K), dtype=np.int8)
    B = r.integers(-128, 128, (N, K), dtype=np.int8)
    sa = (r.random(M).astype(np.float32) + 0.5) * 1e-3
    sb = (r.random(N).astype(np.float32) + 0.5) * 1e-2
    return A, B, sa, sb


@pytest.mark.parametrize("M,N,K", [(64, 64, 128), (200, 300, 272), (128, 256, 4096), (1, 8, 16), (513, 1000, 1040)])
def test_int8_bit_exact(M, N, K):
    import torch
    from kairos_engine_b200.engine import int_gemm_scaled
    A, B, sa, sb = _case(M, N, K, M + N + K)
    ref = orc.int_gemm_scaled(A, B, sa, sb)
    t = lambda a: torch.from_numpy(a).cuda()
    got = int_gemm_scaled(t(A), t(B), t(sa), t(sb))
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy().view(np.uint16), ref)


@pytest.mark.parametrize("M,N,K", [(96, 72, 256), (130, 520, 96)])
def test_packed_int4_bit_exact(M, N, K):
    import torch
    from kairos_engine_b200.engine import int_gemm_scaled
    r = np.random.default_rng(K)
    Aq = r.integers(0, 256, (M, K // 2), dtype=np.uint8)
    Bq = r.integers(0, 256, (N, K // 2), dtype=np.uint8)
    sa = (r.random(M).astype(np.float32) + 0.5) * 1e-2
    sb = (r.random(N).astype(np.float32) + 0.5) * 1e-1

    def unpack(q):                      # low nibble = even index; nib >= 8 -> nib - 16
        lo = (q & 15).astype(np.int16); hi = (q >> 4).astype(np.int16)
        out = np.empty((q.shape[0], q.shape[1] * 2), np.int16)
        out[:, 0::2] = np.where(lo >= 8, lo - 16, lo); out[:, 1::2] = np.where(hi >= 8, hi - 16, hi)
        return out.astype(np.int8)
    ref = orc.int_gemm_scaled(unpack(Aq), unpack(Bq), sa, sb)
    t = lambda a: torch.from_numpy(a).cuda()
    got = int_gemm_scaled(t(Aq), t(Bq), t(sa), t(sb), packed_int4=True)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy().view(np.uint16), ref)


def test_bad_arguments_are_refused():
    import torch
    from kairos_engine_b200 import SpMoeError
    from kairos_engine_b200.engine import int_gemm_scaled
    A = torch.zeros((4, 24), dtype=torch.int8, device="cuda")       # K not a multiple of 16
    with pytest.raises(SpMoeError):
        int_gemm_scaled(A, A, torch.ones(4, device="cuda"), torch.ones(4, device="cuda"))
