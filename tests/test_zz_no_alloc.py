"""The allocation-free GEMV entry point (sp_moe_gemv_q4b_static_dev) against the allocating one
(sp_moe_gemv_q4b_dev), through the C ABI.

It exists for callers that are not allowed to allocate device memory at call time (everything on
the card is already committed to pre-sized arenas, or the component only works in buffers it is
handed); its scratch is a fixed array inside the library. This file is collected last on purpose:
a run that stops at the first failure has then already run every other test. Two calls in a row
must both match bit for bit - the second one reuses whatever the first left in the scratch.
"""
import ctypes as C

import numpy as np
import pytest

import orc

pytestmark = pytest.mark.gpu


def _call(fn, codes, bs, x, rows, cols):
    import torch
    y = torch.empty(rows, dtype=torch.float32, device=codes.device)
    rc = fn(codes.data_ptr(), bs.data_ptr(), cols, rows, x.data_ptr(), y.data_ptr(),
            torch.cuda.current_stream(codes.device).cuda_stream)
    torch.cuda.synchronize()
    return rc, y.cpu().numpy()


def test_static_scratch_gemv_matches_allocating_entry_twice_in_a_row():
    import torch
    from kairos_engine_b200 import _lib, q4b_quantize
    L = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(123)
    shapes = [(1408, 2816), (2816, 704)]            # first call: in = 2816; second: a smaller in, on top of the first call's leftovers
    for rows, cols in shapes:
        w = torch.randn((rows, cols), generator=g, device="cuda") * 0.02
        codes, bs = q4b_quantize(w)
        x = torch.randn(cols, generator=g, device="cuda")
        rc_ref, y_ref = _call(L.sp_moe_gemv_q4b_dev, codes, bs, x, rows, cols)
        rc_new, y_new = _call(L.sp_moe_gemv_q4b_static_dev, codes, bs, x, rows, cols)
        assert rc_ref == 0 and rc_new == 0, L.sp_last_error()
        # same kernels, same arithmetic: the tolerance the other GEMV tests use is bit equality
        assert np.array_equal(y_new.view(np.uint32), y_ref.view(np.uint32))
        # and directly against the CPU checker (itself pinned to the reference's sp_moe_cpu_gemv)
        qx, sx = orc.quant_act(x.cpu().numpy())
        ref = orc.gemv_a(codes.cpu().numpy(), bs.cpu().numpy().view(np.uint16), rows, cols, qx, sx)
        assert np.array_equal(y_new.view(np.uint32), ref.view(np.uint32))


def test_static_scratch_gemv_refuses_sizes_beyond_its_array():
    import torch
    from kairos_engine_b200 import _lib
    L = _lib.lib()
    dummy = torch.zeros(16, device="cuda")
    rc = L.sp_moe_gemv_q4b_static_dev(dummy.data_ptr(), dummy.data_ptr(), 4096 + 32, 1, dummy.data_ptr(), dummy.data_ptr(), None)
    assert rc == -3 and b"exceeds the fixed scratch" in L.sp_last_error()
