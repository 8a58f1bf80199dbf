"""The allocation-free K-split entry point (tesserae_gemm_ksplit_run_noalloc), called through the C ABI.

It serves hosts that cannot call cudaMalloc when they need the GEMM (their own allocator already owns the
GPU's memory, or they cannot take the synchronisation an allocation implies): the fp32 partial products go to
a fixed array inside the library instead of caller scratch.  Its output must equal the ordinary entry point's
bit for bit (same kernels, same order of additions), on two calls in a row that share the array, and sizes
beyond the array must be refused with a clear message.  This file sorts last on purpose: a run that stops at
the first failure has then already run every other test.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import gemm_oracle as O
from tesserae_b200 import api
from tesserae_b200 import _native as N

pytestmark = pytest.mark.gpu


def _dev(torch, bits):
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()


def test_noalloc_matches_ordinary_entry_point_twice():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU path to fall back to")
    torch.cuda.set_device(0)
    lib = N.lib()
    assert lib.tesserae_gemm_ksplit_noalloc_max_elems() == 8388608
    plan = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_b0", elem=api.BF16, tile=(128, 256, 64), cta_group=2,
                                       out_elem=api.F32))
    stream = torch.cuda.current_stream().cuda_stream
    # The set-up call a host makes at start-up: its size is refused, but it still resolves the built-in array on
    # this device, which is when the driver reserves it.  After it, a call must leave free device memory untouched.
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    assert lib.tesserae_gemm_ksplit_run_noalloc(plan._h, C.c_void_p(x.data_ptr()), C.c_void_p(x.data_ptr()),
                                                C.c_void_p(x.data_ptr()), 1.0, 4096, 4096, 1024, 1, None) != 0
    # two calls in a row share the built-in array; the second has other inputs, another shape and another split
    for call, (m, n, k, splits, alpha) in enumerate([(1024, 2048, 1024, 4, 1.0), (520, 1024, 2048, 2, 0.5)]):
        p = O.make_bf16_problem(m, n, k, seed=500 + call, scale=0.5)
        a, b = _dev(torch, p["a_bits"]), _dev(torch, p["b_bits"])
        want = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        nbytes = api.ksplit_scratch_bytes(m, n, splits)
        scratch = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        plan.ksplit_run(a, b, want, scratch, nbytes, m, n, k, splits, alpha=alpha, stream=stream)
        got = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        N.check(lib.tesserae_gemm_ksplit_run_noalloc(plan._h, C.c_void_p(a.data_ptr()), C.c_void_p(b.data_ptr()),
                                                     C.c_void_p(got.data_ptr()), alpha, m, n, k, splits,
                                                     C.c_void_p(stream)), "ksplit_run_noalloc")
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, f"call {call}: free device memory changed across the call"
        assert plan.status() == 0
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), f"call {call}: outputs differ"
        e = O.rel_error(got.float().cpu().numpy(), O.gemm_f32(p["a"], p["b"], alpha))
        assert e["max_rel"] <= 1e-2, e        # and both agree with the oracle within the bf16 tolerance
    plan.close()


def test_noalloc_refuses_sizes_beyond_the_array():
    import torch
    torch.cuda.set_device(0)
    lib = N.lib()
    plan = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_b0", elem=api.BF16, tile=(128, 256, 64), cta_group=2,
                                       out_elem=api.F32))
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    rc = lib.tesserae_gemm_ksplit_run_noalloc(plan._h, C.c_void_p(x.data_ptr()), C.c_void_p(x.data_ptr()),
                                              C.c_void_p(x.data_ptr()), 1.0, 4096, 4096, 1024, 1, None)
    assert rc != 0
    msg = N.last_error()
    assert "16777216" in msg and "8388608" in msg and "exceed" in msg, msg
    plan.close()
