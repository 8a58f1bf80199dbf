"""GPU parity of the NVFP4 kernel (E2M1 operands, UE4M3 scale per 16, fp32 per tensor) against the CPU oracle.

Tolerance (stated by the path's specification): max relative error 3e-2 against the fp32-accumulated
product of the dequantised operands, measured as max |got-ref| / max(|ref|, 2^-7 rms(ref)).
"""
import numpy as np
import pytest

from oracle import gemm_oracle as O
from tesserae_b200 import api

pytestmark = pytest.mark.gpu
TOL_NVFP4 = 3e-2

_plans = {}


def plan_for(cg, bn, out_elem=api.BF16, bias=0):
    key = (cg, bn, out_elem, bias)
    if key not in _plans:
        name = f"gemm_nvfp4_cg{cg}_n{bn}" + ("" if (out_elem == api.BF16 and not bias) else f"_o{out_elem}_b{bias}")
        _plans[key] = api.GemmPlan(api.KernelSpec(name=name, elem=api.F4E2M1, tile=(128, bn, 256), cta_group=cg,
                                                  out_elem=out_elem, has_bias=bias, scale_mode=api.SCALE_NVFP4))
    return _plans[key]


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU path to fall back to")
    torch.cuda.set_device(0)
    return torch


def run(torch, plan, p, m, n, k, out_elem=api.BF16, alpha=1.0):
    dev = lambda x: torch.from_numpy(np.ascontiguousarray(x)).cuda()
    qa, qb, sfa, sfb = dev(p["qa"]), dev(p["qb"]), dev(p["sfa"]), dev(p["sfb"])
    bias = torch.from_numpy(p["bias_bits"].view(np.int16)).view(torch.bfloat16).cuda() if p["bias_bits"] is not None else None
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16 if out_elem == api.BF16 else torch.float32, device="cuda")
    plan.run_scaled(qa, qb, c, sfa, sfb, bias, alpha, m, n, k, stream=torch.cuda.current_stream().cuda_stream,
                    global_a=p["ga"], global_b=p["gb"])
    assert plan.status() == 0, "a bounded wait ran out inside the kernel"
    return c.float().cpu().numpy()


@pytest.mark.parametrize("cg,bn", [(1, 128), (1, 256), (2, 128), (2, 256)])
def test_parity(torch_cuda, cg, bn):
    plan = plan_for(cg, bn, api.F32)
    for i, (m, n, k) in enumerate([(128 * cg, bn, 256), (256, 256, 512), (512, 1024, 1024), (200, 264, 256),
                                   (1, 8, 256), (1000, 1016, 768)]):
        p = O.make_nvfp4_problem(m, n, k, seed=300 + i)
        got = run(torch_cuda, plan, p, m, n, k, api.F32)
        ref = O.gemm_f32(p["a"], p["b"])
        assert not np.isnan(got).any(), (cg, bn, m, n, k)
        e = O.rel_error(got, ref)
        assert e["max_rel"] <= 1e-3, (cg, bn, m, n, k, e)     # fp32 out: products are exact, only summation order differs


def test_bf16_out_bias_alpha(torch_cuda):
    m, n, k = 384, 512, 1024
    p = O.make_nvfp4_problem(m, n, k, seed=41, with_bias=True)
    got = run(torch_cuda, plan_for(2, 256, api.BF16, 1), p, m, n, k, api.BF16, alpha=0.5)
    e = O.rel_error(got, O.gemm_f32(p["a"], p["b"], 0.5, p["bias"]))
    assert e["max_rel"] <= TOL_NVFP4, e


def test_scale_placement(torch_cuda):
    """Every 16-wide block gets a different magnitude, so a misplaced scale byte shows up at once."""
    m, n, k = 256, 256, 512
    rng = np.random.default_rng(5)
    a = O.normal((m, k), 9) * np.repeat(2.0 ** rng.integers(-6, 4, (m, k // 16)), 16, axis=1).astype(np.float32)
    b = O.normal((n, k), 10) * np.repeat(2.0 ** rng.integers(-6, 4, (n, k // 16)), 16, axis=1).astype(np.float32)
    qa, sa, ga = O.quantize_nvfp4(a)
    qb, sb, gb = O.quantize_nvfp4(b)
    p = {"qa": O.pack_e2m1(qa), "qb": O.pack_e2m1(qb), "sfa": O.nvfp4_scale_chunks(sa), "sfb": O.nvfp4_scale_chunks(sb),
         "ga": float(ga), "gb": float(gb), "bias_bits": None}
    got = run(torch_cuda, plan_for(2, 256, api.F32), p, m, n, k, api.F32)
    ref = O.gemm_f32(O.dequantize_nvfp4(qa, sa, ga), O.dequantize_nvfp4(qb, sb, gb))
    assert O.rel_error(got, ref)["max_rel"] <= 1e-3


def test_config4_shape_sampled(torch_cuda):
    """NVFP4 GEMM at a column shard of config 4 (M=16384, N=28672/8, K=8192, N(0,1) sources seed 3): sampled
    entries in fp64 and a row-sum identity over the whole output."""
    m, n, k = 16384, 3584, 8192
    p = O.make_nvfp4_problem(m, n, k, seed=3)
    t = torch_cuda
    dev = lambda x: t.from_numpy(np.ascontiguousarray(x)).cuda()
    plan = plan_for(2, 256, api.F32)
    c = t.empty((m, n), dtype=t.float32, device="cuda")
    plan.run_scaled(dev(p["qa"]), dev(p["qb"]), c, dev(p["sfa"]), dev(p["sfb"]), None, 1.0, m, n, k,
                    stream=t.cuda.current_stream().cuda_stream, global_a=p["ga"], global_b=p["gb"])
    assert plan.status() == 0
    rows = [0, 127, 128, 8191, 16383]
    cols = list(range(0, n, 53)) + [n - 1]
    want = O.gemm_f64_entries(p["a"], p["b"], rows, cols)
    got = c[rows][:, cols].cpu().numpy()
    rms = float(np.sqrt(np.mean(want ** 2)))
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), rms / 128)) <= TOL_NVFP4
    want_rowsum = p["a"].astype(np.float64) @ p["b"].astype(np.float64).sum(axis=0)
    got_rowsum = c.double().sum(dim=1).cpu().numpy()
    assert np.max(np.abs(got_rowsum - want_rowsum)) <= 1e-3 * float(np.sqrt(np.mean(want_rowsum ** 2)))


def test_k_must_be_a_stage_multiple(torch_cuda):
    t = torch_cuda
    x = t.zeros(256, 256, dtype=t.uint8, device="cuda")
    c = t.zeros(256, 256, dtype=t.bfloat16, device="cuda")
    with pytest.raises(api.TesseraeError, match="multiple of 256"):
        plan_for(2, 256).run_scaled(x, x, c, x, x, None, 1.0, 256, 256, 384)


def test_config4_full_size(torch_cuda):
    """NVFP4 GEMM at the full size of config 4 (M=16384, N=28672, K=8192; N(0,1) sources, seed 3).  The sources
    are drawn on the GPU and quantised by the library's GPU quantisers; the check reads the quantised bytes back
    and dequantises them with the oracle: sampled entries in fp64, and the row-sum identity
    sum_n C[m,n] = a[m,:] . sum_n b[n,:] over the whole output."""
    from helpers import fullsize as F
    t = torch_cuda
    m, n, k = 16384, 28672, 8192
    s = t.cuda.current_stream().cuda_stream
    ws4 = t.zeros(4, dtype=t.uint8, device="cuda")
    ops = []
    for rows_, seed in ((m, 3), (n, 1003)):
        src = F.draw(t, (rows_, k), seed)
        q = t.empty((rows_, k // 2), dtype=t.uint8, device="cuda")
        sf = t.zeros((api.nvfp4_scale_bytes(rows_, k),), dtype=t.uint8, device="cuda")
        g = api.quantize_nvfp4(src, q, sf, ws4, rows_, k, stream=s)
        del src
        ops.append((q, sf, g))
    (qa, sfa, ga), (qb, sfb, gb) = ops
    c = t.empty((m, n), dtype=t.float32, device="cuda")
    plan = plan_for(2, 256, api.F32)
    plan.run_scaled(qa, qb, c, sfa, sfb, None, 1.0, m, n, k, stream=s, global_a=ga, global_b=gb)
    assert plan.status() == 0
    rows = [0, 127, 128, 8191, 16383]
    cols = list(range(0, n, 211)) + [n - 1]
    a_s = F.nvfp4_rows_from_device(t, qa, sfa, ga, rows, k)
    b_s = F.nvfp4_rows_from_device(t, qb, sfb, gb, cols, k)
    want = a_s.astype(np.float64) @ b_s.astype(np.float64).T
    got = c[rows][:, cols].cpu().numpy()
    rms = float(np.sqrt(np.mean(want ** 2)))
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), rms / 128)) <= TOL_NVFP4
    colsum = np.zeros(k, dtype=np.float64)
    for _, blk in F.nvfp4_all_from_device(t, qb, sfb, gb, n, k):
        colsum += blk.astype(np.float64).sum(axis=0)
    got_rowsum = c.double().sum(dim=1).cpu().numpy()
    want_rowsum = np.empty(m, dtype=np.float64)
    for r0, blk in F.nvfp4_all_from_device(t, qa, sfa, ga, m, k):
        want_rowsum[r0:r0 + len(blk)] = blk.astype(np.float64) @ colsum
    assert np.max(np.abs(got_rowsum - want_rowsum)) <= 1e-3 * float(np.sqrt(np.mean(want_rowsum ** 2)))


@pytest.mark.parametrize("m,n,k", [(384, 512, 1024), (4608, 1024, 1024)])
def test_host_buffer_entry_point_equals_device_call(torch_cuda, m, n, k):
    """tesserae_gemm_run_scaled_host (operands and chunked scale tables up; C back, inside the call; the larger case
    takes the chunked pipeline with a ragged last chunk) against the device-pointer call: bit-equal."""
    t = torch_cuda
    p = O.make_nvfp4_problem(m, n, k, seed=370)
    plan = plan_for(2, 256)
    want = run(t, plan, p, m, n, k)
    pin = lambda x: t.from_numpy(np.ascontiguousarray(x)).pin_memory()
    qa, qb, sfa, sfb = pin(p["qa"]), pin(p["qb"]), pin(p["sfa"]), pin(p["sfb"])
    c = t.full((m, n), float("nan"), dtype=t.bfloat16).pin_memory()
    plan.run_scaled_host(qa, qb, c, sfa, sfb, None, 1.0, m, n, k, global_a=p["ga"], global_b=p["gb"])
    assert plan.status() == 0
    assert np.array_equal(c.float().numpy(), want)
