"""GPU parity of the block-scaled FP8 (E4M3) kernel against the CPU oracle.

Tolerance (stated by the path's specification): max relative error 3e-2 against the
fp32-accumulated product of the dequantised operands, measured as
max |got-ref| / max(|ref|, 2^-7 rms(ref)).
"""
import numpy as np
import pytest

from oracle import gemm_oracle as O
from tesserae_b200 import api

pytestmark = pytest.mark.gpu
TOL_FP8 = 3e-2

_plans = {}


def plan_for(cg, bn, out_elem=api.BF16, bias=0, scaled=True):
    key = (cg, bn, out_elem, bias, scaled)
    if key not in _plans:
        if scaled:
            name = f"gemm_fp8blk_cg{cg}_n{bn}" + ("" if (out_elem == api.BF16 and not bias) else f"_o{out_elem}_b{bias}")
            spec = api.KernelSpec(name=name, elem=api.F8E4M3, tile=(128, bn, 128), cta_group=cg, out_elem=out_elem,
                                  has_bias=bias, scale_mode=api.SCALE_FP8_BLOCK)
        else:
            spec = api.KernelSpec(name="gemm_fp8_cg2_dense", elem=api.F8E4M3, tile=(128, 256, 128), cta_group=2,
                                  out_elem=api.BF16)
        _plans[key] = api.GemmPlan(spec)
    return _plans[key]


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU path to fall back to")
    torch.cuda.set_device(0)
    return torch


def run_scaled(torch, plan, p, m, n, k, out_elem=api.BF16, alpha=1.0):
    qa, qb = torch.from_numpy(p["qa"]).cuda(), torch.from_numpy(p["qb"]).cuda()
    sa, sb = torch.from_numpy(p["sa"]).cuda(), torch.from_numpy(p["sb"]).cuda()
    bias = torch.from_numpy(p["bias_bits"].view(np.int16)).view(torch.bfloat16).cuda() if p["bias_bits"] is not None else None
    c = torch.full((m, n), float("nan"), dtype=torch.bfloat16 if out_elem == api.BF16 else torch.float32, device="cuda")
    plan.run_scaled(qa, qb, c, sa, sb, bias, alpha, m, n, k, stream=torch.cuda.current_stream().cuda_stream)
    assert plan.status() == 0, "a bounded wait ran out inside the kernel"
    return c.float().cpu().numpy()


@pytest.mark.parametrize("cg,bn", [(1, 128), (1, 256), (2, 128), (2, 256)])
def test_parity_block_scaled(torch_cuda, cg, bn):
    plan = plan_for(cg, bn)
    for i, (m, n, k) in enumerate([(128 * cg, bn, 128), (256, 256, 512), (512, 1024, 1024), (200, 264, 256),
                                   (1, 8, 128), (1000, 1016, 384)]):
        p = O.make_fp8_problem(m, n, k, seed=200 + i)
        got = run_scaled(torch_cuda, plan, p, m, n, k)
        ref = O.gemm_f32(p["a"], p["b"])
        assert not np.isnan(got).any(), (cg, bn, m, n, k)
        e = O.rel_error(got, ref)
        assert e["max_rel"] <= TOL_FP8, (cg, bn, m, n, k, e)


def test_fp32_out_bias_alpha(torch_cuda):
    plan = plan_for(2, 256, api.F32, 1)
    m, n, k = 384, 512, 640
    p = O.make_fp8_problem(m, n, k, seed=31, with_bias=True)
    got = run_scaled(torch_cuda, plan, p, m, n, k, api.F32, alpha=0.5)
    e = O.rel_error(got, O.gemm_f32(p["a"], p["b"], 0.5, p["bias"]))
    assert e["max_rel"] <= 1e-3, e       # fp32 output: only the summation order differs


def test_scales_are_applied_per_block(torch_cuda):
    """Rows and blocks with very different magnitudes: a kernel that ignored or misplaced a scale
    would be off by orders of magnitude."""
    m, n, k = 256, 512, 512
    a = O.normal((m, k), 7) * (10.0 ** np.linspace(-3, 3, m, dtype=np.float32))[:, None]
    b = O.normal((n, k), 8)
    b[128:256] *= 50.0
    b[:, 256:384] *= 0.01
    qa, sa = O.quantize_fp8_rows_1x128(a)
    qb, sb = O.quantize_fp8_blocks_128x128(b)
    p = {"qa": qa, "sa": sa, "qb": qb, "sb": sb, "bias_bits": None}
    got = run_scaled(torch_cuda, plan_for(2, 256, api.F32, 0), p, m, n, k, api.F32)
    ref = O.gemm_f32(O.dequantize_fp8_rows(qa, sa), O.dequantize_fp8_blocks(qb, sb))
    rel_rows = np.abs(got - ref).max(axis=1) / np.maximum(np.abs(ref).max(axis=1), 1e-30)
    assert rel_rows.max() <= 1e-3


def test_unscaled_fp8_dense_kernel(torch_cuda):
    """E4M3 operands through the dense kernel (kind::f8f6f4, no scales): exact products, fp32 accumulation."""
    m, n, k = 512, 512, 1024
    qa = O.f32_to_e4m3_bits(O.normal((m, k), 3))
    qb = O.f32_to_e4m3_bits(O.normal((n, k), 4))
    t = torch_cuda
    c = t.empty((m, n), dtype=t.bfloat16, device="cuda")
    plan = plan_for(2, 256, scaled=False)
    plan.run(t.from_numpy(qa).cuda(), t.from_numpy(qb).cuda(), c, None, 1.0, m, n, k,
             stream=t.cuda.current_stream().cuda_stream)
    assert plan.status() == 0
    e = O.rel_error(c.float().cpu().numpy(), O.gemm_f32(O.e4m3_bits_to_f32(qa), O.e4m3_bits_to_f32(qb)))
    assert e["max_rel"] <= 1e-2


def test_config3_shape_sampled(torch_cuda):
    """FP8 GEMM M=8192, N=14336, K=4096 (N(0,1) sources, seed 2): sampled rows against the oracle in fp64
    and a row-sum identity over the whole output."""
    m, n, k = 8192, 14336, 4096
    p = O.make_fp8_problem(m, n, k, seed=2)
    t = torch_cuda
    plan = plan_for(2, 256, api.F32, 0)
    qa, qb = t.from_numpy(p["qa"]).cuda(), t.from_numpy(p["qb"]).cuda()
    sa, sb = t.from_numpy(p["sa"]).cuda(), t.from_numpy(p["sb"]).cuda()
    c = t.empty((m, n), dtype=t.float32, device="cuda")
    plan.run_scaled(qa, qb, c, sa, sb, None, 1.0, m, n, k, stream=t.cuda.current_stream().cuda_stream)
    assert plan.status() == 0
    rows = [0, 127, 128, 4097, 8191]
    cols = list(range(0, n, 131)) + [n - 1]
    want = O.gemm_f64_entries(p["a"], p["b"], rows, cols)
    got = c[rows][:, cols].cpu().numpy()
    rms = float(np.sqrt(np.mean(want ** 2)))
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), rms / 128)) <= TOL_FP8
    want_rowsum = p["a"].astype(np.float64) @ p["b"].astype(np.float64).sum(axis=0)
    got_rowsum = c.double().sum(dim=1).cpu().numpy()
    assert np.max(np.abs(got_rowsum - want_rowsum)) <= 1e-3 * float(np.sqrt(np.mean(want_rowsum ** 2)))


def test_needs_scales_and_k_multiple(torch_cuda):
    t = torch_cuda
    plan = plan_for(2, 256)
    x = t.zeros(256, 256, dtype=t.uint8, device="cuda")
    c = t.zeros(256, 256, dtype=t.bfloat16, device="cuda")
    with pytest.raises(api.TesseraeError, match="scale factors"):
        plan.run(x, x, c, None, 1.0, 256, 256, 256)
    s = t.ones(256, 2, device="cuda")
    with pytest.raises(api.TesseraeError, match="128-wide"):
        plan.run_scaled(x, x, c, s, s, None, 1.0, 256, 256, 192)


@pytest.mark.parametrize("tuning", ["FP8_SPLIT=0", "FP8_PROMO_WARPS=16"])
def test_structure_variants_agree(torch_cuda, tuning):
    """The kernel's structural variants (one 256-wide MMA chain instead of two 128-wide ones; sixteen promotion warps
    instead of eight) are other schedules of the same arithmetic: per K block the same fp32 partial product, scaled
    and added in the same order.  Their outputs must equal the default build's bit for bit."""
    m, n, k = 640, 768, 1024
    p = O.make_fp8_problem(m, n, k, seed=260)
    want = run_scaled(torch_cuda, plan_for(2, 256), p, m, n, k)
    variant = api.GemmPlan(api.KernelSpec(name="gemm_fp8blk_cg2_n256_variant", elem=api.F8E4M3, tile=(128, 256, 128),
                                          cta_group=2, out_elem=api.BF16, scale_mode=api.SCALE_FP8_BLOCK, tuning=tuning))
    got = run_scaled(torch_cuda, variant, p, m, n, k)
    variant.close()
    assert np.array_equal(got, want)


@pytest.mark.parametrize("m,n,k", [(384, 512, 640), (4608, 2048, 1024)])
def test_host_buffer_entry_point_equals_device_call(torch_cuda, m, n, k):
    """tesserae_gemm_run_scaled_host (operands, scale tables up; C back, inside the call; the larger case takes the
    chunked pipeline with a ragged last chunk) against the device-pointer call on the same inputs: bit-equal."""
    t = torch_cuda
    p = O.make_fp8_problem(m, n, k, seed=270)
    plan = plan_for(2, 256)
    want = run_scaled(t, plan, p, m, n, k)
    pin = lambda x: t.from_numpy(np.ascontiguousarray(x)).pin_memory()
    qa, qb, sa, sb = pin(p["qa"]), pin(p["qb"]), pin(p["sa"]), pin(p["sb"])
    c = t.full((m, n), float("nan"), dtype=t.bfloat16).pin_memory()
    plan.run_scaled_host(qa, qb, c, sa, sb, None, 1.0, m, n, k)
    assert plan.status() == 0
    assert np.array_equal(c.float().numpy(), want)


def tail_plan(cg, out_elem, bias, tuning):
    key = ("tail", cg, out_elem, bias, tuning)
    if key not in _plans:
        _plans[key] = api.GemmPlan(api.KernelSpec(name=f"gemm_fp8blk_tail_cg{cg}_o{out_elem}_b{bias}_{len(tuning)}", elem=api.F8E4M3,
                                                  tile=(128, 256, 128), cta_group=cg, out_elem=out_elem, has_bias=bias,
                                                  scale_mode=api.SCALE_FP8_BLOCK, tuning=tuning))
    return _plans[key]


@pytest.mark.parametrize("cg,out_elem,bias,tuning,shape", [
    (2, api.BF16, 0, "TAIL_SPLITS=16", (8192, 1792, 1024)),  # three whole waves of CTA pairs plus two tiles (one GPU's share of config 3 on 8)
    (2, api.BF16, 0, "TAIL_SPLITS=8", (512, 1024, 2048)),    # asked for: less than half a wave, every tile is split along K
    (2, api.F32, 1, "TAIL_SPLITS=16", (1000, 1016, 1536)),   # ragged edges, bias, fp32 out
    (1, api.BF16, 0, "TAIL_SPLITS=4", (512, 1024, 1024)),
])
def test_stream_k_tail(torch_cuda, cg, out_elem, bias, tuning, shape):
    """The workspace entry point: tiles past the last whole wave are computed as K ranges added into the workspace.
    Whole tiles are bit-equal to the plain entry point, tail tiles agree with the oracle, the workspace is left
    clear, and a second call through the same workspace gives the same answer within rounding."""
    torch = torch_cuda
    m, n, k = shape
    plan = tail_plan(cg, out_elem, bias, tuning)
    nbytes = plan.tail_workspace_bytes(m, n, k)
    assert nbytes > 0, "this shape is meant to have a tail on a B200"
    p = O.make_fp8_problem(m, n, k, seed=900 + m % 7, with_bias=bool(bias))
    ref = O.gemm_f32(p["a"], p["b"], 0.5, p["bias"])
    plain = run_scaled(torch, plan, p, m, n, k, out_elem, alpha=0.5)
    qa, qb = torch.from_numpy(p["qa"]).cuda(), torch.from_numpy(p["qb"]).cuda()
    sa, sb = torch.from_numpy(p["sa"]).cuda(), torch.from_numpy(p["sb"]).cuda()
    bias_d = torch.from_numpy(p["bias_bits"].view(np.int16)).view(torch.bfloat16).cuda() if bias else None
    ws = torch.zeros(nbytes // 4, dtype=torch.float32, device="cuda")
    tol = 1e-3 if out_elem == api.F32 else TOL_FP8
    for _ in range(2):
        c = torch.full((m, n), float("nan"), dtype=torch.bfloat16 if out_elem == api.BF16 else torch.float32, device="cuda")
        plan.run_scaled_ws(qa, qb, c, sa, sb, ws, nbytes, bias_d, 0.5, m, n, k, stream=torch.cuda.current_stream().cuda_stream)
        assert plan.status() == 0
        got = c.float().cpu().numpy()
        assert not np.isnan(got).any()
        assert O.rel_error(got, ref)["max_rel"] <= tol
        assert int(torch.count_nonzero(ws)) == 0, "the closing kernel leaves the workspace clear"
        same = got == plain
        # the entries that differ at all lie in the tail tiles and differ by rounding only
        assert np.abs(got - plain).max() <= 2e-2 * max(1.0, float(np.abs(plain).max()))
        tail_tiles = nbytes // (128 * cg * 256 * 4)
        assert (~same).sum() <= tail_tiles * 128 * cg * 256


def test_tail_workspace_rules(torch_cuda):
    torch = torch_cuda
    assert plan_for(2, 256).tail_workspace_bytes(8192, 1792, 4096) == 0     # a plan that did not ask for it never splits
    plan = tail_plan(2, api.BF16, 0, "TAIL_SPLITS=8")
    assert plan.tail_workspace_bytes(8192, 9472, 4096) == 0                 # 1184 tiles = 16 whole waves of 74 CTA pairs
    assert plan.tail_workspace_bytes(8192, 3328, 4096) == 0                 # 416 tiles: the 46 left over fill more than half the clusters
    assert plan.tail_workspace_bytes(8192, 1792, 4096) == 2 * 256 * 256 * 4
    m, n, k = 512, 1024, 2048
    need = plan.tail_workspace_bytes(m, n, k)
    p = O.make_fp8_problem(m, n, k, seed=5)
    qa, qb = torch.from_numpy(p["qa"]).cuda(), torch.from_numpy(p["qb"]).cuda()
    sa, sb = torch.from_numpy(p["sa"]).cuda(), torch.from_numpy(p["sb"]).cuda()
    c = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    ws = torch.zeros(need // 4, dtype=torch.float32, device="cuda")
    with pytest.raises(api.TesseraeError, match="tail workspace too small"):
        plan.run_scaled_ws(qa, qb, c, sa, sb, ws, need - 4, None, 1.0, m, n, k)
    # a plan told never to split takes no workspace and runs whole tiles
    whole = api.GemmPlan(api.KernelSpec(name="gemm_fp8blk_cg2_n256_notail", elem=api.F8E4M3, tile=(128, 256, 128), cta_group=2,
                                        out_elem=api.BF16, scale_mode=api.SCALE_FP8_BLOCK, tuning="TAIL_SPLITS=1"))
    assert whole.tail_workspace_bytes(m, n, k) == 0
    whole.run_scaled_ws(qa, qb, c, sa, sb, None, 0, None, 1.0, m, n, k)
    torch.cuda.synchronize()
    assert whole.status() == 0
    assert O.rel_error(c.float().cpu().numpy(), O.gemm_f32(p["a"], p["b"]))["max_rel"] <= TOL_FP8
