"""GPU parity: the sm_100a kernels, called through the C ABI, against the CPU oracle.

Tolerance (stated by the path's specification): fp32-accumulated output within max relative
error 1e-2 of the oracle for bf16 operands, measured as max |got-ref| / max(|ref|, 2^-7 rms(ref)).
fp32-output cases are held to 1e-3 (they differ from the oracle only by summation order).
"""
import json

import numpy as np
import pytest

from conftest import ROOT
from oracle import gemm_oracle as O
from tesserae_b200 import api

pytestmark = pytest.mark.gpu
TOL_BF16_OUT = 1e-2
TOL_F32_OUT = 1e-3


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU path to fall back to")
    torch.cuda.set_device(0)
    return torch


_plans = {}


def plan_for(cg, out_elem, bias, tile_n=256):
    key = (cg, out_elem, bias, tile_n)
    if key not in _plans:
        name = f"gemm_bf16_cg{cg}_{'bf16' if out_elem == api.BF16 else 'f32'}_b{bias}" if tile_n == 256 else f"gemm_bf16_cg{cg}_n{tile_n}"
        _plans[key] = api.GemmPlan(api.KernelSpec(name=name, elem=api.BF16, tile=(128, tile_n, 64), cta_group=cg,
                                                  out_elem=out_elem, has_bias=bias))
    return _plans[key]


def to_dev(torch, bits):
    return torch.from_numpy(bits.view(np.int16)).view(torch.bfloat16).cuda()


def run_gpu(torch, plan, p, m, n, k, out_elem, alpha=1.0):
    a, b = to_dev(torch, p["a_bits"]), to_dev(torch, p["b_bits"])
    bias = to_dev(torch, p["bias_bits"]) if p["bias_bits"] is not None else None
    c = torch.full((m, n), float("nan"), dtype=torch.float32 if out_elem == api.F32 else torch.bfloat16, device="cuda")
    plan.run(a, b, c, bias, alpha, m, n, k, stream=torch.cuda.current_stream().cuda_stream)
    assert plan.status() == 0, "a bounded wait ran out inside the kernel"
    return c.float().cpu().numpy()


SHAPES = [(128, 256, 64), (256, 256, 64), (512, 512, 512), (200, 264, 72), (1, 8, 8), (129, 8, 520), (1000, 1016, 1032),
          (64, 4096, 128), (4096, 64, 128)]


@pytest.mark.parametrize("cg", [1, 2])
@pytest.mark.parametrize("out_elem,bias", [(api.F32, 0), (api.BF16, 0), (api.BF16, 1), (api.F32, 1)])
def test_parity_small_and_ragged(torch_cuda, cg, out_elem, bias):
    plan = plan_for(cg, out_elem, bias)
    for i, (m, n, k) in enumerate(SHAPES):
        p = O.make_bf16_problem(m, n, k, seed=100 + i, with_bias=bool(bias))
        got = run_gpu(torch_cuda, plan, p, m, n, k, out_elem, alpha=0.75)
        ref = O.gemm_f32(p["a"], p["b"], 0.75, p["bias"])
        assert not np.isnan(got).any(), (m, n, k)
        e = O.rel_error(got, ref)
        assert e["max_rel"] <= (TOL_F32_OUT if out_elem == api.F32 else TOL_BF16_OUT), (cg, m, n, k, e)


@pytest.mark.parametrize("cg", [1, 2])
def test_config1_bf16_512_cubed(torch_cuda, cg):
    """bf16 GEMM M=N=K=512, U[-1,1) seed 0, fp32 accumulate, bf16 output; also against the committed fixture."""
    g = json.loads((ROOT / "tests" / "golden" / "gemm_goldens.json").read_text())["cases"][0]
    p = O.make_bf16_problem(512, 512, 512, seed=0)
    got = run_gpu(torch_cuda, plan_for(cg, api.BF16, 0), p, 512, 512, 512, api.BF16)
    ref = O.round_to_bf16(O.gemm_f32(p["a"], p["b"]))
    e = O.rel_error(got, ref)
    assert e["max_rel"] <= TOL_BF16_OUT, e
    want = np.array(g["values_f64"])
    sub = got[np.ix_(g["rows"], g["cols"])]
    assert np.max(np.abs(sub - want) / np.maximum(np.abs(want), 2.0 ** -7 * e["rms_ref"])) <= TOL_BF16_OUT


@pytest.mark.parametrize("cg", [1, 2])
def test_fixture_cases_fp32_out(torch_cuda, cg):
    g = json.loads((ROOT / "tests" / "golden" / "gemm_goldens.json").read_text())
    for c in g["cases"]:
        p = O.make_bf16_problem(c["m"], c["n"], c["k"], c["seed"], c["dist"], c["scale"], with_bias=c["bias"])
        got = run_gpu(torch_cuda, plan_for(cg, api.F32, int(c["bias"])), p, c["m"], c["n"], c["k"], api.F32)
        want = np.array(c["values_f64"])
        sub = got[np.ix_(c["rows"], c["cols"])]
        rms = np.sqrt(np.mean(want * want))
        assert np.max(np.abs(sub - want) / np.maximum(np.abs(want), 2.0 ** -7 * rms)) <= TOL_F32_OUT, c["name"]
        assert abs(float(got.astype(np.float64).sum()) - c["c_f32_sum"]) <= 1e-5 * c["c_f32_abs_sum"], c["name"]


def test_tile_n_128_variants(torch_cuda):
    for cg in (1, 2):
        plan = plan_for(cg, api.BF16, 0, tile_n=128)
        p = O.make_bf16_problem(384, 640, 256, seed=21)
        got = run_gpu(torch_cuda, plan, p, 384, 640, 256, api.BF16)
        assert O.rel_error(got, O.gemm_f32(p["a"], p["b"]))["max_rel"] <= TOL_BF16_OUT


def test_config2_full_size_properties(torch_cuda):
    """8192^3 with N(0,1)*0.05 inputs, alpha=1, per-column bias, bf16 out (2-CTA kernel).  The full
    product is checked on sampled rows in fp64, and by size-independent properties: exact
    linearity in a power-of-two alpha, agreement of the 1-CTA and 2-CTA kernels, and a checksum
    identity sum_n C[m,n] = A[m,:] . sum_n B[n,:] + sum(bias)."""
    torch = torch_cuda
    m = n = k = 8192
    p = O.make_bf16_problem(m, n, k, seed=1, dist="normal", scale=0.05, with_bias=True)
    a, b, bias = to_dev(torch, p["a_bits"]), to_dev(torch, p["b_bits"]), to_dev(torch, p["bias_bits"])
    s = torch.cuda.current_stream().cuda_stream

    def run(cg, out_elem, alpha):
        plan = plan_for(cg, out_elem, 1)
        c = torch.empty((m, n), dtype=torch.float32 if out_elem == api.F32 else torch.bfloat16, device="cuda")
        plan.run(a, b, c, bias, alpha, m, n, k, stream=s)
        assert plan.status() == 0
        return c

    c2 = run(2, api.BF16, 1.0)
    rows = [0, 1, 127, 128, 255, 256, 4095, 4096, 8191, 3333, 7001]
    cols = list(range(0, n, 97)) + [n - 1]
    want = O.gemm_f64_entries(p["a"], p["b"], rows, cols, 1.0, p["bias"])
    got = c2[rows][:, cols].float().cpu().numpy()
    rms = float(np.sqrt(np.mean(want * want)))
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), 2.0 ** -7 * rms)) <= TOL_BF16_OUT

    f1 = run(2, api.F32, 1.0)
    # checksum of checksums in fp64 against the inputs
    colsum_b = p["b"].astype(np.float64).sum(axis=0)
    want_rowsum = p["a"].astype(np.float64) @ colsum_b + p["bias"].astype(np.float64).sum()
    got_rowsum = f1.double().sum(dim=1).cpu().numpy()
    scale = float(np.sqrt(np.mean(want_rowsum ** 2)))
    assert np.max(np.abs(got_rowsum - want_rowsum)) <= 1e-3 * scale
    # 1-CTA and 2-CTA kernels agree
    g1 = run(1, api.F32, 1.0)
    assert float((f1 - g1).abs().max()) <= 1e-4 * float(f1.abs().max())
    del g1
    # alpha = 2 scales the accumulator exactly; the bias is added after scaling
    f2 = run(2, api.F32, 2.0)
    bias_f = bias.float()[None, :]
    assert torch.equal(f2 - bias_f, 2.0 * (f1 - bias_f)) or float(((f2 - bias_f) - 2.0 * (f1 - bias_f)).abs().max()) <= 1e-6


def test_run_host_and_runtime_run(torch_cuda):
    """The host-buffer entry point and Runtime.run (float arrays in, float array out; the
    reference's own test feeds all-ones 128x128x128 and checks only the length)."""
    m = n = k = 128
    c = api.runtime_run(api.KernelSpec(name="gemm_blackwell", elem=api.BF16, tile=(128, 256, 64), stages=4), m, n, k,
                        np.ones(m * k, np.float32), np.ones(n * k, np.float32))
    assert c.shape == (m * n,) and np.all(c == 128.0)
    p = O.make_bf16_problem(300, 512, 192, seed=9, with_bias=True)
    out = np.empty((300, 512), dtype=np.uint16)
    plan_for(2, api.BF16, 1).run_host(p["a_bits"], p["b_bits"], out, p["bias_bits"], 1.0, 300, 512, 192)
    e = O.rel_error(O.bf16_bits_to_f32(out), O.gemm_f32(p["a"], p["b"], 1.0, p["bias"]))
    assert e["max_rel"] <= TOL_BF16_OUT


def test_run_host_pipelined_chunks(torch_cuda):
    """A host-buffer call above 32 MiB goes up in row chunks that are multiplied and sent back while the next
    chunk arrives; the result must be the one-shot result (here with a ragged last chunk of 96 rows and page-locked buffers)."""
    t = torch_cuda
    m, n, k = 2400, 1024, 4608                      # 35 MB of A + B + C: chunks of 256 rows
    p = O.make_bf16_problem(m, n, k, seed=17, with_bias=True)
    pin = lambda bits: t.from_numpy(bits.view(np.int16)).pin_memory()
    a, b, bias = pin(p["a_bits"]), pin(p["b_bits"]), pin(p["bias_bits"])
    out = t.empty((m, n), dtype=t.int16).pin_memory()
    plan = plan_for(2, api.BF16, 1)
    for _ in range(2):                               # twice: the streams and events are reused
        out.zero_()
        plan.run_host(a.numpy(), b.numpy(), out.numpy(), bias.numpy(), 1.0, m, n, k)
        got = O.bf16_bits_to_f32(out.numpy().view(np.uint16))
        e = O.rel_error(got, O.gemm_f32(p["a"], p["b"], 1.0, p["bias"]))
        assert e["max_rel"] <= TOL_BF16_OUT
    # bit-identical to the device-pointer call on the same operands
    c = t.empty((m, n), dtype=t.bfloat16, device="cuda")
    plan.run(a.cuda().view(t.bfloat16), b.cuda().view(t.bfloat16), c, bias.cuda().view(t.bfloat16), 1.0, m, n, k,
             stream=t.cuda.current_stream().cuda_stream)
    assert plan.status() == 0
    assert t.equal(c.view(t.int16).cpu(), out)


def test_argument_errors(torch_cuda):
    plan = plan_for(2, api.BF16, 0)
    t = torch_cuda.zeros(16, 16, dtype=torch_cuda.bfloat16, device="cuda")
    with pytest.raises(api.TesseraeError, match="positive"):
        plan.run(t, t, t, None, 1.0, 0, 16, 16)
    with pytest.raises(api.TesseraeError, match="multiple of 16 bytes"):
        plan.run(t, t, t, None, 1.0, 16, 16, 12)
    with pytest.raises(api.TesseraeError, match="bias"):
        plan_for(2, api.BF16, 1).run(t, t, t, None, 1.0, 16, 16, 16)


@pytest.mark.parametrize("cg", [1, 2])
@pytest.mark.parametrize("tile_k,swizzle_b", [(32, 2), (16, 1)])
def test_operand_swizzle_derived_from_tile_k(torch_cuda, cg, tile_k, swizzle_b):
    """tile.k = 32 / 16 bf16 elements gives 64 / 32-byte rows of K per stage, for which Swizzle.smem_selector
    (lib/core/swizzle.ml:46-56) derives Swizzle<2,4,3> / Swizzle<1,4,3>: the tensor maps, the shared-memory
    descriptors and the number of MMAs per stage all follow that B, and the product must not change."""
    spec = api.KernelSpec(name=f"gemm_bf16_cg{cg}_k{tile_k}", elem=api.BF16, tile=(128, 256, tile_k), cta_group=cg,
                          out_elem=api.F32)
    assert api.lower(spec).swizzle_b == swizzle_b
    plan = api.GemmPlan(spec)
    for i, (m, n, k) in enumerate([(256, 256, 64), (512, 512, 512), (200, 264, 72), (129, 8, 520)]):
        p = O.make_bf16_problem(m, n, k, seed=900 + i)
        got = run_gpu(torch_cuda, plan, p, m, n, k, api.F32)
        e = O.rel_error(got, O.gemm_f32(p["a"], p["b"]))
        assert e["max_rel"] <= TOL_F32_OUT, (cg, tile_k, m, n, k, e)
    plan.close()


GROUPED_SHAPES = [(512, 512, 512), (200, 264, 72), (1, 8, 8), (129, 8, 520), (1000, 1016, 1032), (64, 4096, 128),
                  (4096, 64, 128), (256, 256, 64)]


def test_grouped_launch_equals_one_launch_per_problem(torch_cuda):
    """One grouped launch over ragged problems: bit-equal to the ungrouped kernel run problem by problem (the
    tile arithmetic is the same code), and within the bf16 tolerance of the oracle."""
    torch = torch_cuda
    spec = dict(elem=api.BF16, tile=(128, 256, 64), cta_group=2, out_elem=api.BF16, has_bias=1)
    grouped = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_bf16_grouped", grouped=1, **spec))
    single = plan_for(2, api.BF16, 1)
    st = torch.cuda.current_stream().cuda_stream
    keep, problems, refs, singles = [], [], [], []
    for i, (m, n, k) in enumerate(GROUPED_SHAPES):
        p = O.make_bf16_problem(m, n, k, seed=700 + i, with_bias=True)
        a, b, bias = to_dev(torch, p["a_bits"]), to_dev(torch, p["b_bits"]), to_dev(torch, p["bias_bits"])
        c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        c1 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        single.run(a, b, c1, bias, 0.75, m, n, k, stream=st)
        keep.append((a, b, bias, c))
        problems.append((a, b, c, bias, m, n, k))
        refs.append(O.gemm_f32(p["a"], p["b"], 0.75, p["bias"]))
        singles.append(c1)
    nbytes = api.grouped_workspace_bytes(len(problems))
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    for _ in range(2):                                   # the second call reuses the plan's pinned table
        grouped.run_grouped(problems, ws, nbytes, alpha=0.75, stream=st)
    torch.cuda.synchronize()
    assert grouped.status() == 0 and single.status() == 0
    for (m, n, k), (_, _, _, c), c1, ref in zip(GROUPED_SHAPES, keep, singles, refs):
        assert torch.equal(c.view(torch.int16), c1.view(torch.int16)), (m, n, k)
        assert O.rel_error(c.float().cpu().numpy(), ref)["max_rel"] <= TOL_BF16_OUT, (m, n, k)


def test_grouped_argument_errors(torch_cuda):
    torch = torch_cuda
    grouped = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_bf16_grouped", elem=api.BF16, tile=(128, 256, 64), cta_group=2,
                                          out_elem=api.BF16, has_bias=1, grouped=1))
    a = torch.zeros(128, 64, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(128, 128, dtype=torch.bfloat16, device="cuda")
    bias = torch.zeros(128, dtype=torch.bfloat16, device="cuda")
    ws = torch.empty(4096, dtype=torch.uint8, device="cuda")
    with pytest.raises(api.TesseraeError, match="workspace too small"):
        grouped.run_grouped([(a, a, c, bias, 128, 128, 64)], ws, 448)
    with pytest.raises(api.TesseraeError, match="problem 1: .*bias"):
        grouped.run_grouped([(a, a, c, bias, 128, 128, 64), (a, a, c, None, 128, 128, 64)], ws, 4096)
    with pytest.raises(api.TesseraeError, match="use tesserae_gemm_run_grouped"):
        grouped.run(a, a, c, bias, 1.0, 128, 128, 64)
    with pytest.raises(api.TesseraeError, match="grouped = 1"):
        plan_for(2, api.BF16, 1).run_grouped([(a, a, c, bias, 128, 128, 64)], ws, 4096)


@pytest.mark.parametrize("cg", [1, 2])
def test_launch_control_scheduler_equals_static_order(torch_cuda, cg):
    """Tile order by cluster launch control (one cluster per tile; running clusters cancel and take over the ones that
    have not started): every tile is computed exactly once, by the same arithmetic, so the result is bit-equal to the
    static order's.  Shapes from one tile to many times the number of resident clusters."""
    torch = torch_cuda
    dyn = api.GemmPlan(api.KernelSpec(name=f"gemm_bf16_cg{cg}_bf16_b1_clc", elem=api.BF16, tile=(128, 256, 64), cta_group=cg,
                                      out_elem=api.BF16, has_bias=1, tuning="CLC=1"))
    static = plan_for(cg, api.BF16, 1)
    for i, (m, n, k) in enumerate([(128, 256, 64), (200, 264, 72), (1000, 1016, 1032), (4096, 4096, 256), (8192, 2048, 512),
                                   (8192, 8192, 128)]):
        p = O.make_bf16_problem(m, n, k, seed=800 + i, with_bias=True)
        got = run_gpu(torch, dyn, p, m, n, k, api.BF16, alpha=0.75)
        want = run_gpu(torch, static, p, m, n, k, api.BF16, alpha=0.75)
        assert not np.isnan(got).any(), (cg, m, n, k)
        assert np.array_equal(got, want), (cg, m, n, k)
    for _ in range(3):                                    # back-to-back launches: every launch has its own grid to cancel from
        got = run_gpu(torch, dyn, p, m, n, k, api.BF16, alpha=0.75)
        assert np.array_equal(got, want)


def test_grouped_launch_with_launch_control(torch_cuda):
    """Grouped problems of very different K under the dynamic order: bit-equal to one static launch per problem."""
    torch = torch_cuda
    spec = dict(elem=api.BF16, tile=(128, 256, 64), cta_group=2, out_elem=api.BF16, has_bias=1)
    grouped = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_bf16_grouped_clc", grouped=1, tuning="CLC=1", **spec))
    single = plan_for(2, api.BF16, 1)
    st = torch.cuda.current_stream().cuda_stream
    shapes = [(512, 1024, 64), (512, 1024, 4096), (300, 520, 256), (1024, 2048, 1024), (256, 256, 8192), (2048, 1024, 128)] * 3
    keep, problems, singles = [], [], []
    for i, (m, n, k) in enumerate(shapes):
        p = O.make_bf16_problem(m, n, k, seed=850 + i, with_bias=True)
        a, b, bias = to_dev(torch, p["a_bits"]), to_dev(torch, p["b_bits"]), to_dev(torch, p["bias_bits"])
        c = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        c1 = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device="cuda")
        single.run(a, b, c1, bias, 1.0, m, n, k, stream=st)
        keep.append((a, b, bias, c)); problems.append((a, b, c, bias, m, n, k)); singles.append(c1)
    nbytes = api.grouped_workspace_bytes(len(problems))
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    grouped.run_grouped(problems, ws, nbytes, stream=st)
    torch.cuda.synchronize()
    assert grouped.status() == 0 and single.status() == 0
    for (m, n, k), (_, _, _, c), c1 in zip(shapes, keep, singles):
        assert torch.equal(c.view(torch.int16), c1.view(torch.int16)), (m, n, k)


@pytest.mark.parametrize("out_elem,bias,tuning", [(api.BF16, 1, ""), (api.F32, 0, ""), (api.BF16, 1, "CLC=1")])
def test_wide_tile_equals_narrow(torch_cuda, out_elem, bias, tuning):
    """The 512-column tile of the CTA-pair kernel (two MMA groups of 256 columns into one accumulator that fills tensor
    memory, handed back to the MMA issuer group by group): every output element is the same sum over K in the same
    order as with the 256-column tile, so the results are bit-equal."""
    torch = torch_cuda
    wide = api.GemmPlan(api.KernelSpec(name=f"gemm_bf16_cg2_n512_o{out_elem}_b{bias}{tuning.replace('=', '')}", elem=api.BF16,
                                       tile=(128, 512, 64), cta_group=2, out_elem=out_elem, has_bias=bias, tuning=tuning))
    narrow = plan_for(2, out_elem, bias)
    for i, (m, n, k) in enumerate([(256, 512, 64), (200, 264, 72), (1000, 1016, 1032), (300, 1544, 520), (4096, 4096, 256),
                                   (8192, 1024, 128)]):
        p = O.make_bf16_problem(m, n, k, seed=870 + i, with_bias=bool(bias))
        got = run_gpu(torch, wide, p, m, n, k, out_elem, alpha=0.75)
        want = run_gpu(torch, narrow, p, m, n, k, out_elem, alpha=0.75)
        assert not np.isnan(got).any(), (m, n, k)
        assert np.array_equal(got, want), (m, n, k)
    if out_elem == api.BF16 and not tuning:
        # config 2 at full size (8192^3, N(0,1) * 0.05 drawn on the GPU): the wide tile against the narrow one, bit for bit
        from helpers import fullsize as F
        m = n = k = 8192
        a = F.draw(torch, (m, k), 1, "normal", 0.05).to(torch.bfloat16)
        b = F.draw(torch, (n, k), 1001, "normal", 0.05).to(torch.bfloat16)
        bias_d = (F.draw(torch, (n,), 2001, "normal", 0.1)).to(torch.bfloat16)
        st = torch.cuda.current_stream().cuda_stream
        c_wide = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        c_narrow = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        wide.run(a, b, c_wide, bias_d, 1.0, m, n, k, stream=st)
        narrow.run(a, b, c_narrow, bias_d, 1.0, m, n, k, stream=st)
        torch.cuda.synchronize()
        assert wide.status() == 0 and narrow.status() == 0
        assert torch.equal(c_wide.view(torch.int16), c_narrow.view(torch.int16))
