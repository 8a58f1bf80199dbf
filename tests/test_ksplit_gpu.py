"""K-split path on one GPU: fp32 partial products per K slice, then the sum + bf16 cast pass.
The reduce/cast pass is integer-exact against the oracle (same fp32 additions in the same order,
round to nearest even); the GEMM part carries the bf16 tolerance 1e-2."""
import numpy as np
import pytest

from oracle import gemm_oracle as O
from tesserae_b200 import api

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU tests need a CUDA device; there is no CPU path to fall back to")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="module")
def plan_f32():
    return api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_b0", elem=api.BF16, tile=(128, 256, 64), cta_group=2,
                                       out_elem=api.F32))


def test_reduce_cast_bit_exact(torch_cuda):
    t = torch_cuda
    for n, parts, alpha in [(8, 1, 1.0), (1000, 3, 1.0), (4096 * 33 + 5, 4, 0.5), (1 << 22, 8, 1.0)]:
        stride = (n + 3) // 4 * 4 + 8
        host = O.normal((parts, stride), seed=n % 97, std=3.0)
        dev = t.from_numpy(host).cuda()
        out = t.zeros(n, dtype=t.bfloat16, device="cuda")
        api.reduce_cast_bf16(dev, parts, stride, out, n, alpha=alpha, stream=t.cuda.current_stream().cuda_stream)
        acc = host[0, :n].copy()
        for p in range(1, parts):
            acc = (acc + host[p, :n]).astype(np.float32)
        want = O.f32_to_bf16_bits((np.float32(alpha) * acc).astype(np.float32))
        got = out.view(t.int16).cpu().numpy().view(np.uint16)
        assert np.array_equal(got, want), (n, parts)


@pytest.mark.parametrize("k_splits", [1, 2, 4])
def test_ksplit_matches_oracle(torch_cuda, plan_f32, k_splits):
    t = torch_cuda
    m, n, k = 512, 768, 2048
    p = O.make_bf16_problem(m, n, k, seed=60 + k_splits, scale=0.5)
    a = t.from_numpy(p["a_bits"].view(np.int16)).view(t.bfloat16).cuda()
    b = t.from_numpy(p["b_bits"].view(np.int16)).view(t.bfloat16).cuda()
    nbytes = api.ksplit_scratch_bytes(m, n, k_splits)
    assert nbytes == m * n * 4 * k_splits
    scratch = t.empty(nbytes, dtype=t.uint8, device="cuda")
    c = t.full((m, n), float("nan"), dtype=t.bfloat16, device="cuda")
    plan_f32.ksplit_run(a, b, c, scratch, nbytes, m, n, k, k_splits, stream=t.cuda.current_stream().cuda_stream)
    assert plan_f32.status() == 0
    e = O.rel_error(c.float().cpu().numpy(), O.gemm_f32(p["a"], p["b"]))
    assert e["max_rel"] <= 1e-2, e
    # the slices are exactly the products over their K ranges
    parts = scratch.view(t.float32).reshape(k_splits, m, n).cpu().numpy()
    ks = k // k_splits
    for s in range(k_splits):
        ref = O.gemm_f32(p["a"][:, s * ks:(s + 1) * ks], p["b"][:, s * ks:(s + 1) * ks])
        assert O.rel_error(parts[s], ref)["max_rel"] <= 1e-3


def test_ksplit_argument_errors(torch_cuda, plan_f32):
    t = torch_cuda
    x = t.zeros(256, 256, dtype=t.bfloat16, device="cuda")
    s = t.zeros(256 * 256 * 4, dtype=t.uint8, device="cuda")
    with pytest.raises(api.TesseraeError, match="scratch too small"):
        plan_f32.ksplit_run(x, x, x, s, 100, 256, 256, 256, 1)
    with pytest.raises(api.TesseraeError, match="multiple of k_splits"):
        plan_f32.ksplit_run(x, x, x, s, s.numel(), 256, 256, 192, 2)
    bf16_plan = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_bf16_b0", elem=api.BF16, tile=(128, 256, 64), cta_group=2,
                                            out_elem=api.BF16))
    with pytest.raises(api.TesseraeError, match="fp32 output"):
        bf16_plan.ksplit_run(x, x, x, s, s.numel(), 256, 256, 256, 1)


def test_config5_shard_properties(torch_cuda, plan_f32):
    """One GPU's share of the K-split GEMM M=N=8192, K=131072 over 8 GPUs (K slice 16384, U[-0.5,0.5) seed 4):
    sampled entries of the fp32 partial in fp64, and additivity: the partial over the slice equals the sum of
    the partials over its two halves."""
    t = torch_cuda
    m = n = 8192
    k = 131072 // 8
    p = O.make_bf16_problem(m, n, k, seed=4, dist="uniform", scale=0.5)
    a = t.from_numpy(p["a_bits"].view(np.int16)).view(t.bfloat16).cuda()
    b = t.from_numpy(p["b_bits"].view(np.int16)).view(t.bfloat16).cuda()
    nbytes = api.ksplit_scratch_bytes(m, n, 2)
    scratch = t.empty(nbytes, dtype=t.uint8, device="cuda")
    s = t.cuda.current_stream().cuda_stream
    plan_f32.ksplit_partials(a, b, scratch, nbytes, m, n, k, 1, stream=s)
    assert plan_f32.status() == 0
    whole = scratch.view(t.float32)[: m * n].reshape(m, n).clone()
    rows, cols = [0, 255, 4096, 8191], list(range(0, n, 211)) + [n - 1]
    want = O.gemm_f64_entries(p["a"], p["b"], rows, cols)
    got = whole[rows][:, cols].cpu().numpy()
    rms = float(np.sqrt(np.mean(want ** 2)))
    # fp32 accumulation over 16384 products: absolute error ~2e-4 on entries of magnitude ~10, measured
    # against the floored magnitude rms/128
    assert np.max(np.abs(got - want) / np.maximum(np.abs(want), rms / 128)) <= 5e-3
    plan_f32.ksplit_partials(a, b, scratch, nbytes, m, n, k, 2, stream=s)
    halves = scratch.view(t.float32).reshape(2, m, n)
    assert float((halves[0] + halves[1] - whole).abs().max()) <= 1e-3 * float(whole.abs().max())


@pytest.mark.parametrize("tile_n", [256, 512])
def test_scatter_epilogue_matches_plain_partial(torch_cuda, plan_f32, tile_n):
    """The row-scattered epilogue (the GEMM -> reduce-scatter fusion) with all destinations on this GPU: owner g's
    buffer must hold exactly rows [g*R, (g+1)*R) of the ordinary fp32 partial, bit for bit (both tile widths)."""
    t = torch_cuda
    m, n, k, owners = 1024 + 256, 768, 1024, 4          # the last owner gets a short slice
    rpo = 384
    p = O.make_bf16_problem(m, n, k, seed=71, scale=0.5)
    a = t.from_numpy(p["a_bits"].view(np.int16)).view(t.bfloat16).cuda()
    b = t.from_numpy(p["b_bits"].view(np.int16)).view(t.bfloat16).cuda()
    s = t.cuda.current_stream().cuda_stream
    plain = t.empty((m, n), dtype=t.float32, device="cuda")
    plan_f32.ksplit_partials(a, b, plain, plain.numel() * 4, m, n, k, 1, stream=s)
    scat = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_scatter" + ("" if tile_n == 256 else f"_n{tile_n}"), elem=api.BF16,
                                       tile=(128, tile_n, 64), cta_group=2, out_elem=api.F32, scatter=1))
    dst = [t.full((rpo, n), float("nan"), dtype=t.float32, device="cuda") for _ in range(owners)]
    scat.ksplit_scatter(a, b, [d.data_ptr() for d in dst], rpo, m, n, k, stream=s, start_owner=2)   # a rotated tile order
    assert scat.status() == 0 and plan_f32.status() == 0
    for g in range(owners):
        rows = min(rpo, m - g * rpo)
        assert t.equal(dst[g][:rows], plain[g * rpo:g * rpo + rows]), g
        assert t.isnan(dst[g][rows:]).all()              # nothing written past the owner's slice
    with pytest.raises(api.TesseraeError, match="scatter"):
        scat.run(a, b, plain, None, 1.0, m, n, k)
    with pytest.raises(api.TesseraeError, match="multiple of 128"):
        scat.ksplit_scatter(a, b, [d.data_ptr() for d in dst], 100, m, n, k)
    scat.close()


def test_config5_full_size(torch_cuda, plan_f32):
    """The whole K-split GEMM of config 5 on one GPU: M=N=8192, K=131072 (U[-0.5,0.5), seed 4, drawn on the GPU),
    four K slices of 32768 into fp32 partials, then sum + bf16 cast.  Sampled entries of the bf16 output in fp64
    (tolerance 1e-2), the row-sum identity sum_n C[m,n] = a[m,:] . sum_n b[n,:] on the summed fp32 partials, and
    the bf16 output must be exactly the rounded sum of the partials."""
    from helpers import fullsize as F
    t = torch_cuda
    m = n = 8192
    k, splits = 131072, 4
    a = F.draw(t, (m, k), 4, "uniform", 0.5).to(t.bfloat16)
    b = F.draw(t, (n, k), 1004, "uniform", 0.5).to(t.bfloat16)
    nbytes = api.ksplit_scratch_bytes(m, n, splits)
    scratch = t.empty(nbytes, dtype=t.uint8, device="cuda")
    c = t.empty((m, n), dtype=t.bfloat16, device="cuda")
    plan_f32.ksplit_run(a, b, c, scratch, nbytes, m, n, k, splits, stream=t.cuda.current_stream().cuda_stream)
    assert plan_f32.status() == 0
    rows, cols = [0, 255, 4096, 8191], list(range(0, n, 211)) + [n - 1]
    want = a[rows].double() @ b[cols].double().T                      # fp64 on the device: 4 x 40 x 131072 products
    got = c[rows][:, cols].double()
    rms = float(want.pow(2).mean().sqrt())
    rel = ((got - want).abs() / want.abs().clamp_min(rms / 128)).max()
    assert float(rel) <= 1e-2, float(rel)
    parts = scratch.view(t.float32).reshape(splits, m, n)
    total = parts[0].double()
    for p_ in range(1, splits):
        total += parts[p_].double()
    # the cast pass sums the partials in slice order in fp32 and rounds once
    fp32_sum = ((parts[0] + parts[1]) + parts[2]) + parts[3]
    assert t.equal(c, fp32_sum.to(t.bfloat16))
    colsum = b.double().sum(dim=0)                                    # host-independent fp64 reduction of B
    want_rowsum = (a.double() @ colsum).cpu().numpy()
    got_rowsum = total.sum(dim=1).cpu().numpy()
    assert np.max(np.abs(got_rowsum - want_rowsum)) <= 1e-3 * float(np.sqrt(np.mean(want_rowsum ** 2)))


@pytest.mark.parametrize("tile_n", [256, 512])
def test_scatter_add_epilogue_matches_plain_partial(torch_cuda, plan_f32, tile_n):
    """The adding form of the row-scattered epilogue (TMA reduce at the destination) with all owners on this GPU:
    into zeroed buffers it must leave exactly the rows of the ordinary fp32 partial (0 + x = x), and a second launch
    on top of the first exactly twice that (x + x is exact in fp32)."""
    t = torch_cuda
    m, n, k, owners = 1024 + 256, 768, 1024, 4
    rpo = 384
    p = O.make_bf16_problem(m, n, k, seed=72, scale=0.5)
    a = t.from_numpy(p["a_bits"].view(np.int16)).view(t.bfloat16).cuda()
    b = t.from_numpy(p["b_bits"].view(np.int16)).view(t.bfloat16).cuda()
    s = t.cuda.current_stream().cuda_stream
    plain = t.empty((m, n), dtype=t.float32, device="cuda")
    plan_f32.ksplit_partials(a, b, plain, plain.numel() * 4, m, n, k, 1, stream=s)
    radd = api.GemmPlan(api.KernelSpec(name="gemm_bf16_cg2_f32_scatter_add" + ("" if tile_n == 256 else f"_n{tile_n}"), elem=api.BF16,
                                       tile=(128, tile_n, 64), cta_group=2, out_elem=api.F32, scatter=2))
    dst = [t.zeros((rpo, n), dtype=t.float32, device="cuda") for _ in range(owners)]
    for times in (1, 2):
        radd.ksplit_scatter(a, b, [d.data_ptr() for d in dst], rpo, m, n, k, stream=s)
        assert radd.status() == 0
        for g in range(owners):
            rows = min(rpo, m - g * rpo)
            assert t.equal(dst[g][:rows], plain[g * rpo:g * rpo + rows] * times), (g, times)
            assert (dst[g][rows:] == 0).all()              # nothing added past the owner's slice
    radd.close()


def test_cast_clear(torch_cuda):
    """tesserae_cast_clear_bf16: the cast of the adding epilogue's buffer, which leaves the buffer zeroed; same
    rounding as tesserae_reduce_cast_bf16 of one partial, ragged length included."""
    t = torch_cuda
    for n in (8 * 1024 + 5, 3, 1 << 20, (1 << 24) + 7):        # the last one takes several passes of the whole grid
        acc = t.randn(n + 3, device="cuda")[:n].contiguous() if n % 4 else t.randn(n, device="cuda")
        want = t.empty(n, dtype=t.bfloat16, device="cuda")
        api.reduce_cast_bf16(acc, 1, 0, want, n, alpha=0.5, stream=t.cuda.current_stream().cuda_stream)
        got = t.full((n,), float("nan"), dtype=t.bfloat16, device="cuda")
        api.cast_clear_bf16(acc, got, n, alpha=0.5, stream=t.cuda.current_stream().cuda_stream)
        assert t.equal(got.view(t.int16), want.view(t.int16)) and not acc.any()
