"""The Tirix IR behind the C ABI: lowering, text round trip, the verifier's messages (the reference's,
lib/tirix/tirix_verify.ml:9-183, exercised the way lib/tirix/tests/test_tirix_verify.ml:54-216 does: a valid
program, then one defect at a time), and emission through the IR with the text properties the reference's emit
tests hold (lib/tirix/tests/test_tirix_emit.ml:243-321).  CPU only."""
import pytest

from tesserae_b200 import api

BF16 = dict(name="gemm_blackwell", arch=api.SM100, elem=api.BF16, tile=(128, 256, 64), out_elem=api.BF16, has_bias=1)
SPECS = {
    "bf16": api.KernelSpec(**BF16),
    "bf16_cg1": api.KernelSpec(name="gemm_cg1", elem=api.BF16, tile=(128, 256, 64), cta_group=1),
    "scatter_add": api.KernelSpec(name="gemm_scatter_add", elem=api.BF16, tile=(128, 256, 64), out_elem=api.F32, scatter=2),
    "fp8_block": api.KernelSpec(name="gemm_fp8blk", elem=api.F8E4M3, tile=(128, 256, 128), out_elem=api.BF16, scale_mode=api.SCALE_FP8_BLOCK),
    "nvfp4": api.KernelSpec(name="gemm_nvfp4", elem=api.F4E2M1, tile=(128, 256, 256), out_elem=api.BF16, scale_mode=api.SCALE_NVFP4),
    "grouped": api.KernelSpec(name="gemm_grouped", elem=api.BF16, tile=(128, 256, 64), out_elem=api.BF16, has_bias=1, grouped=1),
    "clc": api.KernelSpec(name="gemm_clc", elem=api.BF16, tile=(128, 256, 64), out_elem=api.BF16, has_bias=1, tuning="CLC=1"),
    "fp8_tail": api.KernelSpec(name="gemm_fp8blk_tail", elem=api.F8E4M3, tile=(128, 256, 128), out_elem=api.BF16,
                               scale_mode=api.SCALE_FP8_BLOCK, tuning="TAIL_SPLITS=8"),
}


@pytest.mark.parametrize("which", sorted(SPECS))
def test_lowered_programs_verify_round_trip_and_emit(which):
    spec = SPECS[which]
    prog = api.Tirix.lower(spec)
    assert prog.verify() == []
    text = prog.text()
    again = api.Tirix.parse(text)
    assert again.text() == text and again.verify() == []
    out = again.emit()
    direct = api.backend_emit(spec)
    # the IR listing leads the source; below it the source is the backend's own for that spec
    assert out.full_source.startswith("// Tirix program this source was emitted from:")
    assert out.full_source.endswith(direct.full_source)
    assert out.kernel_func == direct.kernel_func and out.producer_body == direct.producer_body


def test_structure_follows_the_spec():
    bf16, fp8, nv = (api.Tirix.lower(SPECS[k]) for k in ("bf16", "fp8_block", "nvfp4"))
    for p in (bf16, fp8, nv):
        assert p.count_ops("TmemAlloc") == 1 and p.count_ops("TmemDealloc") == 1 and p.count_ops("Mma") == 1
        assert p.count_ops("MbarWaitParity") >= 4                   # every wait is a bounded wait with a status bit
    assert bf16.count_ops("ScaleFma") == 0 and fp8.count_ops("ScaleFma") == 1
    assert nv.count_ops("TmemStore") == 1 and bf16.count_ops("TmemStore") == 0
    text = bf16.text()
    for needle in ("family=2", "cluster=2,1,1", "warpgroup Producer", "warpgroup Consumer", "warpgroup Epilogue",
                   "tensor smem_A space=1", "sub=TmaPair tensors=A,smem_A var=full_bar", "sub=Sm100Tcgen05.f16",
                   "op MbarArriveExpect var=full_bar expr=65536", "sub=TmaStore tensors=smem_C,C", "param A_tmap tma"):
        assert needle in text, needle
    assert "sub=TmaLoad tensors=A,smem_A" in api.Tirix.lower(SPECS["bf16_cg1"]).text()
    assert "sub=TmaReduceAdd tensors=smem_C,C" in api.Tirix.lower(SPECS["scatter_add"]).text()
    # smem ring as Desc_to_tirix states it: (depth, rows, K extent), here with the stage count the smem fit gives
    assert "tensor smem_A space=1 elem=1 swizzle=3 shape=6,128,128 stride=16384,128,1" in text


def test_scheduler_role_of_the_launch_control_variant():
    """Cluster's Scheduler role (lib/pipeline/cluster.mli:17-21): present only when the spec asks for launch control;
    then the kernel has a seventh warp, the ring's barriers, and every role takes its next tile from the ring."""
    static, clc = api.Tirix.lower(SPECS["bf16"]), api.Tirix.lower(SPECS["clc"])
    assert "warpgroup Scheduler" not in static.text() and static.count_ops("ClcTryCancel") == 0
    text = clc.text()
    assert "warpgroup Scheduler" in text
    assert clc.count_ops("ClcTryCancel") == 1 and clc.count_ops("ClcQuery") == 1 and clc.count_ops("StoreCluster") == 2
    assert "op MbarInit var=sched_empty_bar imm=11" in text          # 2 producer lanes + the MMA warp + 8 epilogue warps of the pair
    assert text.count("sub=TIMEOUT_SCHED") == 5                      # producer, MMA issuer, epilogue, and the scheduler's two waits
    src = api.backend_emit(SPECS["clc"])
    assert "#define TS_CLC 1" in src.includes and "clusterlaunchcontrol.try_cancel" in src.full_source
    assert "block=224 threads" in src.full_source and "block=192 threads" in api.backend_emit(SPECS["bf16"]).full_source
    with pytest.raises(api.TesseraeError, match="launch-control scheduler is for the unscaled kernels"):
        api.backend_emit(api.KernelSpec(name="k", elem=api.F8E4M3, tile=(128, 256, 128), scale_mode=api.SCALE_FP8_BLOCK, tuning="CLC=1"))


def _edit(text: str, old: str, new: str) -> api.Tirix:
    assert old in text, old
    return api.Tirix.parse(text.replace(old, new, 1))


def test_verifier_messages():
    text = api.Tirix.lower(SPECS["bf16"]).text()
    cases = [
        ("let num_tiles = num_m * num_n", "let num_tiles = num_m * n_cols", "undefined variable 'n_cols'"),
        ("assign it = it + 1", "assign warp_id = it + 1", "assigning to immutable variable 'warp_id'"),
        ("assign it = it + 1", "assign nowhere = it + 1", "undefined variable 'nowhere' in SAssign"),
        ("for kb = 0 ; num_k_blocks ; 1", "for kb = 0 ; num_k_blocks ; 0", "SFor 'kb' has zero step"),
        ("sub=TmaPair tensors=A,smem_A var=full_bar", "sub=TmaPair tensors=Q,smem_A var=full_bar", "unknown tensor 'Q' in copy.src"),
        ("sub=TmaPair tensors=A,smem_A var=full_bar", "sub=TmaPair tensors=A,smem_A var=no_bar", "undefined mbar 'no_bar' in copy"),
        ("warpgroup Producer", "warpgroup Scheduler", "SWarpGroup role not in cluster warp_roles"),
        ("op MbarWaitParity sub=TIMEOUT_EMPTY var=empty_bar", "op MbarWaitParity var=empty_bar", "names no status bit"),
        ("op TmemDealloc", "op CtaSync\n      # op TmemDealloc", "tensor memory is allocated 1 time(s) and freed 0"),
    ]
    for old, new, want in cases:
        errs = _edit(text, old, new).verify()
        assert any(want in e for e in errs), (want, errs)
    # several defects at once are all reported (test_tirix_verify.ml:200-216)
    two = text.replace("for kb = 0 ; num_k_blocks ; 1", "for kb = 0 ; num_k_blocks ; 0").replace("tensors=A,smem_A", "tensors=Q,smem_A")
    assert len(api.Tirix.parse(two).verify()) >= 3
    # a pipeline statement with no stages (test_tirix_verify.ml:117-133)
    piped = text.replace("body\n", "body\n  pipeline stages=0\n  mainloop\n  epilogue\n  end\n", 1)
    assert any("SPipeline has invalid stage count 0" in e for e in api.Tirix.parse(piped).verify())
    ok = text.replace("body\n", "body\n  pipeline stages=4\n    empty\n  mainloop\n  epilogue\n  end\n", 1)
    assert api.Tirix.parse(ok).verify() == []


def test_emission_is_driven_by_the_ir():
    text = api.Tirix.lower(SPECS["bf16"]).text()
    # a program that does not verify is not emitted
    with pytest.raises(api.TesseraeError, match="does not verify"):
        _edit(text, "for kb = 0 ; num_k_blocks ; 1", "for kb = 0 ; num_k_blocks ; 0").emit()
    # a program that verifies but states another structure than the mainloop its origin selects is refused
    with pytest.raises(api.TesseraeError, match="not that of the mainloop"):
        _edit(text, "sub=TmaPair tensors=B,smem_B var=full_bar", "sub=TmaPair tensors=A,smem_B var=full_bar").emit()
    # editing the origin selects another kernel: the structure must then be that kernel's
    with pytest.raises(api.TesseraeError, match="not that of the mainloop"):
        _edit(text, "cta_group=0", "cta_group=1").emit()
    fp32 = api.Tirix.lower(api.KernelSpec(**dict(BF16, out_elem=api.F32))).emit()
    assert "#define TS_OUT_F32 1" in fp32.includes
    # malformed text names its line
    with pytest.raises(ValueError, match="line 3"):
        api.Tirix.parse("tirix k\nbody\n  frobnicate\nend\n")


def test_emitted_text_properties():
    out = api.Tirix.lower(SPECS["bf16"]).emit()
    for needle in ("__global__", "gemm_blackwell", "warp_id", "tcgen05.alloc", "__cluster_dims__", "cudaLaunchKernelEx"):
        assert needle in out.full_source, needle
    assert "kStages" in out.shared_storage and "smem_a" in out.full_source and "mbar" in out.full_source
