"""Backend text and compile path on CPU: the emitted source carries the properties the
reference's own backend tests pin (lib/backend/tests/test_backend_cute.ml:46-225), NVRTC turns
it into an sm_100a cubin without a GPU, and the cubin cache hits, survives corruption and is
keyed by content."""
import ctypes as C
import os

import pytest

from tesserae_b200 import api
from tesserae_b200 import _native as N

BLACKWELL = dict(name="gemm_blackwell", arch=api.SM100, elem=api.BF16, tile=(128, 256, 64), stages=4)


def test_emit_sections_and_text_properties():
    out = api.backend_emit(api.KernelSpec(**BLACKWELL))
    assert out.filename == "gemm_blackwell.cuh"
    src = out.full_source
    # substrings asserted by the reference's Blackwell emit tests
    for needle in ("#pragma once", "__global__", "gemm_blackwell", "warp_id", "smem_a", "smem_b", "mbar", "tmem",
                   "tcgen05", "tcgen05.ld", "alloc", "TensorMap", "cluster", "for (", "< M", "__cluster_dims__",
                   "cudaLaunchKernelEx", "TmaPair"):
        assert needle in src, needle
    assert "tcgen05.mma.cta_group::2.kind::f16" in out.helpers
    assert "expect_tx" in out.producer_body and "ts_tma_load_2d" in out.producer_body
    assert "ts_umma<" in out.consumer_body and "ts_umma_commit" in out.consumer_body
    assert "ts_tmem_ld_32x32b_x32" in out.epilogue_body and "ts_tma_store_2d" in out.epilogue_body
    assert "kStages" in out.shared_storage
    assert out.kernel_func.lstrip().startswith('extern "C" __global__')
    assert "#define TS_CTA_GROUP 2" in out.includes and "#define TS_BLOCK_N 256" in out.includes
    # every operand load is a plain per-CTA TMA load: no bulk copy carries a cluster-wide qualifier
    banned = "multi" + "cast"
    for line in src.splitlines():
        if "cp.async.bulk" in line:
            assert banned not in line, line


def test_emit_rejects_what_the_reference_rejects():
    with pytest.raises(api.TesseraeError, match="UnsupportedElem"):
        api.backend_emit(api.KernelSpec(name="k", elem=api.F32))
    with pytest.raises(api.TesseraeError, match="powers of 2"):
        api.backend_emit(api.KernelSpec(name="k", tile=(128, 192, 64)))
    with pytest.raises(api.TesseraeError, match="UnsupportedArch"):
        api.backend_emit(api.KernelSpec(name="k", arch=api.SM90))
    with pytest.raises(api.TesseraeError, match="32, 64 or 128 bytes"):
        api.backend_emit(api.KernelSpec(name="k", tile=(128, 256, 128)))          # 256 bytes of K per row
    with pytest.raises(api.TesseraeError, match="exactly 128 bytes"):
        api.backend_emit(api.KernelSpec(name="k", elem=api.F8E4M3, tile=(128, 256, 64), scale_mode=api.SCALE_FP8_BLOCK))


def test_grouped_kernel_takes_a_problem_table():
    plain = api.backend_emit(api.KernelSpec(name="k", tile=(128, 256, 64), cta_group=2, out_elem=api.BF16))
    grouped = api.backend_emit(api.KernelSpec(name="k", tile=(128, 256, 64), cta_group=2, out_elem=api.BF16, grouped=1))
    assert "#define TS_GROUPED 1" in grouped.includes and "TS_GROUPED" not in plain.includes
    with pytest.raises(api.TesseraeError, match="grouped launches are for the unscaled kernels"):
        api.backend_emit(api.KernelSpec(name="k", tile=(128, 256, 64), cta_group=2, scatter=1, grouped=1))
    with pytest.raises(api.TesseraeError, match="grouped launches are for the unscaled kernels"):
        api.backend_emit(api.KernelSpec(name="k", elem=api.F8E4M3, tile=(128, 256, 128), scale_mode=api.SCALE_FP8_BLOCK, grouped=1))
    assert api.grouped_workspace_bytes(3) == 4 * 448 and api.grouped_workspace_bytes(0) == 0


def test_wide_tile_is_for_unscaled_cta_pairs():
    wide = api.backend_emit(api.KernelSpec(name="k", tile=(128, 512, 64), cta_group=2, out_elem=api.BF16))
    assert "#define TS_BLOCK_N 512" in wide.includes and "#define TS_STAGES 4" in wide.includes
    with pytest.raises(api.TesseraeError, match="512 for an unscaled CTA-pair kernel"):
        api.backend_emit(api.KernelSpec(name="k", tile=(128, 512, 64), cta_group=1))
    with pytest.raises(api.TesseraeError, match="512 for an unscaled CTA-pair kernel"):
        api.backend_emit(api.KernelSpec(name="k", elem=api.F8E4M3, tile=(128, 512, 128), scale_mode=api.SCALE_FP8_BLOCK))


def test_operand_swizzle_follows_the_tile():
    """Swizzle.smem_selector (lib/core/swizzle.ml:46-56) decides the operand tiles' swizzle from tile.k; the
    emitted kernel is specialised on that B, it is not a constant of the backend."""
    for tile_k, b in ((64, 3), (32, 2), (16, 1)):
        spec = api.KernelSpec(name=f"sw{b}", elem=api.BF16, tile=(128, 256, tile_k))
        assert api.lower(spec).swizzle_b == b
        out = api.backend_emit(spec)
        assert f"#define TS_SWIZZLE_B {b}" in out.includes
        assert f"swizzle=Swizzle<{b},4,3>" in out.includes
    # and the host-side descriptor builder changes with it: stride byte offset = 8 rows, layout type 2 / 4 / 6
    lib = N.lib()
    for b, sbo, layout in ((3, 1024, 2), (2, 512, 4), (1, 256, 6)):
        d = lib.tesserae_umma_smem_desc(0x4000, b)
        assert (d >> 32) & 0x3FFF == sbo >> 4 and (d >> 61) & 7 == layout and d & 0x3FFF == 0x4000 >> 4


def test_tuning_is_part_of_the_spec():
    base = api.KernelSpec(name="t0", elem=api.BF16, tile=(128, 256, 64))
    tuned = api.KernelSpec(name="t0", elem=api.BF16, tile=(128, 256, 64), tuning="GROUP_M=16; STORE_BUFS=3")
    a, b = api.backend_emit(base).includes, api.backend_emit(tuned).includes
    assert "raster group height: chosen per launch" in a and "#define TS_STORE_BUFS 2" in a
    assert "raster group height: 16 M-tiles" in b and "#define TS_STORE_BUFS 3" in b
    with pytest.raises(api.TesseraeError, match="unknown tuning name 'NOPE'"):
        api.backend_emit(api.KernelSpec(name="t1", tuning="NOPE=1"))
    with pytest.raises(api.TesseraeError, match="out of range: GROUP_M=0"):
        api.backend_emit(api.KernelSpec(name="t1", tuning="GROUP_M=0"))
    with pytest.raises(api.TesseraeError, match="malformed tuning entry"):
        api.backend_emit(api.KernelSpec(name="t1", tuning="GROUP_M"))


def test_no_environment_variable_changes_the_kernel(monkeypatch):
    spec = api.KernelSpec(name="envfree", elem=api.F8E4M3, tile=(128, 256, 128), scale_mode=api.SCALE_FP8_BLOCK,
                          out_elem=api.BF16)
    before = api.backend_emit(spec).full_source
    for k, v in (("TESSERAE_GROUP_M", "4"), ("TESSERAE_FP8_SPLIT", "0"), ("TESSERAE_FP8_PROMO_WARPS", "16"),
                 ("TESSERAE_STORE_BUFS", "4"), ("TESSERAE_TRACE", "1")):
        monkeypatch.setenv(k, v)
    assert api.backend_emit(spec).full_source == before


def test_compile_to_source_and_cubin_with_cache(tmp_path, monkeypatch):
    spec = api.KernelSpec(name="cache_probe_kernel", elem=api.BF16, tile=(128, 128, 64), cta_group=1, out_elem=api.BF16)
    src = api.compile_to_source(spec)
    assert src.kernel_name == "cache_probe_kernel" and not src.cubin and "cache_probe_kernel" in src.source
    first = api.compile_to_cubin(spec)
    assert first.cubin[:4] == b"\x7fELF" and first.cubin_size == len(first.cubin)
    second = api.compile_to_cubin(spec)
    assert second.cache_hit and second.cubin == first.cubin
    # corrupt the entry: it must be detected, recompiled and repaired
    cache_dir = N.lib().tesserae_cache_dir().decode()
    newest = max((os.path.join(cache_dir, f) for f in os.listdir(cache_dir)), key=os.path.getmtime)
    if first.cache_hit:   # entry predates this run; find it by content instead
        for f in os.listdir(cache_dir):
            p = os.path.join(cache_dir, f)
            if open(p, "rb").read()[40:] == first.cubin:
                newest = p
    blob = bytearray(open(newest, "rb").read())
    assert bytes(blob[:8]) == b"TSCUBIN1"
    blob[len(blob) // 2] ^= 0xFF
    open(newest, "wb").write(bytes(blob))
    third = api.compile_to_cubin(spec)
    assert not third.cache_hit and third.cubin == first.cubin
    assert api.compile_to_cubin(spec).cache_hit


def test_nvrtc_plain_c_api():
    """create / compile / get_ptx / get_log / destroy, as lib/runtime/tests/test_nvrtc_stub.c does."""
    lib = N.lib()
    kernel = b'extern "C" __global__ void trivial_kernel(float* out) { out[threadIdx.x] = 1.0f; }'
    p = lib.tesserae_nvrtc_create(kernel, b"trivial.cu")
    assert lib.tesserae_nvrtc_is_valid(p) == 1
    assert lib.tesserae_nvrtc_get_source(p) == kernel and lib.tesserae_nvrtc_get_name(p) == b"trivial.cu"
    assert not lib.tesserae_nvrtc_get_ptx(p)          # NULL before compile
    assert not lib.tesserae_nvrtc_get_log(p)
    opts = (C.c_char_p * 1)(b"--gpu-architecture=compute_100a")
    assert lib.tesserae_nvrtc_compile(p, opts, 1) == 0
    ptx = N.take_string(lib.tesserae_nvrtc_get_ptx(p))
    assert "trivial_kernel" in ptx and ".target sm_100a" in ptx
    assert N.take_string(lib.tesserae_nvrtc_get_log(p)) is not None
    opts = (C.c_char_p * 1)(b"--gpu-architecture=sm_100a")
    assert lib.tesserae_nvrtc_compile(p, opts, 1) == 0
    img, size = C.c_void_p(), C.c_size_t()
    assert lib.tesserae_nvrtc_get_cubin(p, C.byref(img), C.byref(size)) == 0 and C.string_at(img, 4) == b"\x7fELF"
    lib.tesserae_nvrtc_destroy(p)
    assert lib.tesserae_nvrtc_is_valid(p) == 0
    lib.tesserae_nvrtc_destroy(p)                      # idempotent
    bad = lib.tesserae_nvrtc_create(b"this is not CUDA", b"bad.cu")
    assert lib.tesserae_nvrtc_compile(bad, None, 0) != 0
    assert "error" in N.take_string(lib.tesserae_nvrtc_get_log(bad))
    assert not lib.tesserae_nvrtc_get_ptx(bad)
    lib.tesserae_nvrtc_destroy(bad)
