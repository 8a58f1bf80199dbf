"""The product's integer descriptor model, called through the C ABI, against the reference's
known-answer values and against the oracle on seeded random layouts (bit-exact)."""
import random

import pytest

from conftest import flat, to_modes
from oracle import layout_oracle as L
from tesserae_b200 import api
from tesserae_b200 import _native as N

ELEM = {"f16": api.F16, "bf16": api.BF16, "f32": api.F32, "s8": api.S8, "s32": api.S32}


def fl(pair):
    return flat(pair[0]), flat(pair[1])


def test_goldens_layout(goldens):
    for g in goldens["layout_cosize"]:
        assert api.layout_cosize(*fl(g["layout"])) == g["expect"], g["src"]
    for g in goldens["layout_idx"]:
        assert api.layout_idx(flat(g["layout"][1]), flat(g["coord"])) == g["expect"], g["src"]
    for g in goldens["compose"]:
        shape, stride = api.layout_compose(fl(g["outer"]), fl(g["inner"]))
        for coord, want in g["idx"]:
            assert api.layout_idx(stride, flat(coord)) == want, g["src"]
    for g in goldens["compose_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            api.layout_compose(fl(g["outer"]), fl(g["inner"]))
    for g in goldens["tile"]:
        s, d = api.layout_tile(*fl(g["layout"]), flat(g["tile"]))
        for coord, want in g["idx"]:
            assert api.layout_idx(d, flat(coord)) == want, g["src"]
    for g in goldens["tile_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            api.layout_tile(*fl(g["layout"]), flat(g["tile"]))


def test_goldens_algebra(goldens):
    for name, fn in (("sort", api.layout_sort), ("coalesce", api.layout_coalesce)):
        for g in goldens[name]:
            assert fn(*fl(g["layout"])) == (g["shapes"], g["strides"]), g["src"]
    for g in goldens["is_admissible"]:
        assert api.layout_is_admissible(*fl(g["layout"]), g["m"]) == g["expect"], g["src"]
    for g in goldens["complement"]:
        assert api.layout_complement(*fl(g["layout"]), g["m"]) == (g["shapes"], g["strides"]), g["src"]
    for g in goldens["complement_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            api.layout_complement(*fl(g["layout"]), g["m"])
    for g in goldens["flat_divide"]:
        assert api.layout_flat_divide(*fl(g["layout"]), g["divisor"]) == (g["shapes"], g["strides"]), g["src"]
    for g in goldens["flat_divide_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            api.layout_flat_divide(*fl(g["layout"]), g["divisor"])
    for g in goldens["logical_divide"]:
        s, d = api.layout_logical_divide(*fl(g["layout"]), flat(g["tile"][0]))
        if "shapes" in g:
            assert (s, d) == (g["shapes"], g["strides"])
        for coord, want in g["idx"]:
            assert api.layout_idx(d, flat(coord)) == want, g["src"]
    for g in goldens["logical_divide_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            api.layout_logical_divide(*fl(g["layout"]), flat(g["tile"][0]))


def test_goldens_swizzle_pipeline_tmem(goldens):
    lib = N.lib()
    for g in goldens["swizzle_apply"]:
        for x, want in g["cases"]:
            assert api.swizzle_apply(*g["sw"], x) == want, g["src"]
    for g in goldens["swizzle_self_inverse"]:
        for x in range(g["upto"] + 1):
            assert api.swizzle_apply(*g["sw"], api.swizzle_apply(*g["sw"], x)) == x
    with pytest.raises(ValueError, match=goldens["swizzle_misc"]["make_error"]["expect"]):
        api.swizzle_apply(*goldens["swizzle_misc"]["make_error"]["args"], 0)
    for g in goldens["smem_selector"]:
        assert list(api.swizzle_smem_selector(ELEM[g["elem"]], g["tile_m"], g["tile_k"])) == g["expect"], g["src"]
    for g in goldens["elemtype"]:
        assert lib.tesserae_elem_byte_width(ELEM[g["elem"]]) == g["bytes"]
        assert lib.tesserae_elem_vec_width(ELEM[g["elem"]]) == g["vec"]
    p = goldens["pipeline"]
    assert lib.tesserae_pipeline_smem_bytes(p["make"]["depth"], p["make"]["tile_bytes"]) == p["make"]["smem_bytes"]
    for e in p["errors"]:
        assert lib.tesserae_pipeline_smem_bytes(e["depth"], e["tile_bytes"]) == -1 and N.last_error() == e["expect"]
    for it, d, want in p["stage_of"]:
        assert lib.tesserae_pipeline_stage_of(it, d) == want
    for it, d, want in p["phase_of"]:
        assert lib.tesserae_pipeline_phase_of(it, d) == want
    for st, want in p["smem_offset_of"]:
        assert lib.tesserae_pipeline_smem_offset_of(p["make"]["tile_bytes"], st) == want
    for st, bm, bk, eb, want in p["b_smem_offset_of"]:
        assert lib.tesserae_pipeline_b_smem_offset_of(p["make"]["tile_bytes"], st, bm, bk, eb) == want
    t = goldens["tmem"]
    for r, c, want in t["address"]:
        assert lib.tesserae_tmem_address(r, c) == want
    for w, want in t["warp_row_offset"]:
        assert lib.tesserae_tmem_warp_row_offset(w) == want
    for cols, want in t["num_loads_per_warp"]:
        assert lib.tesserae_tmem_num_loads_per_warp(cols) == want
    for e in t["errors"]:
        assert lib.tesserae_tmem_validate(e["cta_group"], e["cols"], e["rows"]) == -1 and N.last_error() == e["expect"]
    for g in goldens["smem_desc_encode"]:
        want = g["expect"] if "expect" in g else (g["expect_shift"][0] << g["expect_shift"][1])
        assert lib.tesserae_smem_desc_encode(*g["args"]) & ((1 << 63) - 1) == want & ((1 << 63) - 1), g["src"]
    t = goldens["tile_io"]
    assert lib.tesserae_tile_io_bytes_a(api.BF16, 128, 64) == t["bytes_a"]["expect"]
    assert lib.tesserae_tile_io_bytes_b(api.BF16, 256, 64, 2) == t["bytes_b_2sm"]["expect"]
    assert lib.tesserae_tile_io_bytes_b(api.BF16, 256, 64, 1) == t["bytes_b_1sm"]["expect"]
    assert lib.tesserae_tile_io_expect_tx(api.BF16, api.TMA_PAIR, 128, 256, 64) == t["expect_tx_2sm"]["expect"]
    assert lib.tesserae_tile_io_expect_tx(api.BF16, 1, 128, 256, 64) == t["expect_tx_1sm"]["expect"]
    pr = goldens["predicate"]
    import ctypes as C
    for g in pr["count_valid"]:
        n = len(g["shape"])
        assert lib.tesserae_predicate_count_valid((C.c_int64 * n)(*g["shape"]), (C.c_int64 * n)(*g["bounds"]), n) == g["expect"]
    for g in pr["residue"]:
        n = len(g["shape"])
        out = (C.c_int64 * n)()
        assert lib.tesserae_predicate_residue((C.c_int64 * n)(*g["shape"]), (C.c_int64 * n)(*g["bounds"]), n, out) == 0
        assert list(out) == g["expect"]


def test_goldens_lower(goldens):
    g = goldens["kernel_desc_blackwell"]
    h = g["hand_evaluated"]
    d = api.lower(api.KernelSpec(name="gemm_blackwell", arch=api.SM100, elem=api.BF16, tile=(128, 256, 64), stages=4))
    lib = N.lib()
    assert lib.tesserae_kernel_desc_validate(d) == 0
    assert d.family == 2 and d.num_warps == g["num_warps"] and d.strategy == api.TMA_PAIR
    assert (d.cluster_x, d.cluster_y, d.cluster_z) == (2, 1, 1)
    assert list(d.warp_roles)[:6] == [api.ROLE_PRODUCER, api.ROLE_CONSUMER, api.ROLE_EPILOGUE, api.ROLE_EPILOGUE,
                                      api.ROLE_EPILOGUE, api.ROLE_SCHEDULER]
    assert [d.swizzle_b, d.swizzle_m, d.swizzle_s] == h["swizzle"]
    assert d.tile_bytes == h["tile_bytes"] and d.smem_bytes == h["smem_bytes"] <= g["smem_le"]
    assert d.pipeline_depth == h["depth"] and d.sm_count == h["sm_count"]
    assert lib.tesserae_kernel_desc_arithmetic_intensity(d) == h["ai"]
    assert list(d.pred_a_bounds) == h["pred_a"] and list(d.pred_b_bounds) == h["pred_b"] and list(d.pred_c_bounds) == h["pred_c"]
    assert (d.tmem_cta_group, d.tmem_rows, d.tmem_cols, d.tmem_double_buf) == (2, 128, 512, 1)
    assert (d.atom_m, d.atom_n, d.atom_k, d.atom_threads) == (128, 128, 16, 128)
    import ctypes as C
    gx, gy, th = C.c_int(), C.c_int(), C.c_int()
    assert lib.tesserae_kernel_desc_grid(d, 8192, 8192, gx, gy, th) == 0
    assert [gx.value, gy.value] == h["grid_8192"] and th.value == h["block"]
    with pytest.raises(api.LowerError) as e:
        api.lower(api.KernelSpec(name="k", arch=api.SM100, elem=api.F32, tile=(128, 256, 64)))
    assert e.value.kind == "UnsupportedElem" and "arch=SM100 elem=F32" in str(e.value)
    # matches the oracle's descriptor field by field
    o = L.lower_sm100("gemm_blackwell", "bf16", 128, 256, 64)
    assert d.copy_vec == o["copy_vec"] and d.copy_bulk_bytes == o["copy_bulk_bytes"]
    assert (d.m, d.n, d.k) == (128 * 32, 256 * 32, 64 * 32)


def _rand_layout(rng, n):
    shape = [rng.choice([1, 2, 3, 4, 6, 8]) for _ in range(n)]
    stride = [rng.choice([0, 1, 2, 3, 4, 8, 12, 16, 32]) for _ in range(n)]
    return shape, stride


def _same(fn_api, fn_oracle, *args):
    """Both raise (same message) or both return the same flat layout."""
    try:
        want = fn_oracle()
    except ValueError as e:
        with pytest.raises(ValueError, match=str(e).replace("(", r"\(").replace(")", r"\)")):
            fn_api()
        return
    except (ZeroDivisionError, IndexError):
        return   # the reference would die with an OCaml exception here; not a defined result
    got = fn_api()
    assert got == (L.flatten(want.shape), L.flatten(want.stride)), args


def test_random_layouts_match_oracle():
    rng = random.Random(1234)
    for _ in range(400):
        n = rng.randint(1, 4)
        shape, stride = _rand_layout(rng, n)
        lo = L.Layout(tuple(shape), tuple(stride))
        assert api.layout_cosize(shape, stride) == L.cosize(lo)
        coord = [rng.randrange(s) for s in shape]
        assert api.layout_idx(stride, coord) == L.idx(lo, tuple(coord))
        _same(lambda: api.layout_sort(shape, stride), lambda: L.sort(lo), shape, stride)
        _same(lambda: api.layout_coalesce(shape, stride), lambda: L.coalesce(lo), shape, stride)
        m = rng.choice([8, 16, 24, 64, 96])
        try:
            adm = L.is_admissible(lo, m)
        except ZeroDivisionError:
            continue
        assert api.layout_is_admissible(shape, stride, m) == adm
        _same(lambda: api.layout_complement(shape, stride, m), lambda: L.complement(lo, m), shape, stride, m)
        div = rng.choice([1, 2, 3, 4])
        _same(lambda: api.layout_flat_divide(shape, stride, div), lambda: L.flat_divide(lo, div), shape, stride, div)
        tile = [rng.choice([1, 2, 3]) for _ in range(n)]
        _same(lambda: api.layout_tile(shape, stride, tile), lambda: L.tile(lo, tuple(tile)), shape, stride, tile)
        ishape, istride = _rand_layout(rng, n)
        li = L.Layout(tuple(ishape), tuple(istride))
        try:
            want = L.compose(lo, li)
        except ValueError as e:
            with pytest.raises(ValueError):
                api.layout_compose((shape, stride), (ishape, istride))
            continue
        except ZeroDivisionError:
            continue
        assert api.layout_compose((shape, stride), (ishape, istride))[1] == L.flatten(want.stride)


def test_random_swizzle_matches_oracle():
    rng = random.Random(7)
    for _ in range(2000):
        b, m, s = rng.randint(0, 5), rng.randint(0, 7), rng.randint(0, 5)
        x = rng.randrange(1 << 20)
        assert api.swizzle_apply(b, m, s, x) == L.swizzle_apply((b, m, s), x)


def test_swizzle_apply_to_layout_matches_oracle():
    """Swizzle.apply_to_layout: leaf-wise on the strides, nested in the oracle, flattened in the product."""
    rng = random.Random(11)
    lay = L.Layout((2, (3, 4)), (1, (2, 6)))
    assert L.flatten(L.swizzle_apply_to_layout((0, 4, 3), lay).stride) == [1, 2, 6]          # Swizzle<0,...> is the identity
    assert api.swizzle_apply_to_strides(3, 4, 3, [1023, 128, 1]) == [911, 144, 1]               # 1023 -> 911 (test_swizzle.ml:43-46)
    for _ in range(300):
        b, m, s = rng.randint(0, 4), rng.randint(0, 6), rng.randint(0, 4)
        strides = (rng.randrange(1 << 14), (rng.randrange(1 << 14), rng.randrange(1 << 14)))
        want = L.swizzle_apply_to_layout((b, m, s), L.Layout((2, (2, 2)), strides))
        assert want.shape == (2, (2, 2))
        assert api.swizzle_apply_to_strides(b, m, s, L.flatten(strides)) == L.flatten(want.stride)
    with pytest.raises(api.TesseraeError, match="non-negative"):
        api.swizzle_apply_to_strides(-1, 4, 3, [1])


def test_hardware_descriptors():
    """The descriptors the kernels build on the device, restated on the host: field positions
    of the sm_100 shared-memory matrix descriptor and instruction descriptor."""
    lib = N.lib()
    d = lib.tesserae_umma_smem_desc(0x12340, 3)
    assert d & 0x3FFF == 0x1234 and (d >> 16) & 0x3FFF == 1 and (d >> 32) & 0x3FFF == 64
    assert (d >> 46) & 3 == 1 and (d >> 61) & 7 == 2
    i = lib.tesserae_umma_instr_desc(api.BF16, 256, 256)
    assert (i >> 4) & 3 == 1 and (i >> 7) & 7 == 1 and (i >> 10) & 7 == 1 and (i >> 17) & 63 == 32 and (i >> 24) & 31 == 16
    assert (i >> 15) & 3 == 0   # both operands K-major


def _size(pair):
    n = 1
    for x in flat(pair[0]):
        n *= x
    return n


def test_goldens_memspace_and_atoms(goldens):
    g = goldens["memspace"]
    for name, want in g["names"].items():
        assert api.memspace_name(name) == want
    for src, dst, want in g["can_transfer"]:
        assert api.memspace_can_transfer(src, dst) is want, (src, dst)
    g = goldens["mma_atom"]
    for name, want in g["shape"]:
        a = api.mma_atom(name)
        assert [a.m, a.n, a.k] == want
    for name, want in g["thread_count"]:
        assert api.mma_atom_thread_count(api.mma_atom(name)) == want
    for name, want in g["is_wgmma"]:
        assert api.mma_atom_is_wgmma(api.mma_atom(name)) is want
    for name, am, bm, want in g["emit_cpp"]:
        assert api.mma_atom_emit_cpp(api.mma_atom(name, am, bm)) == want
    g = goldens["copy_atom"]
    for kind, elem, want in g["bulk_bytes"]:
        assert api.copy_atom(kind, elem).bulk_bytes == want
    for kind, elem, want in g["vec_width"]:
        assert api.copy_atom(kind, elem).vec_width == want
    for key, fn in (("is_async", api.copy_atom_is_async), ("is_tma", api.copy_atom_is_tma),
                    ("requires_mbar", api.copy_atom_requires_mbar)):
        for kind, elem, want in g[key]:
            assert fn(api.copy_atom(kind, elem)) is want, (key, kind)
    for kind, elem, parts in g["emit_cpp"]:
        assert api.copy_atom_emit_cpp(api.copy_atom(kind, elem)) == "".join(parts)


def test_goldens_tiled_atoms_and_tile_op(goldens):
    g = goldens["tiled_mma"]
    for c in g["cases"]:
        t = api.tiled_mma(api.mma_atom(c["atom"]), _size(c["thread_layout"]), _size(c["warp_layout"]), *c["tiler_mn"])
        assert (t.thread_count, t.warp_count) == (c["thread_count"], c["warp_count"])
        assert [t.tile_m, t.tile_n, t.tile_k] == c["tile_mnk"] and t.partition_c == c["partition_c_size"]
    e = g["error"]
    with pytest.raises(ValueError, match=e["expect"]):
        api.tiled_mma(api.mma_atom(e["atom"]), _size(e["thread_layout"]), _size(e["warp_layout"]), *e["tiler_mn"])
    g = goldens["tiled_copy"]
    for c in g["cases"]:
        t = api.tiled_copy(api.copy_atom(c["kind"], c["elem"]), _size(c["thread_layout"]), _size(c["val_layout"]))
        assert (t.thread_count, t.elements_per_thread, t.tile_size) == (c["thread_count"], c["elements_per_thread"], c["tile_size"])
        assert bool(t.is_tma) is c["is_tma"] and bool(t.requires_mbar) is c["requires_mbar"]
    p = g["partition"]
    shape, _ = api.tiled_copy_partition(_size(p["thread_layout"]), *fl(p["layout"]))
    assert shape == p["size"]
    e = g["error"]
    with pytest.raises(ValueError, match=e["expect"]):
        api.tiled_copy(api.copy_atom(e["kind"], e["elem"]), _size(e["thread_layout"]), _size(e["val_layout"]))

    g = goldens["tile_op"]

    def make(o):
        tmem = (o["tmem"]["cta_group"], o["tmem"]["num_cols"], o["tmem"]["num_rows"]) if o["tmem"] else None
        return api.tile_op(api.mma_atom(o["atom"]), _size(o["thread_layout"]), _size(o["warp_layout"]), *o["tiler_mn"],
                           o["accum"], tmem, o["double_buf"])
    ops = {k: make(v) for k, v in g["ops"].items()}
    for k, want in g["is_tmem"].items():
        assert api.tile_op_is_tmem(ops[k]) is want
    for k, want in g["is_wgmma"].items():
        assert api.tile_op_is_wgmma(ops[k]) is want
    for k, want in g["accum_elems_per_thread"].items():
        assert api.tile_op_accum_elems_per_thread(ops[k]) == want
    decl = api.tile_op_emit(ops["sm80"], "accum_decl", "acc")
    assert all(x in decl for x in g["accum_decl"]["sm80_contains"])
    assert api.tile_op_emit(ops["sm100"], "accum_decl", "acc") == g["accum_decl"]["sm100"]
    for k, want in g["emit_mma_contains"].items():
        assert want in api.tile_op_emit(ops[k], "mma", "a_desc", "b_desc", 0)
    assert api.tile_op_emit(ops["sm80"], "commit", "mbar", "", 0) == g["emit_commit"]["sm80_mask0"]
    assert all(x in api.tile_op_emit(ops["sm100"], "commit", "mbar", "", 3) for x in g["emit_commit"]["sm100_mask3_contains"])
    assert api.tile_op_emit(ops["sm80"], "tmem_alloc", "tmem_addr") == g["tmem_alloc"]["sm80"]
    assert g["tmem_alloc"]["sm100_contains"] in api.tile_op_emit(ops["sm100"], "tmem_alloc", "tmem_addr")
    assert g["tmem_dealloc_contains"]["sm100"] in api.tile_op_emit(ops["sm100"], "tmem_dealloc", "taddr")
    with pytest.raises(ValueError, match="TensorMem requires a tmem descriptor"):
        api.tile_op(api.mma_atom("sm100_64x64x16_f32f16f16f32"), 128, 1, 64, 64, "TensorMem", None)


def test_atoms_product_equals_oracle_everywhere():
    """Every constructor x major pair, every copy kind x element, and the Tile_op text of both accumulator
    locations: the C++ model behind the C ABI against the independent Python restatement, string for string."""
    for name in api.MMA_ATOM_IDS:
        for am in ("RowMajor", "ColMajor"):
            for bm in ("RowMajor", "ColMajor"):
                pa, oa = api.mma_atom(name, am, bm), L.mma_atom(name, am, bm)
                assert api.mma_atom_emit_cpp(pa) == L.mma_atom_emit_cpp(oa)
                assert api.mma_atom_thread_count(pa) == L.mma_atom_thread_count(oa)
                assert [pa.m, pa.n, pa.k] == [oa["m"], oa["n"], oa["k"]]
    for kind in api.COPY_KINDS:
        for elem in api.ELEMS:
            pa, oa = api.copy_atom(kind, elem), L.copy_atom(kind, elem)
            assert (pa.vec_width, pa.bulk_bytes) == (oa["vec_width"], oa["bulk_bytes"]), (kind, elem)
            assert api.copy_atom_emit_cpp(pa) == L.copy_atom_emit_cpp(oa)
            assert api.memspace_name(["global", "shared", "register", "tensor"][pa.src_space]) == oa["src"]
    for src in api.SPACES:
        for dst in api.SPACES:
            assert api.memspace_can_transfer(src, dst) is L.memspace_can_transfer(src, dst), (src, dst)
    for name, accum, tmem in (("sm80_16x8x16_f32f16f16f32", "Registers", None), ("sm100_128x128x16_f32f16f16f32", "TensorMem", (2, 512, 128)),
                              ("sm100_64x64x32_s32s8s8s32", "TensorMem", (1, 64, 128))):
        threads = 32 if name.startswith("sm80") else 128
        po = api.tile_op(api.mma_atom(name), threads, 1, 64, 64, accum, tmem)
        otm = L.tiled_mma_make(L.mma_atom(name), L.Layout(threads, 1), L.Layout(1, 0), (64, 64))
        oo = L.tile_op_make(otm, accum, L.tmem_make(*tmem) if tmem else None)
        assert api.tile_op_emit(po, "mma", "da", "db", 1) == L.tile_op_emit_mma(oo, "da", "db", True)
        for mask in (0, 1, 3):
            assert api.tile_op_emit(po, "commit", "bar", "", mask) == L.tile_op_emit_commit(oo, "bar", mask)
        assert api.tile_op_emit(po, "accum_decl", "acc") == L.tile_op_emit_accum_decl(oo, "acc")
        assert api.tile_op_emit(po, "tmem_alloc", "slot") == L.tile_op_emit_tmem_alloc(oo, "slot")
        assert api.tile_op_emit(po, "tmem_dealloc", "addr") == L.tile_op_emit_tmem_dealloc(oo, "addr")
        assert api.tile_op_accum_elems_per_thread(po) == L.tile_op_accum_elems_per_thread(oo)
