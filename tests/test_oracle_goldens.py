"""The integer oracle (oracle/layout_oracle.py) against every known-answer value the reference's
own tests hold for these functions (tests/golden/layout_goldens.json)."""
import pytest

from conftest import to_modes
from oracle import layout_oracle as L


def lay(pair):
    return L.Layout(to_modes(pair[0]), to_modes(pair[1]))


def test_modes(goldens):
    for g in goldens["modes"]:
        m = to_modes(g["mode"])
        assert L.size(m) == g["size"] and L.depth(m) == g["depth"] and L.rank(m) == g["rank"]
        assert L.flatten(m) == g["flatten"] and L.pp_modes(m) == g["pp"]


def test_layout(goldens):
    for g in goldens["layout_cosize"]:
        assert L.cosize(lay(g["layout"])) == g["expect"], g["src"]
    for g in goldens["layout_idx"]:
        assert L.idx(lay(g["layout"]), to_modes(g["coord"])) == g["expect"], g["src"]
    for g in goldens["layout_make_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            L.Layout(to_modes(g["shape"]), to_modes(g["stride"]))


def test_compose_and_tile(goldens):
    for g in goldens["compose"]:
        c = L.compose(lay(g["outer"]), lay(g["inner"]))
        assert L.layout_size(c) == g["size"]
        for coord, want in g["idx"]:
            assert L.idx(c, to_modes(coord)) == want, g["src"]
    for g in goldens["compose_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            L.compose(lay(g["outer"]), lay(g["inner"]))
    for g in goldens["tile"]:
        t = L.tile(lay(g["layout"]), to_modes(g["tile"]))
        assert L.layout_size(t) == g["size"]
        if "cosize" in g:
            assert L.cosize(t) == g["cosize"]
        for coord, want in g["idx"]:
            assert L.idx(t, to_modes(coord)) == want, g["src"]
    for g in goldens["tile_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            L.tile(lay(g["layout"]), to_modes(g["tile"]))


def test_algebra(goldens):
    for name, fn in (("sort", L.sort), ("coalesce", L.coalesce)):
        for g in goldens[name]:
            r = fn(lay(g["layout"]))
            assert L.flatten(r.shape) == g["shapes"] and L.flatten(r.stride) == g["strides"], g["src"]
    for g in goldens["is_admissible"]:
        assert L.is_admissible(lay(g["layout"]), g["m"]) == g["expect"], g["src"]
    for g in goldens["complement"]:
        r = L.complement(lay(g["layout"]), g["m"])
        assert L.layout_size(r) == g["size"]
        assert L.flatten(r.shape) == g["shapes"] and L.flatten(r.stride) == g["strides"], g["src"]
    for g in goldens["complement_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            L.complement(lay(g["layout"]), g["m"])


def test_divide(goldens):
    for g in goldens["flat_divide"]:
        r = L.flat_divide(lay(g["layout"]), g["divisor"])
        assert L.flatten(r.shape) == g["shapes"] and L.flatten(r.stride) == g["strides"], g["src"]
    for g in goldens["flat_divide_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            L.flat_divide(lay(g["layout"]), g["divisor"])
    for g in goldens["logical_divide"]:
        r = L.logical_divide(lay(g["layout"]), lay(g["tile"]))
        assert L.layout_size(r) == g["size"]
        if "shapes" in g:
            assert L.flatten(r.shape) == g["shapes"] and L.flatten(r.stride) == g["strides"]
        if "rank" in g:
            assert L.layout_rank(r) == g["rank"]
        for coord, want in g["idx"]:
            assert L.idx(r, to_modes(coord)) == want, g["src"]
    for g in goldens["logical_divide_error"]:
        with pytest.raises(ValueError, match=g["expect"]):
            L.logical_divide(lay(g["layout"]), lay(g["tile"]))
    for g in goldens["zipped_divide"]:
        ld = L.logical_divide(lay(g["layout"]), lay(g["tile"]))
        zd = L.zipped_divide(lay(g["layout"]), lay(g["tile"]))
        assert L.layout_size(zd) == g["size"] and L.layout_rank(zd) == g["rank"]

        def indices(l):
            shapes, out = L.flatten(l.shape), []
            for k in range(L.layout_size(l)):
                rem, co = k, []
                for sh in shapes:
                    co.append(rem % sh)
                    rem //= sh
                out.append(L.idx(l, tuple(co)))
            return sorted(out)
        assert indices(ld) == indices(zd), g["src"]


def test_swizzle(goldens):
    for g in goldens["swizzle_apply"]:
        sw = L.swizzle_make(*g["sw"])
        for x, want in g["cases"]:
            assert L.swizzle_apply(sw, x) == want, g["src"]
    for g in goldens["swizzle_self_inverse"]:
        sw = L.swizzle_make(*g["sw"])
        for x in range(g["upto"] + 1):
            assert L.swizzle_apply(sw, L.swizzle_apply(sw, x)) == x
    misc = goldens["swizzle_misc"]
    with pytest.raises(ValueError, match=misc["make_error"]["expect"]):
        L.swizzle_make(*misc["make_error"]["args"])
    for sw, want in misc["mask_bits"]:
        assert L.swizzle_mask_bits(tuple(sw)) == want
    assert list(L.swizzle_compose(tuple(misc["compose"]["a"]), tuple(misc["compose"]["b"]))) == misc["compose"]["expect"]
    with pytest.raises(ValueError, match=misc["compose_error"]["expect"]):
        L.swizzle_compose(tuple(misc["compose_error"]["a"]), tuple(misc["compose_error"]["b"]))
    for g in goldens["smem_selector"]:
        assert list(L.smem_selector(g["elem"], g["tile_m"], g["tile_k"])) == g["expect"], g["src"]
    for g in goldens["elemtype"]:
        assert L.ELEM_BYTES[g["elem"]] == g["bytes"] and L.ELEM_CPP[g["elem"]] == g["cpp"]
        assert L.elem_vec_width(g["elem"]) == g["vec"]


def test_pipeline_cluster_tmem(goldens):
    p = goldens["pipeline"]
    made = L.pipeline_make(p["make"]["depth"], p["make"]["tile_bytes"])
    assert made["smem_bytes"] == p["make"]["smem_bytes"]
    for e in p["errors"]:
        with pytest.raises(ValueError, match=e["expect"]):
            L.pipeline_make(e["depth"], e["tile_bytes"])
    for it, d, want in p["stage_of"]:
        assert L.stage_of(it, d) == want
    for it, d, want in p["phase_of"]:
        assert L.phase_of(it, d) == want
    for st, want in p["smem_offset_of"]:
        assert L.smem_offset_of(made, st) == want
    for st, bm, bk, eb, want in p["b_smem_offset_of"]:
        assert L.b_smem_offset_of(made, st, bm, bk, eb) == want

    c = goldens["cluster_blackwell"]
    d = L.make_blackwell("k", 128, 256, 64, "bf16", 4096, 8192, 2048)
    cl = d["cluster"]
    assert cl["dims"][0] * cl["dims"][1] * cl["dims"][2] == c["cta_count"] and cl["num_warps"] * 32 == c["threads"]
    assert L.warps_with_role(cl, "Producer") == [c["producer"]] and L.warps_with_role(cl, "Consumer") == [c["consumer"]]
    assert L.warps_with_role(cl, "Epilogue") == c["epilogue"] and L.warps_with_role(cl, "Scheduler") == [c["scheduler"]]
    for e in c["errors"]:
        with pytest.raises(ValueError, match=e["expect"]):
            L.cluster_make(e["dims"], e["num_warps"], [tuple(r) for r in e["roles"]])

    t = goldens["tmem"]
    for r, col, want in t["address"]:
        assert L.tmem_address(r, col) == want
    for w, want in t["warp_row_offset"]:
        assert L.tmem_warp_row_offset(w) == want
    for cols, want in t["num_loads_per_warp"]:
        assert L.tmem_num_loads_per_warp(L.tmem_make(1, cols, 128)) == want
    te = t["total_elems"]
    assert L.tmem_total_elems(L.tmem_make(1, te["cols"], te["rows"])) == te["expect"] and te["expect"] * 4 == te["bytes"]
    for e in t["errors"]:
        with pytest.raises(ValueError, match=e["expect"]):
            L.tmem_make(e["cta_group"], e["cols"], e["rows"])


def test_smem_desc_predicate_tile_io(goldens):
    for g in goldens["smem_desc_encode"]:
        want = g["expect"] if "expect" in g else (g["expect_shift"][0] << g["expect_shift"][1]) & ((1 << 63) - 1)
        assert L.smem_desc_encode(*g["args"]) == want, g["src"]
    pr = goldens["predicate"]
    for g in pr["count_valid"]:
        assert L.predicate_count_valid(tuple(g["shape"]), g["bounds"]) == g["expect"]
    for g in pr["residue"]:
        assert L.predicate_residue(tuple(g["shape"]), g["bounds"]) == g["expect"]
    with pytest.raises(ValueError, match=pr["error"]["expect"]):
        L.predicate_count_valid(tuple(pr["error"]["shape"]), pr["error"]["bounds"])
    t = goldens["tile_io"]
    assert L.bytes_per_load_a("bf16", 128, 64) == t["bytes_a"]["expect"]
    assert L.bytes_per_load_b("bf16", 256, 64, 2) == t["bytes_b_2sm"]["expect"]
    assert L.bytes_per_load_b("bf16", 256, 64, 1) == t["bytes_b_1sm"]["expect"]
    assert L.expect_tx("bf16", "TmaPair", 128, 256, 64) == t["expect_tx_2sm"]["expect"]
    assert L.expect_tx("bf16", "TmaLoad", 128, 256, 64) == t["expect_tx_1sm"]["expect"]


def test_kernel_desc_and_lower(goldens):
    g = goldens["kernel_desc_blackwell"]
    d = L.lower_sm100("gemm_blackwell", "bf16", 128, 256, 64)
    h = g["hand_evaluated"]
    assert L.validate(d) is None and d["cluster"]["num_warps"] == g["num_warps"]
    assert d["pipeline"]["smem_bytes"] <= g["smem_le"] and L.is_2sm(d["cluster"]) and d["strategy"] == g["strategy"]
    assert list(d["swizzle"]) == h["swizzle"] and d["pipeline"]["tile_bytes"] == h["tile_bytes"]
    assert d["pipeline"]["smem_bytes"] == h["smem_bytes"] and d["pipeline"]["depth"] == h["depth"]
    assert L.arithmetic_intensity(d) == h["ai"] > 64.0
    assert d["pred_a_bounds"] == h["pred_a"] and d["pred_b_bounds"] == h["pred_b"] and d["pred_c_bounds"] == h["pred_c"]
    assert d["tmem"] == {"cta_group": 2, "num_cols": 512, "num_rows": 128}
    for e in goldens["lower_errors"]:
        with pytest.raises(ValueError, match=e["expect_kind"]):
            L.lower_sm100("k", e["elem"], 128, 256, 64)


def test_memspace(goldens):
    g = goldens["memspace"]
    for name, want in g["names"].items():
        assert name in L.SPACES and name == want
    for src, dst, want in g["can_transfer"]:
        assert L.memspace_can_transfer(src, dst) is want, (src, dst)
    assert not L.memspace_can_transfer("tensor", "global") and L.memspace_can_transfer("tensor", "tensor")


def test_mma_and_copy_atoms(goldens):
    g = goldens["mma_atom"]
    for name, want in g["shape"]:
        a = L.mma_atom(name)
        assert [a["m"], a["n"], a["k"]] == want
    for name, want in g["thread_count"]:
        assert L.mma_atom_thread_count(L.mma_atom(name)) == want
    for name, want in g["is_wgmma"]:
        assert L.mma_atom_is_wgmma(L.mma_atom(name)) is want
    for name, am, bm, want in g["emit_cpp"]:
        assert L.mma_atom_emit_cpp(L.mma_atom(name, am, bm)) == want
    g = goldens["copy_atom"]
    for kind, elem, want in g["bulk_bytes"]:
        assert L.copy_atom(kind, elem)["bulk_bytes"] == want
    for kind, elem, want in g["vec_width"]:
        assert L.copy_atom(kind, elem)["vec_width"] == want
    for key, fn in (("is_async", L.copy_atom_is_async), ("is_tma", L.copy_atom_is_tma), ("requires_mbar", L.copy_atom_requires_mbar)):
        for kind, elem, want in g[key]:
            assert fn(L.copy_atom(kind, elem)) is want, (key, kind)
    for kind, elem, parts in g["emit_cpp"]:
        assert L.copy_atom_emit_cpp(L.copy_atom(kind, elem)) == "".join(parts)


def _lay(x):
    return L.Layout(to_modes(x[0]), to_modes(x[1]))


def test_tiled_atoms(goldens):
    g = goldens["tiled_mma"]
    for c in g["cases"]:
        t = L.tiled_mma_make(L.mma_atom(c["atom"]), _lay(c["thread_layout"]), _lay(c["warp_layout"]), to_modes(c["tiler_mn"]))
        assert L.tiled_mma_thread_count(t) == c["thread_count"] and L.tiled_mma_warp_count(t) == c["warp_count"]
        assert list(L.tiled_mma_tile_shape_mnk(t)) == c["tile_mnk"]
        assert L.layout_size(L.tiled_mma_partition(t, "c")) == c["partition_c_size"]
    e = g["error"]
    with pytest.raises(ValueError, match=e["expect"]):
        L.tiled_mma_make(L.mma_atom(e["atom"]), _lay(e["thread_layout"]), _lay(e["warp_layout"]), to_modes(e["tiler_mn"]))
    g = goldens["tiled_copy"]
    for c in g["cases"]:
        t = L.tiled_copy_make(L.copy_atom(c["kind"], c["elem"]), _lay(c["thread_layout"]), _lay(c["val_layout"]))
        assert L.layout_size(t["thread_layout"]) == c["thread_count"]
        assert L.layout_size(t["val_layout"]) == c["elements_per_thread"]
        assert L.tiled_copy_tile_size(t) == c["tile_size"]
        assert L.copy_atom_is_tma(t["atom"]) is c["is_tma"] and L.copy_atom_requires_mbar(t["atom"]) is c["requires_mbar"]
    p = g["partition"]
    t = L.tiled_copy_make(L.copy_atom(p["kind"], p["elem"]), _lay(p["thread_layout"]), _lay(p["val_layout"]))
    assert L.layout_size(L.tiled_copy_partition(t, _lay(p["layout"]))) == p["size"]
    e = g["error"]
    with pytest.raises(ValueError, match=e["expect"]):
        L.tiled_copy_make(L.copy_atom(e["kind"], e["elem"]), _lay(e["thread_layout"]), _lay(e["val_layout"]))


def _oracle_tile_op(o):
    tm = L.tiled_mma_make(L.mma_atom(o["atom"]), _lay(o["thread_layout"]), _lay(o["warp_layout"]), to_modes(o["tiler_mn"]))
    tmem = L.tmem_make(o["tmem"]["cta_group"], o["tmem"]["num_cols"], o["tmem"]["num_rows"]) if o["tmem"] else None
    return L.tile_op_make(tm, o["accum"], tmem, o["double_buf"])


def test_tile_op(goldens):
    g = goldens["tile_op"]
    ops = {k: _oracle_tile_op(v) for k, v in g["ops"].items()}
    for k, want in g["is_tmem"].items():
        assert L.tile_op_is_tmem(ops[k]) is want
    for k, want in g["is_wgmma"].items():
        assert L.tile_op_is_wgmma(ops[k]) is want
    for k, want in g["double_buf"].items():
        assert ops[k]["double_buf"] is want
    for k, want in g["accum_elems_per_thread"].items():
        assert L.tile_op_accum_elems_per_thread(ops[k]) == want
    decl = L.tile_op_emit_accum_decl(ops["sm80"], "acc")
    assert all(x in decl for x in g["accum_decl"]["sm80_contains"]) and decl == "float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};"
    assert L.tile_op_emit_accum_decl(ops["sm100"], "acc") == g["accum_decl"]["sm100"]
    for k, want in g["emit_mma_contains"].items():
        assert want in L.tile_op_emit_mma(ops[k], "a_desc", "b_desc", False)
    assert L.tile_op_emit_commit(ops["sm80"], "mbar", 0) == g["emit_commit"]["sm80_mask0"]
    assert all(x in L.tile_op_emit_commit(ops["sm100"], "mbar", 3) for x in g["emit_commit"]["sm100_mask3_contains"])
    assert L.tile_op_emit_tmem_alloc(ops["sm80"], "tmem_addr") == g["tmem_alloc"]["sm80"]
    assert g["tmem_alloc"]["sm100_contains"] in L.tile_op_emit_tmem_alloc(ops["sm100"], "tmem_addr")
    assert g["tmem_dealloc_contains"]["sm100"] in L.tile_op_emit_tmem_dealloc(ops["sm100"], "taddr")
    with pytest.raises(ValueError, match="TensorMem requires a tmem descriptor"):
        L.tile_op_make(ops["sm80"]["tiled_mma"], "TensorMem", None)
