"""CPU restatement of tesserae's integer descriptor functions.  TEST INFRASTRUCTURE ONLY:
imported by tests/ (and smoke), never by the product.

Each function follows the cited reference file line by line in plain Python, keeping the
nested shape/stride trees the reference uses (a mode is an int or a tuple of modes, as
Modes.t in lib/core/modes.ml:3-5), so it is independent of the product's flattened C++ model
(tesserae_b200/csrc/spec/tesserae_spec.hpp).  It is pinned by the reference's own
known-answer tests, transcribed in tests/golden/layout_goldens.json with the test file and
line of each value.  Where the reference raises, these raise ValueError with the same message.
"""
from __future__ import annotations

from functools import reduce

# --------------------------------------------------------------------------- Modes (lib/core/modes.ml:7-38)
def size(m) -> int:
    return m if isinstance(m, int) else reduce(lambda a, x: a * size(x), m, 1)


def depth(m) -> int:
    return 0 if isinstance(m, int) else 1 + max([depth(x) for x in m], default=0)


def rank(m) -> int:
    return 1 if isinstance(m, int) else len(m)


def flatten(m) -> list:
    return [m] if isinstance(m, int) else [y for x in m for y in flatten(x)]


def compatible(shape, stride) -> bool:
    if isinstance(shape, int) and isinstance(stride, int):
        return True
    if isinstance(shape, tuple) and isinstance(stride, tuple):
        return len(shape) == len(stride) and all(compatible(a, b) for a, b in zip(shape, stride))
    return False


def pp_modes(m) -> str:
    return str(m) if isinstance(m, int) else "(" + ", ".join(pp_modes(x) for x in m) + ")"


# --------------------------------------------------------------------------- Layout (lib/core/layout.ml:8-38)
class Layout:
    def __init__(self, shape, stride):
        if not compatible(shape, stride):
            raise ValueError("incompatible shape and stride")
        self.shape, self.stride = shape, stride

    def __repr__(self):
        return f"{pp_modes(self.shape)}:{pp_modes(self.stride)}"


def layout_rank(l: Layout) -> int:
    return rank(l.shape)


def layout_size(l: Layout) -> int:
    return size(l.shape)


def cosize(l: Layout) -> int:
    return sum((s - 1) * d for s, d in zip(flatten(l.shape), flatten(l.stride))) + 1


def idx(l: Layout, coord) -> int:
    st, co = flatten(l.stride), flatten(coord)
    if len(st) != len(co):
        raise ValueError("length mismatch in map2_exn")
    return sum(c * s for c, s in zip(co, st))


# --------------------------------------------------------------------------- Compose (lib/core/compose.ml:3-47)
def compose(outer: Layout, inner: Layout) -> Layout:
    if cosize(inner) > layout_size(outer):
        raise ValueError("inner cosize exceeds outer size")
    inner_shapes, outer_strides = flatten(inner.shape), flatten(outer.stride)

    def apply_outer(s: int) -> int:
        digits, rem = [], s
        for sh in inner_shapes:
            digits.append(rem % sh)
            rem //= sh
        if len(digits) != len(outer_strides):
            raise ValueError("length mismatch in fold2_exn")
        return sum(d * st for d, st in zip(digits, outer_strides))

    def new_stride(m):
        return apply_outer(m) if isinstance(m, int) else tuple(new_stride(x) for x in m)

    return Layout(inner.shape, new_stride(inner.stride))


def tile(layout: Layout, tile_shape) -> Layout:
    ls, lst, ts = flatten(layout.shape), flatten(layout.stride), flatten(tile_shape)
    if not (len(ls) == len(lst) == len(ts)):
        raise ValueError("Layout.tile: structural mismatch")
    in_s, out_s, in_st, out_st = [], [], [], []
    for l_s, l_st, t_s in zip(ls, lst, ts):
        if t_s == 0 or l_s % t_s != 0:
            raise ValueError("tile shape does not divide layout shape")
        in_s.append(t_s); out_s.append(l_s // t_s); in_st.append(l_st); out_st.append(l_st * t_s)
    return Layout((tuple(in_s), tuple(out_s)), (tuple(in_st), tuple(out_st)))


# --------------------------------------------------------------------------- Algebra (lib/core/algebra.ml:6-135)
def sort(l: Layout) -> Layout:
    pairs = sorted(zip(flatten(l.shape), flatten(l.stride)), key=lambda p: p[1])   # stable, by stride only
    return Layout(tuple(p[0] for p in pairs), tuple(p[1] for p in pairs))


def coalesce(l: Layout) -> Layout:
    def walk(ss, st):
        if ss and st and ss[0] == 1:
            return walk(ss[1:], st[1:])
        if len(ss) >= 2 and len(st) >= 2 and st[1] == ss[0] * st[0]:
            return walk([ss[0] * ss[1]] + ss[2:], [st[0]] + st[2:])
        if ss and st:
            ns, nd = walk(ss[1:], st[1:])
            return [ss[0]] + ns, [st[0]] + nd
        return ss, st

    s, d = walk(flatten(l.shape), flatten(l.stride))
    return Layout(tuple(s), tuple(d))


def is_admissible(l: Layout, m: int) -> bool:
    shapes, strides = flatten(l.shape), flatten(l.stride)
    if strides != sorted(strides):
        return False

    def check(ss, ds):
        if len(ss) >= 2 and len(ds) >= 2:
            if ds[1] % (ss[0] * ds[0]) == 0:
                return check(ss[1:], ds[1:])
            return False
        if len(ss) == 1 and len(ds) == 1:
            return m % (ss[0] * ds[0]) == 0
        return not ss and not ds

    return check(shapes, strides)


def complement(l: Layout, m: int) -> Layout:
    if m <= 0 or not is_admissible(l, m):
        raise ValueError("layout is not admissible for complementation")
    ss, ds = flatten(l.shape), flatten(l.stride)
    comp_s, comp_d, last = [], [], 1
    for n_i, d_i in zip(ss, ds):
        comp_s.append(d_i // last); comp_d.append(last)
        last = n_i * d_i
    comp_s.append(m // last); comp_d.append(last)
    return Layout(tuple(comp_s), tuple(comp_d))


def flat_divide(layout: Layout, divisor: int) -> Layout:
    flat = coalesce(layout)
    d0 = flatten(flat.stride)[0]
    if layout_size(flat) % divisor != 0:
        raise ValueError("divisor does not divide layout size")
    return Layout((divisor, layout_size(flat) // divisor), (d0, divisor * d0))


def logical_divide(layout: Layout, tile_layout: Layout) -> Layout:
    ls, ts = flatten(layout.shape), flatten(tile_layout.shape)
    if len(ls) != len(ts):
        raise ValueError("length mismatch in for_all2_exn")
    if not all(a % b == 0 for a, b in zip(ls, ts)):
        raise ValueError("tile does not divide layout")
    return tile(layout, tile_layout.shape)


def zipped_divide(layout: Layout, tile_layout: Layout) -> Layout:
    ld = logical_divide(layout, tile_layout)
    (within_s, across_s), (within_d, across_d) = ld.shape, ld.stride
    return Layout(tuple((a, b) for a, b in zip(within_s, across_s)),
                  tuple((a, b) for a, b in zip(within_d, across_d)))


# --------------------------------------------------------------------------- Swizzle (lib/core/swizzle.ml:9-62)
def swizzle_make(b: int, m: int, s: int):
    if b < 0 or m < 0 or s < 0:
        raise ValueError("swizzle parameters must be non-negative")
    return (b, m, s)


def swizzle_apply(sw, offset: int) -> int:
    b, m, s = sw
    mask = ((1 << b) - 1) << (m + max(0, s))
    return offset ^ ((offset & mask) >> s)


def swizzle_apply_to_layout(sw, layout):
    """lib/core/swizzle.ml:36-43: every stride leaf goes through the swizzle; the shape is kept."""
    def walk(m):
        return swizzle_apply(sw, m) if isinstance(m, int) else tuple(walk(x) for x in m)
    return Layout(layout.shape, walk(layout.stride))


def swizzle_compose(a, b):
    if a[1] != b[1] or a[2] != b[2]:
        raise ValueError("incompatible swizzle shifts for composition")
    return (a[0] + b[0], a[1], a[2])


def swizzle_mask_bits(sw) -> int:
    return 1 << sw[0]


ELEM_BYTES = {"f32": 4, "f16": 2, "bf16": 2, "s8": 1, "s32": 4}          # lib/core/elemtype.ml:24-30
ELEM_CPP = {"f32": "float", "f16": "__half", "bf16": "__nv_bfloat16", "s8": "int8_t", "s32": "int32_t"}


def elem_vec_width(e: str) -> int:
    return 128 // (8 * ELEM_BYTES[e])


def smem_selector(elem: str, _tile_m: int, tile_k: int):
    n = (tile_k * ELEM_BYTES[elem]) // 16
    b = 0
    while n > 1:
        n //= 2
        b += 1
    return swizzle_make(min(3, max(0, b)), 4, 3)


# --------------------------------------------------------------------------- Pipeline (lib/pipeline/pipeline.ml:9-31)
def pipeline_make(depth_: int, tile_bytes: int) -> dict:
    if depth_ < 1:
        raise ValueError("pipeline depth must be >= 1")
    if tile_bytes <= 0:
        raise ValueError("tile_bytes must be > 0")
    return {"depth": depth_, "tile_bytes": tile_bytes, "smem_bytes": depth_ * tile_bytes}


def stage_of(it: int, depth_: int) -> int:
    return it % depth_


def phase_of(it: int, depth_: int) -> int:
    return (it // depth_) % 2


def smem_offset_of(p: dict, stage: int) -> int:
    return stage * p["tile_bytes"]


def b_smem_offset_of(p: dict, stage: int, bm: int, bk: int, elem_bytes: int) -> int:
    return stage * p["tile_bytes"] + bm * bk * elem_bytes


# --------------------------------------------------------------------------- Cluster (lib/pipeline/cluster.ml:21-74)
def cluster_make(dims, num_warps: int, roles) -> dict:
    if dims[0] * dims[1] * dims[2] > 8:
        raise ValueError("cluster CTA count must be <= 8")
    if any(w >= num_warps for w, _ in roles):
        raise ValueError("warp_id out of range")
    if num_warps <= 0:
        raise ValueError("num_warps must be greater than 0")
    return {"dims": tuple(dims), "num_warps": num_warps, "roles": list(roles)}


def is_2sm(c: dict) -> bool:
    return c["dims"] == (2, 1, 1)


def warps_with_role(c: dict, role: str) -> list:
    return [w for w, r in c["roles"] if r == role]


# --------------------------------------------------------------------------- Tmem (lib/pipeline/tmem.ml:24-110)
def tmem_make(cta_group: int, num_cols: int, num_rows: int) -> dict:
    if num_rows > 128:
        raise ValueError("num_rows must be <= 128")
    if num_cols > 512:
        raise ValueError("num_cols must be <= 512")
    if cta_group == 1 and num_cols > 256:
        raise ValueError("CTA1 num_cols must be <= 256")
    return {"cta_group": cta_group, "num_cols": num_cols, "num_rows": num_rows}


def tmem_address(row: int, col: int) -> int:
    return (row << 16) | col


def tmem_warp_row_offset(warp_id: int) -> int:
    return warp_id * 32


def tmem_num_loads_per_warp(t: dict) -> int:
    return t["num_cols"] // 8


def tmem_total_elems(t: dict) -> int:
    return t["num_rows"] * t["num_cols"]


def tmem_buf_col_offset(buf: int) -> int:
    return buf * 256


def tmem_alloc_ptx(t: dict, smem_var: str) -> str:           # lib/pipeline/tmem.ml:72-75
    return f"tcgen05.alloc.cta_group::{t['cta_group']}.sync.aligned.shared::cta.b32 [{smem_var}], {t['num_cols']};"


def tmem_dealloc_ptx(t: dict, taddr_var: str) -> str:        # lib/pipeline/tmem.ml:77-80
    return f"tcgen05.dealloc.cta_group::{t['cta_group']}.sync.aligned.b32 {taddr_var}, {t['num_cols']};"


def tmem_commit_ptx(t: dict, mbar_var: str) -> str:          # lib/pipeline/tmem.ml:91-94
    return f"tcgen05.commit.cta_group::{t['cta_group']}.mbarrier::arrive::one.shared::cluster.b64 [{mbar_var}];"


def tmem_commit_mask_ptx(t: dict, mbar_var: str, cta_mask: int) -> str:    # lib/pipeline/tmem.ml:115-118
    return (f"tcgen05.commit.cta_group::{t['cta_group']}.mbarrier::arrive::one.multicast::cluster.shared::cluster.b64 "
            f"[{mbar_var}], {cta_mask};")


# --------------------------------------------------------------------------- Memspace (lib/core/memspace.ml:14-47)
SPACES = ("global", "shared", "register", "tensor")


def memspace_can_transfer(src: str, dst: str) -> bool:
    if src == dst:
        return True
    return (src, dst) in {("global", "shared"), ("global", "register"), ("shared", "register"), ("register", "shared"),
                          ("register", "global")}


# --------------------------------------------------------------------------- Mma_atom (lib/atoms/mma_atom.ml:31-157)
_ELEM_TAG = {"f32": "F32", "f16": "F16", "bf16": "BF16", "s8": "S8", "s32": "S32"}
MMA_ATOMS = {   # constructor name -> (arch, m, n, k, a/b type, c/d type), in the order of the reference file
    "sm80_16x8x8_f32f16f16f32": ("SM80", 16, 8, 8, "f16", "f32"),
    "sm80_16x8x16_f32f16f16f32": ("SM80", 16, 8, 16, "f16", "f32"),
    "sm80_16x8x16_f32bf16bf16f32": ("SM80", 16, 8, 16, "bf16", "f32"),
    "sm80_16x8x32_s32s8s8s32": ("SM80", 16, 8, 32, "s8", "s32"),
    "sm90_64x64x16_f32f16f16f32": ("SM90", 64, 64, 16, "f16", "f32"),
    "sm90_64x128x16_f32f16f16f32": ("SM90", 64, 128, 16, "f16", "f32"),
    "sm90_64x64x16_f32bf16bf16f32": ("SM90", 64, 64, 16, "bf16", "f32"),
    "sm100_64x64x16_f32f16f16f32": ("SM100", 64, 64, 16, "f16", "f32"),
    "sm100_128x128x16_f32f16f16f32": ("SM100", 128, 128, 16, "f16", "f32"),
    "sm100_64x64x32_s32s8s8s32": ("SM100", 64, 64, 32, "s8", "s32"),
}


def mma_atom(name: str, a_major: str = "ColMajor", b_major: str = "RowMajor") -> dict:
    arch, m, n, k, ab, cd = MMA_ATOMS[name]
    return {"arch": arch, "m": m, "n": n, "k": k, "a_type": ab, "b_type": ab, "c_type": cd, "d_type": cd,
            "a_major": a_major, "b_major": b_major}


def mma_atom_thread_count(a: dict) -> int:
    return 32 if a["arch"] == "SM80" else 128


def mma_atom_is_wgmma(a: dict) -> bool:
    return a["arch"] != "SM80"


def mma_atom_emit_cpp(a: dict) -> str:
    mc = lambda mj: "T" if mj == "ColMajor" else "N"
    return (f"{a['arch']}_{a['m']}x{a['n']}x{a['k']}_{_ELEM_TAG[a['d_type']]}{_ELEM_TAG[a['a_type']]}"
            f"{_ELEM_TAG[a['b_type']]}{_ELEM_TAG[a['c_type']]}_{mc(a['a_major'])}{mc(a['b_major'])}")


# --------------------------------------------------------------------------- Copy_atom (lib/atoms/copy_atom.ml:23-137)
# "TmaLoadPair" is this build's name for the reference's fifth kind (its SM100 cluster-wide TMA load).
def copy_atom(kind: str, elem: str, src: str = "global", dst: str = "shared") -> dict:
    bw = ELEM_BYTES[elem]
    if kind in ("AsyncCopyGlobal", "AsyncCopyCached"):
        return {"kind": kind, "src": "global", "dst": "shared", "elem": elem, "bulk_bytes": 16, "vec_width": 16 // bw}
    if kind in ("Ldmatrix", "LdmatrixTrans"):
        return {"kind": kind, "src": "shared", "dst": "register", "elem": elem, "bulk_bytes": 32, "vec_width": 8}
    if kind in ("TmaLoad", "TmaLoadPair"):
        return {"kind": kind, "src": "global", "dst": "shared", "elem": elem, "bulk_bytes": 128, "vec_width": 128 // bw}
    if kind == "TmaStore":
        return {"kind": kind, "src": "shared", "dst": "global", "elem": elem, "bulk_bytes": 128, "vec_width": 128 // bw}
    if kind == "UniversalCopy":
        return {"kind": kind, "src": src, "dst": dst, "elem": elem, "bulk_bytes": bw, "vec_width": 1}
    raise ValueError("unknown copy atom kind")


def copy_atom_is_tma(a: dict) -> bool:
    return a["kind"] in ("TmaLoad", "TmaStore", "TmaLoadPair")


def copy_atom_is_async(a: dict) -> bool:
    return a["kind"] in ("AsyncCopyGlobal", "AsyncCopyCached") or copy_atom_is_tma(a)


def copy_atom_requires_mbar(a: dict) -> bool:
    return copy_atom_is_tma(a)


def copy_atom_emit_cpp(a: dict) -> str:
    fixed = {"AsyncCopyGlobal": "SM80_CP_ASYNC_CACHEGLOBAL<cute::uint128_t>", "AsyncCopyCached": "SM80_CP_ASYNC_CACHEALL<cute::uint128_t>",
             "TmaLoad": "SM90_TMA_LOAD", "TmaStore": "SM90_TMA_STORE", "TmaLoadPair": "SM100_TMA_LOAD_" + "MULTI" + "CAST",
             "Ldmatrix": "SM80_U32x4_LDSM_N", "LdmatrixTrans": "SM80_U16x8_LDSM_T"}
    return fixed.get(a["kind"]) or f"UniversalCopy<{ELEM_CPP[a['elem']]}>"


# --------------------------------------------------------------------------- Tiled_mma (lib/atoms/tiled_mma.ml:12-53)
def tiled_mma_make(atom: dict, thread_layout: Layout, warp_layout: Layout, tiler_mn) -> dict:
    if layout_size(thread_layout) != mma_atom_thread_count(atom):
        raise ValueError("thread_layout size does not match atom thread count")
    return {"atom": atom, "thread_layout": thread_layout, "warp_layout": warp_layout, "tiler_mn": tiler_mn}


def tiled_mma_thread_count(t: dict) -> int:
    return layout_size(t["thread_layout"]) * layout_size(t["warp_layout"])


def tiled_mma_warp_count(t: dict) -> int:
    return layout_size(t["warp_layout"])


def tiled_mma_tile_shape_mnk(t: dict):
    mn = flatten(t["tiler_mn"])
    if len(mn) != 2:
        raise ValueError("tiler_mn must represent exactly two dimensions (M and N)")
    return (mn[0], mn[1], t["atom"]["k"])


def tiled_mma_partition(t: dict, which: str) -> Layout:
    a = t["atom"]
    total = {"a": a["m"] * a["k"], "b": a["n"] * a["k"], "c": a["m"] * a["n"]}[which]
    return Layout(total // layout_size(t["thread_layout"]), 1)


# --------------------------------------------------------------------------- Tiled_copy (lib/atoms/tiled_copy.ml:10-50)
def tiled_copy_make(atom: dict, thread_layout: Layout, val_layout: Layout) -> dict:
    if layout_size(val_layout) != atom["vec_width"]:
        raise ValueError("val_layout size does not match atom vec_width")
    if layout_size(thread_layout) <= 0:
        raise ValueError("thread_layout size must be positive")
    return {"atom": atom, "thread_layout": thread_layout, "val_layout": val_layout}


def tiled_copy_tile_size(t: dict) -> int:
    return layout_size(t["thread_layout"]) * layout_size(t["val_layout"])


def tiled_copy_partition(t: dict, layout: Layout) -> Layout:
    d = flat_divide(layout, layout_size(t["thread_layout"]))
    return Layout(d.shape[1], d.stride[1])


# --------------------------------------------------------------------------- Tile_op (lib/pipeline/tile_op.ml:18-107)
def tile_op_make(tiled_mma: dict, accum_loc: str, tmem: dict | None = None, double_buf: bool = False) -> dict:
    if accum_loc == "TensorMem" and tmem is None:
        raise ValueError("TensorMem requires a tmem descriptor")
    return {"tiled_mma": tiled_mma, "accum_loc": accum_loc, "tmem": tmem, "double_buf": double_buf}


def tile_op_is_tmem(t: dict) -> bool:
    return t["accum_loc"] == "TensorMem"


def tile_op_is_wgmma(t: dict) -> bool:
    return mma_atom_is_wgmma(t["tiled_mma"]["atom"])


def tile_op_accum_elems_per_thread(t: dict) -> int:
    return layout_size(tiled_mma_partition(t["tiled_mma"], "c"))


def tile_op_emit_mma(t: dict, a_desc: str, b_desc: str, enable_accum: bool) -> str:
    if t["accum_loc"] == "Registers":
        return f"mma.sync.aligned.{mma_atom_emit_cpp(t['tiled_mma']['atom'])} acc, {a_desc}, {b_desc}, acc;"
    cg = t["tmem"]["cta_group"] if t["tmem"] else 1
    return f"tcgen05.mma.cta_group::{cg}.kind::mxf16 [tmem_addr], {a_desc}, {b_desc}, [i_desc], {1 if enable_accum else 0};"


def tile_op_emit_commit(t: dict, mbar_var: str, cta_mask: int) -> str:
    if t["accum_loc"] == "Registers" or t["tmem"] is None:
        return ""
    return tmem_commit_mask_ptx(t["tmem"], mbar_var, cta_mask) if cta_mask > 1 else tmem_commit_ptx(t["tmem"], mbar_var)


def tile_op_emit_accum_decl(t: dict, var: str) -> str:
    if t["accum_loc"] == "TensorMem":
        return ""
    n = tile_op_accum_elems_per_thread(t)
    return f"float {var}[{n}] = {{{', '.join(['0.0f'] * n)}}};"


def tile_op_emit_tmem_alloc(t: dict, smem_var: str) -> str:
    return tmem_alloc_ptx(t["tmem"], smem_var) if t["tmem"] else ""


def tile_op_emit_tmem_dealloc(t: dict, taddr_var: str) -> str:
    return tmem_dealloc_ptx(t["tmem"], taddr_var) if t["tmem"] else ""


# --------------------------------------------------------------------------- Smem_desc (lib/pipeline/smem_desc.ml:17-43)
def smem_desc_encode(base: int, leading: int, stride: int, sw_bits: int) -> int:
    # OCaml native ints are 63 bits wide: the value is reported as that bit pattern (unsigned).
    return (base | (leading << 16) | (stride << 32) | (sw_bits << 61)) & ((1 << 63) - 1)


# --------------------------------------------------------------------------- Tile_io (lib/pipeline/tile_io.ml:75-87,119-127)
def bytes_per_load_a(elem: str, bm: int, bk: int) -> int:
    return bm * bk * ELEM_BYTES[elem]


def bytes_per_load_b(elem: str, bn: int, bk: int, cta_group: int) -> int:
    return (bn // 2 if cta_group == 2 else bn) * bk * ELEM_BYTES[elem]


def expect_tx(elem: str, strategy: str, bm: int, bn: int, bk: int) -> int:
    # "TmaPair" is this build's name for the reference's SM100 strategy tag (tile_io.ml:8)
    b_cols = bn // 2 if strategy == "TmaPair" else bn
    return (bm + b_cols) * bk * ELEM_BYTES[elem]


# --------------------------------------------------------------------------- Predicate (lib/pipeline/predicate.ml:9-41)
def predicate_count_valid(shape, bounds) -> int:
    shapes = flatten(shape)
    if len(bounds) != rank(shape):
        raise ValueError("bounds length must match layout rank")
    count = 0
    for k in range(size(shape)):
        rem, coords = k, []
        for sh in shapes:
            coords.append(rem % sh)
            rem //= sh
        count += all(c < b for c, b in zip(coords, bounds))
    return count


def predicate_residue(shape, bounds) -> list:
    return [b % s for b, s in zip(bounds, flatten(shape))]


# --------------------------------------------------------------------------- Kernel_desc / Lower (lib/kernel/kernel_desc.ml:118-202, lower.ml:36-97)
def make_blackwell(name: str, bm: int, bn: int, bk: int, elem: str, m: int, n: int, k: int) -> dict:
    cluster = cluster_make((2, 1, 1), 6, [(0, "Producer"), (1, "Consumer"), (2, "Epilogue"), (3, "Epilogue"),
                                          (4, "Epilogue"), (5, "Scheduler")])
    pipeline = pipeline_make(4, (bm + bn) * bk * ELEM_BYTES[elem])
    return {"family": "Blackwell", "name": name, "bm": bm, "bn": bn, "bk": bk, "elem": elem,
            "swizzle": smem_selector(elem, bm, bk), "cluster": cluster, "pipeline": pipeline,
            "strategy": "TmaPair", "copy_bulk_bytes": 128, "copy_vec": 128 // ELEM_BYTES[elem],
            "atom": (128, 128, 16), "atom_threads": 128, "tmem": tmem_make(2, 512, bm), "double_buf": True,
            "pred_a_bounds": [m, k], "pred_b_bounds": [k, n], "pred_c_bounds": [m, n], "sm_count": 148}


def validate(d: dict):
    pow2 = lambda x: x > 0 and (x & (x - 1)) == 0
    am, an, ak = d["atom"]
    if not (pow2(d["bm"]) and pow2(d["bn"]) and pow2(d["bk"])):
        return "Matrix dimensions (bm, bn, bk) must be positive powers of 2"
    if d["bm"] % am or d["bn"] % an or d["bk"] % ak:
        return f"Tile dimensions must be divisible by atoms: M={am}, N={an}, K={ak}"
    if d["pipeline"]["smem_bytes"] > d["sm_count"] * 227 * 1024:
        return "Total pipeline shared memory exceeds the limit of sm_count * 227KB"
    if d["family"] == "Blackwell" and not is_2sm(d["cluster"]):
        return "Blackwell requires 2SM cluster"
    return None


def arithmetic_intensity(d: dict) -> float:
    eff_bn = d["bn"] // 2 if d["family"] == "Blackwell" else d["bn"]
    return 2.0 * d["bm"] * d["bn"] * d["bk"] / ((d["bm"] + eff_bn) * d["bk"] * ELEM_BYTES[d["elem"]])


def lower_sm100(name: str, elem: str, bm: int, bn: int, bk: int) -> dict:
    if elem not in ("f16", "bf16", "s8"):
        raise ValueError(f"UnsupportedElem: arch=SM100 elem={elem.upper()}")
    return make_blackwell(name, bm, bn, bk, elem, bm * 32, bn * 32, bk * 32)
