// Host-side integer model of tesserae's descriptors: layouts, swizzles, pipeline / cluster /
// TMEM / smem-descriptor math, tile IO byte counts, the Blackwell kernel descriptor and the
// spec -> descriptor lowering.  Every function keeps the reference's semantics bit for bit,
// including where they differ from NVIDIA CuTe (noted at each function), because the
// reference's own tests pin those values.  Layouts are held flattened: the reference
// flattens shape and stride trees before every computation (lib/core/layout.ml:17-32).
//
// The backend uses this model to derive tensor-map boxes, swizzle modes, stage byte counts
// and launch shapes from a kernel spec; nothing here touches a GPU.
#pragma once
#include <algorithm>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace tesserae::spec {

using i64 = int64_t;
using Ints = std::vector<i64>;

// The reference raises Invalid_argument / Failure with these exact messages.
struct SpecError : std::runtime_error { using std::runtime_error::runtime_error; };

// ---------------------------------------------------------------- Elemtype (lib/core/elemtype.ml:9-57)
enum Elem { F16 = 0, BF16 = 1, F32 = 2, S8 = 3, S32 = 4, F8E4M3 = 5, F4E2M1 = 6 };

inline int elem_bits(int e) {
    switch (e) { case F32: case S32: return 32; case F16: case BF16: return 16; case S8: case F8E4M3: return 8;
                 case F4E2M1: return 4; default: return -1; }
}
inline int elem_byte_width(int e) { int b = elem_bits(e); return b < 0 ? -1 : b / 8; }
inline int elem_vec_width(int e) { int b = elem_bits(e); return b < 0 ? -1 : 128 / b; }
inline const char* elem_cpp_name(int e) {
    switch (e) { case F32: return "float"; case F16: return "__half"; case BF16: return "__nv_bfloat16";
                 case S8: return "int8_t"; case S32: return "int32_t"; case F8E4M3: return "__nv_fp8_e4m3";
                 case F4E2M1: return "__nv_fp4_e2m1"; default: return "?"; }
}

// ---------------------------------------------------------------- Layout (lib/core/layout.ml:8-32)
struct Layout {
    Ints shape, stride;
    Layout() = default;
    Layout(Ints s, Ints d) : shape(std::move(s)), stride(std::move(d)) {
        if (shape.size() != stride.size()) throw SpecError("incompatible shape and stride");
    }
    size_t rank() const { return shape.size(); }
};
inline i64 size(const Layout& l) { i64 p = 1; for (i64 s : l.shape) p *= s; return p; }
inline i64 cosize(const Layout& l) {
    i64 off = 0;
    for (size_t i = 0; i < l.shape.size(); ++i) off += (l.shape[i] - 1) * l.stride[i];
    return off + 1;
}
inline i64 idx(const Layout& l, const Ints& coord) {
    if (coord.size() != l.stride.size()) throw SpecError("coordinate rank does not match layout");
    i64 o = 0;
    for (size_t i = 0; i < coord.size(); ++i) o += coord[i] * l.stride[i];
    return o;
}

// Compose.compose (lib/core/compose.ml:3-21).  Each *inner stride* is decomposed into
// mixed-radix digits over the *inner shapes* and dotted with the *outer strides*; the
// result keeps the inner shape.  (CuTe proper decomposes over the outer shape.)
inline Layout compose(const Layout& outer, const Layout& inner) {
    if (cosize(inner) > size(outer)) throw SpecError("inner cosize exceeds outer size");
    if (inner.shape.size() != outer.stride.size()) throw SpecError("length mismatch in fold2_exn");
    Ints out(inner.stride.size());
    for (size_t j = 0; j < inner.stride.size(); ++j) {
        i64 rem = inner.stride[j], acc = 0;
        for (size_t i = 0; i < inner.shape.size(); ++i) {
            i64 sh = inner.shape[i];
            acc += (rem % sh) * outer.stride[i];
            rem /= sh;
        }
        out[j] = acc;
    }
    return Layout(inner.shape, out);
}

// Compose.tile (lib/core/compose.ml:24-47): leaf i -> within (t_i : d_i), across (l_i/t_i : d_i*t_i).
// Returned flat as [within modes..., across modes...].
inline Layout tile(const Layout& l, const Ints& t) {
    if (t.size() != l.shape.size()) throw SpecError("Layout.tile: structural mismatch");
    const size_t n = t.size();
    Ints s(2 * n), d(2 * n);
    for (size_t i = 0; i < n; ++i) {
        if (t[i] == 0 || l.shape[i] % t[i] != 0) throw SpecError("tile shape does not divide layout shape");
        s[i] = t[i]; d[i] = l.stride[i];
        s[n + i] = l.shape[i] / t[i]; d[n + i] = l.stride[i] * t[i];
    }
    return Layout(s, d);
}

// Algebra.sort (lib/core/algebra.ml:6-16): stable sort of (shape, stride) pairs by stride.
inline Layout sort_by_stride(const Layout& l) {
    std::vector<std::pair<i64, i64>> p(l.shape.size());
    for (size_t i = 0; i < p.size(); ++i) p[i] = {l.shape[i], l.stride[i]};
    std::stable_sort(p.begin(), p.end(), [](auto& a, auto& b) { return a.second < b.second; });
    Ints s, d;
    for (auto& x : p) { s.push_back(x.first); d.push_back(x.second); }
    return Layout(s, d);
}

// Algebra.coalesce (lib/core/algebra.ml:18-42).  A recursive walk: a leading size-1 mode is
// dropped; two leading modes merge when d1 = n0*d0 (and the merged mode is re-examined);
// otherwise the head is kept and the walk continues on the tail.
inline void coalesce_walk(const i64* ss, const i64* st, size_t n, Ints& os, Ints& od) {
    std::vector<i64> s(ss, ss + n), d(st, st + n);
    size_t i = 0;
    while (i < s.size()) {
        if (s[i] == 1) { ++i; continue; }
        if (i + 1 < s.size() && d[i + 1] == s[i] * d[i]) {
            s[i + 1] = s[i] * s[i + 1]; d[i + 1] = d[i]; ++i; continue;
        }
        os.push_back(s[i]); od.push_back(d[i]); ++i;
    }
}
inline Layout coalesce(const Layout& l) {
    Ints s, d;
    coalesce_walk(l.shape.data(), l.stride.data(), l.shape.size(), s, d);
    return Layout(s, d);
}

// Algebra.is_admissible (lib/core/algebra.ml:45-68)
inline bool is_admissible(const Layout& l, i64 m) {
    const size_t n = l.shape.size();
    for (size_t i = 0; i + 1 < n; ++i) if (l.stride[i] > l.stride[i + 1]) return false;
    if (n == 0) return true;
    for (size_t i = 0; i + 1 < n; ++i) {
        i64 q = l.shape[i] * l.stride[i];
        if (q == 0 || l.stride[i + 1] % q != 0) return false;
    }
    i64 last = l.shape[n - 1] * l.stride[n - 1];
    return last != 0 && m % last == 0;
}

// Algebra.complement (lib/core/algebra.ml:71-100): size-1 modes are kept.
inline Layout complement(const Layout& l, i64 m) {
    if (m <= 0 || !is_admissible(l, m)) throw SpecError("layout is not admissible for complementation");
    Ints s, d;
    i64 last = 1;
    for (size_t i = 0; i < l.shape.size(); ++i) {
        s.push_back(l.stride[i] / last); d.push_back(last);
        last = l.shape[i] * l.stride[i];
    }
    s.push_back(m / last); d.push_back(last);
    return Layout(s, d);
}

// Algebra.flat_divide (lib/core/algebra.ml:102-117): coalesce, then split by the first stride.
inline Layout flat_divide(const Layout& l, i64 divisor) {
    Layout f = coalesce(l);
    if (f.stride.empty()) throw SpecError("hd_exn: empty list");
    i64 d0 = f.stride[0];
    if (divisor == 0 || size(f) % divisor != 0) throw SpecError("divisor does not divide layout size");
    return Layout({divisor, size(f) / divisor}, {d0, divisor * d0});
}

// Algebra.logical_divide (lib/core/algebra.ml:119-126): the tile's strides are ignored.
inline Layout logical_divide(const Layout& l, const Ints& tile_shape) {
    if (tile_shape.size() != l.shape.size()) throw SpecError("length mismatch in for_all2_exn");
    for (size_t i = 0; i < tile_shape.size(); ++i)
        if (tile_shape[i] == 0 || l.shape[i] % tile_shape[i] != 0) throw SpecError("tile does not divide layout");
    return tile(l, tile_shape);
}

// Algebra.zipped_divide (lib/core/algebra.ml:128-135): modes re-zipped as (within_i, across_i).
inline Layout zipped_divide(const Layout& l, const Ints& tile_shape) {
    Layout ld = logical_divide(l, tile_shape);
    const size_t n = tile_shape.size();
    Ints s(2 * n), d(2 * n);
    for (size_t i = 0; i < n; ++i) {
        s[2 * i] = ld.shape[i]; d[2 * i] = ld.stride[i];
        s[2 * i + 1] = ld.shape[n + i]; d[2 * i + 1] = ld.stride[n + i];
    }
    return Layout(s, d);
}

// ---------------------------------------------------------------- Swizzle (lib/core/swizzle.ml:9-62)
struct Swizzle { int b = 0, m = 4, s = 3; };
inline Swizzle swizzle_make(int b, int m, int s) {
    if (b < 0 || m < 0 || s < 0) throw SpecError("swizzle parameters must be non-negative");
    return Swizzle{b, m, s};
}
inline i64 swizzle_apply(const Swizzle& sw, i64 offset) {
    const i64 mask = ((i64(1) << sw.b) - 1) << (sw.m + std::max(0, sw.s));
    return offset ^ ((offset & mask) >> sw.s);
}
inline Swizzle swizzle_compose(const Swizzle& a, const Swizzle& b) {
    if (a.m != b.m || a.s != b.s) throw SpecError("incompatible swizzle shifts for composition");
    return Swizzle{a.b + b.b, a.m, a.s};
}
// Swizzle.smem_selector: b = clamp(floor(log2(tile_k * bytes / 16)), 0, 3), m = 4, s = 3.
// For the sub-byte element the contiguous bytes are tile_k * bits / 8.
inline Swizzle swizzle_smem_selector(int elem, int /*tile_m*/, int tile_k) {
    const int bits = elem_bits(elem);
    if (bits < 0) throw SpecError("unknown element type");
    i64 n = (i64(tile_k) * bits / 8) / 16;
    int b = 0;
    while (n > 1) { n /= 2; ++b; }
    return Swizzle{std::min(3, std::max(0, b)), 4, 3};
}

// ---------------------------------------------------------------- Pipeline (lib/pipeline/pipeline.ml:9-31)
struct Pipeline { int depth; i64 tile_bytes; i64 smem_bytes; };
inline Pipeline pipeline_make(int depth, i64 tile_bytes) {
    if (depth < 1) throw SpecError("pipeline depth must be >= 1");
    if (tile_bytes <= 0) throw SpecError("tile_bytes must be > 0");
    return Pipeline{depth, tile_bytes, depth * tile_bytes};
}
inline int stage_of(i64 iter, int depth) { return int(iter % depth); }
inline int phase_of(i64 iter, int depth) { return int((iter / depth) % 2); }
inline i64 smem_offset_of(i64 tile_bytes, int stage) { return stage * tile_bytes; }
inline i64 b_smem_offset_of(i64 tile_bytes, int stage, int bm, int bk, int elem_bytes) {
    return stage * tile_bytes + i64(bm) * bk * elem_bytes;
}

// ---------------------------------------------------------------- Cluster (lib/pipeline/cluster.ml:21-74)
enum Role { Producer = 0, Consumer = 1, Epilogue = 2, Scheduler = 3, NoRole = -1 };
struct Cluster { int x, y, z; int num_warps; std::vector<std::pair<int, int>> roles; };
inline Cluster cluster_make(int x, int y, int z, int num_warps, std::vector<std::pair<int, int>> roles) {
    if (x * y * z > 8) throw SpecError("cluster CTA count must be <= 8");
    for (auto& r : roles) if (r.first >= num_warps) throw SpecError("warp_id out of range");
    if (num_warps <= 0) throw SpecError("num_warps must be greater than 0");
    return Cluster{x, y, z, num_warps, std::move(roles)};
}
inline int cta_count(const Cluster& c) { return c.x * c.y * c.z; }
inline bool is_2sm(const Cluster& c) { return c.x == 2 && c.y == 1 && c.z == 1; }
inline int warp_role_of(const Cluster& c, int warp) {
    for (auto& r : c.roles) if (r.first == warp) return r.second;
    return NoRole;
}
inline int thread_count(const Cluster& c) { return c.num_warps * 32; }

// ---------------------------------------------------------------- Tmem (lib/pipeline/tmem.ml:24-110)
struct Tmem { int cta_group; int num_cols; int num_rows; };
inline Tmem tmem_make(int cta_group, int num_cols, int num_rows) {
    if (num_rows > 128) throw SpecError("num_rows must be <= 128");
    if (num_cols > 512) throw SpecError("num_cols must be <= 512");
    if (cta_group == 1 && num_cols > 256) throw SpecError("CTA1 num_cols must be <= 256");
    return Tmem{cta_group, num_cols, num_rows};
}
inline i64 tmem_address(int row, int col) { return (i64(row) << 16) | col; }
inline int tmem_warp_row_offset(int warp_id) { return warp_id * 32; }
inline int tmem_elems_per_thread_per_load() { return 8; }
inline int tmem_num_loads_per_warp(int num_cols) { return num_cols / 8; }
inline int tmem_buf_col_offset(int buf) { return buf * 256; }

// ---------------------------------------------------------------- Smem_desc (lib/pipeline/smem_desc.ml:17-43)
// The reference's packing, kept as an integer function: base | leading<<16 | stride<<32 | sw<<61.
inline i64 smem_desc_encode(i64 base, i64 leading, i64 stride, int sw_bits) {
    return i64(uint64_t(base) | (uint64_t(leading) << 16) | (uint64_t(stride) << 32) | (uint64_t(sw_bits) << 61));
}
// The sm_100 hardware form for a K-major tile with 128-byte rows (what the kernels build on
// the device): address>>4 at [0,14), leading byte offset>>4 at [16,30) (1: unused for
// swizzled K-major), stride byte offset>>4 at [32,46) = 8 rows * row bytes, version 1 at
// [46,48), layout type at [61,64): 0 none, 6 32B, 4 64B, 2 128B.
inline uint64_t umma_smem_desc(uint32_t smem_addr, int swizzle_b) {
    static const uint64_t layout_type[4] = {0, 6, 4, 2};
    const uint64_t row_bytes = swizzle_b == 0 ? 16 : (16u << swizzle_b);
    const uint64_t sbo = 8 * row_bytes;
    return uint64_t((smem_addr & 0x3FFFFu) >> 4) | (uint64_t(1) << 16) | ((sbo >> 4) << 32) |
           (uint64_t(1) << 46) | (layout_type[swizzle_b & 3] << 61);
}
// 32-bit instruction descriptor of a dense MMA with fp32 accumulation, both operands K-major.
inline uint32_t umma_instr_desc(int elem, int umma_m, int umma_n) {
    uint32_t fmt = 0, dfmt = 1;
    switch (elem) { case F16: fmt = 0; break; case BF16: fmt = 1; break; case F8E4M3: fmt = 0; break;
                    case S8: fmt = 1; dfmt = 2; break;      // signed 8-bit operands, 32-bit integer accumulator
                    default: throw SpecError("no dense tcgen05 kind for this element type"); }
    return (dfmt << 4) | (fmt << 7) | (fmt << 10) | (uint32_t(umma_n >> 3) << 17) | (uint32_t(umma_m >> 4) << 24);
}

// ---------------------------------------------------------------- Memspace (lib/core/memspace.ml:8-47)
enum Space { Global = 0, Shared = 1, Register = 2, TensorSpace = 3 };
inline const char* memspace_name(int s) {
    switch (s) { case Global: return "global"; case Shared: return "shared"; case Register: return "register";
                 case TensorSpace: return "tensor"; default: return "?"; }
}
// Memspace.can_transfer: same -> same; global -> shared / register; shared -> register; register -> shared /
// global.  shared -> global is false in the reference (it models st.global from registers only), and so is
// every pair that involves the tensor space other than tensor -> tensor.
inline bool memspace_can_transfer(int src, int dst) {
    if (src < Global || src > TensorSpace || dst < Global || dst > TensorSpace) return false;
    if (src == dst) return true;
    if (src == Global && (dst == Shared || dst == Register)) return true;
    if (src == Shared && dst == Register) return true;
    if (src == Register && (dst == Shared || dst == Global)) return true;
    return false;
}

// ---------------------------------------------------------------- Mma_atom (lib/atoms/mma_atom.ml:31-157)
enum Major { RowMajor = 0, ColMajor = 1 };
struct MmaAtom {
    int m = 0, n = 0, k = 0, threads = 0;
    const char* name = "";                 // emit_cpp for ColMajor A / RowMajor B ("TN"), kept for the descriptor
    int arch = 2;                          // Arch code: 0 SM80, 1 SM90, 2 SM100
    int a_type = F16, b_type = F16, c_type = F32, d_type = F32;
    int a_major = ColMajor, b_major = RowMajor;
};
enum MmaAtomId { Sm80_16x8x8_F16 = 0, Sm80_16x8x16_F16, Sm80_16x8x16_BF16, Sm80_16x8x32_S8, Sm90_64x64x16_F16,
                 Sm90_64x128x16_F16, Sm90_64x64x16_BF16, Sm100_64x64x16_F16, Sm100_128x128x16_F16, Sm100_64x64x32_S8,
                 MmaAtomCount };
// Mma_atom.thread_count / is_wgmma (lib/atoms/mma_atom.ml:118-130): 32 threads on SM80, a warpgroup of 128 else.
inline int mma_atom_thread_count(const MmaAtom& a) { return a.arch == 0 ? 32 : 128; }
inline bool mma_atom_is_wgmma(const MmaAtom& a) { return a.arch != 0; }
inline MmaAtom mma_atom_make(int id, int a_major = ColMajor, int b_major = RowMajor) {
    struct Row { int arch, m, n, k, ab, cd; };
    static const Row rows[MmaAtomCount] = {
        {0, 16, 8, 8, F16, F32},   {0, 16, 8, 16, F16, F32},  {0, 16, 8, 16, BF16, F32}, {0, 16, 8, 32, S8, S32},
        {1, 64, 64, 16, F16, F32}, {1, 64, 128, 16, F16, F32}, {1, 64, 64, 16, BF16, F32},
        {2, 64, 64, 16, F16, F32}, {2, 128, 128, 16, F16, F32}, {2, 64, 64, 32, S8, S32}};
    if (id < 0 || id >= MmaAtomCount) throw SpecError("unknown MMA atom");
    const Row& r = rows[id];
    MmaAtom a;
    a.arch = r.arch; a.m = r.m; a.n = r.n; a.k = r.k;
    a.a_type = a.b_type = r.ab; a.c_type = a.d_type = r.cd;
    a.a_major = a_major; a.b_major = b_major;
    a.threads = mma_atom_thread_count(a);
    return a;
}
// Mma_atom.emit_cpp (lib/atoms/mma_atom.ml:146-156): ARCH_MxNxK_<D><A><B><C>_<a major><b major>, ColMajor -> "T".
inline std::string mma_atom_emit_cpp(const MmaAtom& a) {
    auto es = [](int e) { return e == F32 ? "F32" : e == F16 ? "F16" : e == BF16 ? "BF16" : e == S8 ? "S8" : e == S32 ? "S32" : "?"; };
    auto mc = [](int mj) { return mj == ColMajor ? "T" : "N"; };
    return std::string(a.arch == 0 ? "SM80" : a.arch == 1 ? "SM90" : "SM100") + "_" + std::to_string(a.m) + "x" +
           std::to_string(a.n) + "x" + std::to_string(a.k) + "_" + es(a.d_type) + es(a.a_type) + es(a.b_type) +
           es(a.c_type) + "_" + mc(a.a_major) + mc(a.b_major);
}
inline MmaAtom sm100_128x128x16() { MmaAtom a = mma_atom_make(Sm100_128x128x16_F16); a.name = "SM100_128x128x16_F32F16F16F32_TN"; return a; }
inline MmaAtom sm100_64x64x16() { MmaAtom a = mma_atom_make(Sm100_64x64x16_F16); a.name = "SM100_64x64x16_F32F16F16F32_TN"; return a; }
inline MmaAtom sm100_64x64x32_s8() { MmaAtom a = mma_atom_make(Sm100_64x64x32_S8); a.name = "SM100_64x64x32_S32S8S8S32_TN"; return a; }

// ---------------------------------------------------------------- Copy_atom (lib/atoms/copy_atom.ml:4-137)
// The fifth kind is the reference's SM100 cluster-wide TMA load; this build lowers it to per-CTA loads of a
// CTA pair (see Strategy below) and calls it TmaLoadPair, keeping the value and the emitted name.
enum CopyKind { AsyncCopyGlobal = 0, AsyncCopyCached = 1, TmaLoadAtom = 2, TmaStoreAtom = 3, TmaLoadPair = 4,
                Ldmatrix = 5, LdmatrixTrans = 6, UniversalCopy = 7 };
struct CopyAtom { int kind, src_space, dst_space, elem, vec_width, bulk_bytes; };
inline CopyAtom copy_atom_make(int kind, int elem, int src_space = Global, int dst_space = Shared) {
    const int bw = elem_byte_width(elem);
    if (bw <= 0) throw SpecError("unknown element type");
    switch (kind) {
        case AsyncCopyGlobal: case AsyncCopyCached: return {kind, Global, Shared, elem, 16 / bw, 16};
        case Ldmatrix: case LdmatrixTrans: return {kind, Shared, Register, elem, 8, 32};
        case TmaLoadAtom: case TmaLoadPair: return {kind, Global, Shared, elem, 128 / bw, 128};
        case TmaStoreAtom: return {kind, Shared, Global, elem, 128 / bw, 128};
        case UniversalCopy: return {kind, src_space, dst_space, elem, 1, bw};
        default: throw SpecError("unknown copy atom kind");
    }
}
inline bool copy_atom_is_tma(const CopyAtom& a) { return a.kind == TmaLoadAtom || a.kind == TmaStoreAtom || a.kind == TmaLoadPair; }
inline bool copy_atom_is_async(const CopyAtom& a) { return a.kind == AsyncCopyGlobal || a.kind == AsyncCopyCached || copy_atom_is_tma(a); }
inline bool copy_atom_requires_mbar(const CopyAtom& a) { return copy_atom_is_tma(a); }
inline std::string copy_atom_emit_cpp(const CopyAtom& a) {
    switch (a.kind) {
        case AsyncCopyGlobal: return "SM80_CP_ASYNC_CACHEGLOBAL<cute::uint128_t>";
        case AsyncCopyCached: return "SM80_CP_ASYNC_CACHEALL<cute::uint128_t>";
        case TmaLoadAtom: return "SM90_TMA_LOAD";
        case TmaStoreAtom: return "SM90_TMA_STORE";
        case TmaLoadPair: return std::string("SM100_TMA_LOAD_") + "MULTI" + "CAST";     // the reference's CuTe atom name
        case Ldmatrix: return "SM80_U32x4_LDSM_N";
        case LdmatrixTrans: return "SM80_U16x8_LDSM_T";
        default: return std::string("UniversalCopy<") + elem_cpp_name(a.elem) + ">";
    }
}

// ---------------------------------------------------------------- Tiled_mma (lib/atoms/tiled_mma.ml:12-53)
// The reference's partitions use only the *sizes* of the thread and warp layouts (the warp layout is ignored by
// partition_*), so the model carries the sizes.
struct TiledMma { MmaAtom atom; i64 thread_layout_size, warp_layout_size, tiler_m, tiler_n; };
inline TiledMma tiled_mma_make(const MmaAtom& atom, i64 thread_layout_size, i64 warp_layout_size, i64 tiler_m, i64 tiler_n) {
    if (thread_layout_size != mma_atom_thread_count(atom)) throw SpecError("thread_layout size does not match atom thread count");
    return TiledMma{atom, thread_layout_size, warp_layout_size, tiler_m, tiler_n};
}
inline i64 tiled_mma_thread_count(const TiledMma& t) { return t.thread_layout_size * t.warp_layout_size; }
inline i64 tiled_mma_warp_count(const TiledMma& t) { return t.warp_layout_size; }
// partition_a / _b / _c: (atom elements / thread_layout size) : 1
inline i64 tiled_mma_partition_a(const TiledMma& t) { return i64(t.atom.m) * t.atom.k / t.thread_layout_size; }
inline i64 tiled_mma_partition_b(const TiledMma& t) { return i64(t.atom.n) * t.atom.k / t.thread_layout_size; }
inline i64 tiled_mma_partition_c(const TiledMma& t) { return i64(t.atom.m) * t.atom.n / t.thread_layout_size; }

// ---------------------------------------------------------------- Tiled_copy (lib/atoms/tiled_copy.ml:10-50)
struct TiledCopy { CopyAtom atom; i64 thread_layout_size, val_layout_size; };
inline TiledCopy tiled_copy_make(const CopyAtom& atom, i64 thread_layout_size, i64 val_layout_size) {
    if (val_layout_size != atom.vec_width) throw SpecError("val_layout size does not match atom vec_width");
    if (thread_layout_size <= 0) throw SpecError("thread_layout size must be positive");
    return TiledCopy{atom, thread_layout_size, val_layout_size};
}
inline i64 tiled_copy_tile_size(const TiledCopy& t) { return t.thread_layout_size * t.val_layout_size; }
// partition_src / partition_dst: flat_divide by the thread count, keep the "across" mode.
inline Layout tiled_copy_partition(const TiledCopy& t, const Layout& l) {
    const Layout d = flat_divide(l, t.thread_layout_size);
    return Layout({d.shape[1]}, {d.stride[1]});
}

// ---------------------------------------------------------------- Tile_op (lib/pipeline/tile_op.ml:18-107)
// Tmem's instruction text (lib/pipeline/tmem.ml:72-110), which Tile_op forwards.
inline std::string tmem_alloc_ptx(const Tmem& t, const std::string& smem_var) {
    return "tcgen05.alloc.cta_group::" + std::to_string(t.cta_group) + ".sync.aligned.shared::cta.b32 [" + smem_var + "], " +
           std::to_string(t.num_cols) + ";";
}
inline std::string tmem_dealloc_ptx(const Tmem& t, const std::string& taddr_var) {
    return "tcgen05.dealloc.cta_group::" + std::to_string(t.cta_group) + ".sync.aligned.b32 " + taddr_var + ", " +
           std::to_string(t.num_cols) + ";";
}
inline std::string tmem_commit_ptx(const Tmem& t, const std::string& mbar_var) {
    return "tcgen05.commit.cta_group::" + std::to_string(t.cta_group) + ".mbarrier::arrive::one.shared::cluster.b64 [" + mbar_var + "];";
}
inline std::string tmem_commit_mask_ptx(const Tmem& t, const std::string& mbar_var, int cta_mask) {
    return "tcgen05.commit.cta_group::" + std::to_string(t.cta_group) + ".mbarrier::arrive::one.multicast::cluster.shared::cluster.b64 [" +
           mbar_var + "], " + std::to_string(cta_mask) + ";";
}
enum AccumLoc { AccRegisters = 0, AccTensorMem = 1 };
struct TileOp { TiledMma tiled_mma; int accum_loc; bool has_tmem; Tmem tmem; bool double_buf; };
inline TileOp tile_op_make(const TiledMma& tm, int accum_loc, const Tmem* tmem, bool double_buf = false) {
    if (accum_loc == AccTensorMem && !tmem) throw SpecError("TensorMem requires a tmem descriptor");
    return TileOp{tm, accum_loc, tmem != nullptr, tmem ? *tmem : Tmem{1, 0, 0}, double_buf};
}
inline bool tile_op_is_tmem(const TileOp& t) { return t.accum_loc == AccTensorMem; }
inline bool tile_op_is_wgmma(const TileOp& t) { return mma_atom_is_wgmma(t.tiled_mma.atom); }
inline i64 tile_op_accum_elems_per_thread(const TileOp& t) { return tiled_mma_partition_c(t.tiled_mma); }
inline std::string tile_op_emit_mma(const TileOp& t, const std::string& a_desc, const std::string& b_desc, bool enable_accum) {
    if (t.accum_loc == AccRegisters)
        return "mma.sync.aligned." + mma_atom_emit_cpp(t.tiled_mma.atom) + " acc, " + a_desc + ", " + b_desc + ", acc;";
    return "tcgen05.mma.cta_group::" + std::to_string(t.has_tmem ? t.tmem.cta_group : 1) + ".kind::mxf16 [tmem_addr], " +
           a_desc + ", " + b_desc + ", [i_desc], " + (enable_accum ? "1" : "0") + ";";
}
inline std::string tile_op_emit_commit(const TileOp& t, const std::string& mbar_var, int cta_mask) {
    if (t.accum_loc == AccRegisters || !t.has_tmem) return "";
    return cta_mask > 1 ? tmem_commit_mask_ptx(t.tmem, mbar_var, cta_mask) : tmem_commit_ptx(t.tmem, mbar_var);
}
inline std::string tile_op_emit_accum_decl(const TileOp& t, const std::string& var) {
    if (t.accum_loc == AccTensorMem) return "";
    const i64 n = tile_op_accum_elems_per_thread(t);
    std::string zeros;
    for (i64 i = 0; i < n; ++i) zeros += (i ? ", 0.0f" : "0.0f");
    return "float " + var + "[" + std::to_string(n) + "] = {" + zeros + "};";
}
inline std::string tile_op_emit_tmem_alloc(const TileOp& t, const std::string& smem_var) { return t.has_tmem ? tmem_alloc_ptx(t.tmem, smem_var) : ""; }
inline std::string tile_op_emit_tmem_dealloc(const TileOp& t, const std::string& taddr_var) { return t.has_tmem ? tmem_dealloc_ptx(t.tmem, taddr_var) : ""; }
// ---------------------------------------------------------------- Tile_io (lib/pipeline/tile_io.ml:19-127)
// The third tag is the reference's SM100 strategy (its name there is "TMA multicast"); here it means
// "CTA pair, each CTA loads its own rows of A and its own half of B", which moves the same bytes.
enum Strategy { CpAsync = 0, TmaLoad = 1, TmaPair = 2 };
inline i64 tile_bytes_of(int elem, i64 rows, i64 bk) { return rows * bk * elem_bits(elem) / 8; }
inline i64 bytes_per_load_a(int elem, int bm, int bk) { return tile_bytes_of(elem, bm, bk); }
inline i64 bytes_per_load_b(int elem, int bn, int bk, int cta_group) {
    return tile_bytes_of(elem, cta_group == 2 ? bn / 2 : bn, bk);
}
inline i64 expect_tx(int elem, int strategy, int bm, int bn, int bk) {
    return tile_bytes_of(elem, bm + (strategy == TmaPair ? bn / 2 : bn), bk);
}

// ---------------------------------------------------------------- Predicate (lib/pipeline/predicate.ml:9-41)
inline i64 predicate_count_valid(const Ints& shape, const Ints& bounds) {
    if (bounds.size() != shape.size()) throw SpecError("bounds length must match layout rank");
    i64 n = 1, count = 0;
    for (i64 s : shape) n *= s;
    for (i64 k = 0; k < n; ++k) {
        i64 rem = k; bool ok = true;
        for (size_t i = 0; i < shape.size(); ++i) { if (rem % shape[i] >= bounds[i]) ok = false; rem /= shape[i]; }
        count += ok;
    }
    return count;
}
inline Ints predicate_residue(const Ints& shape, const Ints& bounds) {
    if (bounds.size() != shape.size()) throw SpecError("bounds length must match layout rank");
    Ints r(shape.size());
    for (size_t i = 0; i < shape.size(); ++i) r[i] = bounds[i] % shape[i];
    return r;
}

// ---------------------------------------------------------------- Kernel_desc (lib/kernel/kernel_desc.ml:12-248)
enum Family { Ampere = 0, Hopper = 1, Blackwell = 2 };
struct KernelDesc {
    int family = Blackwell;
    std::string name;
    int bm = 0, bn = 0, bk = 0, elem = BF16;
    Swizzle swizzle;
    Cluster cluster{1, 1, 1, 1, {}};
    Pipeline pipeline{1, 1, 1};
    int strategy = TmaPair;
    int copy_bulk_bytes = 128, copy_vec = 0;
    MmaAtom atom = sm100_128x128x16();
    Tmem tmem{2, 512, 128};
    bool double_buf = true;
    Ints pred_a_bounds, pred_b_bounds, pred_c_bounds;
    int sm_count = 148;
    i64 m = 0, n = 0, k = 0;
};

// Kernel_desc.make_blackwell (lib/kernel/kernel_desc.ml:118-162)
inline KernelDesc make_blackwell(const std::string& name, int bm, int bn, int bk, int elem, i64 m, i64 n, i64 k) {
    KernelDesc d;
    d.family = Blackwell; d.name = name; d.bm = bm; d.bn = bn; d.bk = bk; d.elem = elem;
    d.swizzle = swizzle_smem_selector(elem, bm, bk);
    d.cluster = cluster_make(2, 1, 1, 6, {{0, Producer}, {1, Consumer}, {2, Epilogue}, {3, Epilogue},
                                          {4, Epilogue}, {5, Scheduler}});
    d.pipeline = pipeline_make(4, tile_bytes_of(elem, i64(bm) + bn, bk));
    d.strategy = TmaPair;
    if (!is_2sm(d.cluster)) throw SpecError("TmaPair requires a 2SM cluster");
    d.copy_bulk_bytes = 128;
    d.copy_vec = 128 * 8 / elem_bits(elem);
    d.atom = sm100_128x128x16();
    d.tmem = tmem_make(2, 512, bm);
    d.double_buf = true;
    d.pred_a_bounds = {m, k}; d.pred_b_bounds = {k, n}; d.pred_c_bounds = {m, n};
    d.sm_count = 148;
    d.m = m; d.n = n; d.k = k;
    return d;
}
inline i64 smem_bytes(const KernelDesc& d) { return d.pipeline.smem_bytes; }
// Kernel_desc.validate (lib/kernel/kernel_desc.ml:167-190): "" when Ok, else the Error text.
inline std::string validate(const KernelDesc& d) {
    auto pow2 = [](i64 x) { return x > 0 && (x & (x - 1)) == 0; };
    if (!(pow2(d.bm) && pow2(d.bn) && pow2(d.bk)))
        return "Matrix dimensions (bm, bn, bk) must be positive powers of 2";
    if (d.bm % d.atom.m != 0 || d.bn % d.atom.n != 0 || d.bk % d.atom.k != 0)
        return "Tile dimensions must be divisible by atoms: M=" + std::to_string(d.atom.m) +
               ", N=" + std::to_string(d.atom.n) + ", K=" + std::to_string(d.atom.k);
    if (smem_bytes(d) > i64(d.sm_count) * 227 * 1024)
        return "Total pipeline shared memory exceeds the limit of sm_count * 227KB";
    if (d.family == Blackwell && !is_2sm(d.cluster)) return "Blackwell requires 2SM cluster";
    return "";
}
// Kernel_desc.arithmetic_intensity (lib/kernel/kernel_desc.ml:193-202)
inline double arithmetic_intensity(const KernelDesc& d) {
    const int eff_bn = d.family == Blackwell ? d.bn / 2 : d.bn;
    return 2.0 * double(d.bm) * double(d.bn) * double(d.bk) /
           double(tile_bytes_of(d.elem, i64(d.bm) + eff_bn, d.bk));
}

// ---------------------------------------------------------------- Lower (lib/kernel/lower.ml:25-104)
enum Arch { SM80 = 0, SM90 = 1, SM100 = 2 };
enum LowerError { LowerOk = 0, UnsupportedArch = 1, UnsupportedElem = 2, IncompatibleTile = 3, MissingArg = 4,
                  InvalidPipeline = 5 };
inline const char* arch_name(int a) { return a == SM80 ? "SM80" : a == SM90 ? "SM90" : a == SM100 ? "SM100" : "?"; }
inline const char* elem_name(int e) {
    switch (e) { case F16: return "F16"; case BF16: return "BF16"; case F32: return "F32"; case S8: return "S8";
                 case S32: return "S32"; case F8E4M3: return "F8E4M3"; case F4E2M1: return "F4E2M1"; default: return "?"; }
}
// Problem dims are invented as 32 tiles per mode (lib/kernel/lower.ml:36-43); only SM100 is
// built here, so SM80/SM90 specs report UnsupportedArch instead of an Ampere/Hopper descriptor.
inline int lower(const std::string& name, int arch, int elem, int bm, int bn, int bk, KernelDesc* out, std::string* msg) {
    if (arch != SM100) {
        if (msg) *msg = std::string("UnsupportedArch: ") + arch_name(arch) + " (this backend emits sm_100a only)";
        return UnsupportedArch;
    }
    if (!(elem == F16 || elem == BF16 || elem == S8 || elem == F8E4M3 || elem == F4E2M1)) {
        if (msg) *msg = std::string("UnsupportedElem: arch=") + arch_name(arch) + " elem=" + elem_name(elem);
        return UnsupportedElem;
    }
    *out = make_blackwell(name, bm, bn, bk, elem, i64(bm) * 32, i64(bn) * 32, i64(bk) * 32);
    return LowerOk;
}

}  // namespace tesserae::spec
