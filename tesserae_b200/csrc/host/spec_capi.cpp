// C ABI over the integer descriptor model (csrc/spec/tesserae_spec.hpp).  Where the
// reference raises, these return -1 and leave the reference's message in
// tesserae_last_error().
#include "../../../include/tesserae_b200.h"
#include "../rt/errors.hpp"
#include "../spec/tesserae_spec.hpp"

#include <cstring>

namespace sp = tesserae::spec;
using tesserae::fail;

namespace {
sp::Layout mk(const int64_t* shape, const int64_t* stride, int n) {
    return sp::Layout(sp::Ints(shape, shape + n), sp::Ints(stride, stride + n));
}
int put(const sp::Layout& l, int64_t* os, int64_t* od) {
    for (size_t i = 0; i < l.shape.size(); ++i) { if (os) os[i] = l.shape[i]; if (od) od[i] = l.stride[i]; }
    return (int)l.shape.size();
}
}  // namespace

#define TS_GUARD(expr)                                             \
    try { expr; } catch (const std::exception& e) { return fail(e.what()); }

extern "C" {

int64_t tesserae_swizzle_apply(int b, int m, int s, int64_t offset) {
    TS_GUARD(return sp::swizzle_apply(sp::swizzle_make(b, m, s), offset));
}
int tesserae_swizzle_apply_to_strides(int b, int m, int s, const int64_t* stride, int n, int64_t* out_stride) {
    if (!stride || !out_stride || n < 0) return fail("swizzle_apply_to_strides: null argument");
    try {
        const sp::Swizzle sw = sp::swizzle_make(b, m, s);
        for (int i = 0; i < n; ++i) out_stride[i] = sp::swizzle_apply(sw, stride[i]);
        return 0;
    } catch (const std::exception& e) { return fail(e.what()); }
}
int tesserae_swizzle_smem_selector(int elem, int tile_m, int tile_k, int* b, int* m, int* s) {
    TS_GUARD({
        sp::Swizzle sw = sp::swizzle_smem_selector(elem, tile_m, tile_k);
        if (b) *b = sw.b; if (m) *m = sw.m; if (s) *s = sw.s;
        return 0;
    });
}
int tesserae_elem_byte_width(int elem) { return sp::elem_byte_width(elem); }
int tesserae_elem_bits(int elem) { return sp::elem_bits(elem); }
int tesserae_elem_vec_width(int elem) { return sp::elem_vec_width(elem); }

int64_t tesserae_layout_size(const int64_t* shape, int n) {
    int64_t p = 1;
    for (int i = 0; i < n; ++i) p *= shape[i];
    return p;
}
int64_t tesserae_layout_cosize(const int64_t* shape, const int64_t* stride, int n) {
    TS_GUARD(return sp::cosize(mk(shape, stride, n)));
}
int64_t tesserae_layout_idx(const int64_t* stride, const int64_t* coord, int n) {
    int64_t o = 0;
    for (int i = 0; i < n; ++i) o += coord[i] * stride[i];
    return o;
}
int tesserae_layout_compose(const int64_t* outer_shape, const int64_t* outer_stride, int n_outer,
                            const int64_t* inner_shape, const int64_t* inner_stride, int n_inner,
                            int64_t* out_stride) {
    TS_GUARD({
        sp::Layout r = sp::compose(mk(outer_shape, outer_stride, n_outer), mk(inner_shape, inner_stride, n_inner));
        return put(r, nullptr, out_stride);
    });
}
int tesserae_layout_tile(const int64_t* shape, const int64_t* stride, int n, const int64_t* tile,
                         int64_t* out_shape, int64_t* out_stride) {
    TS_GUARD(return put(sp::tile(mk(shape, stride, n), sp::Ints(tile, tile + n)), out_shape, out_stride));
}
int tesserae_layout_sort(const int64_t* shape, const int64_t* stride, int n, int64_t* out_shape, int64_t* out_stride) {
    TS_GUARD(return put(sp::sort_by_stride(mk(shape, stride, n)), out_shape, out_stride));
}
int tesserae_layout_coalesce(const int64_t* shape, const int64_t* stride, int n, int64_t* out_shape, int64_t* out_stride) {
    TS_GUARD(return put(sp::coalesce(mk(shape, stride, n)), out_shape, out_stride));
}
int tesserae_layout_is_admissible(const int64_t* shape, const int64_t* stride, int n, int64_t m) {
    TS_GUARD(return sp::is_admissible(mk(shape, stride, n), m) ? 1 : 0);
}
int tesserae_layout_complement(const int64_t* shape, const int64_t* stride, int n, int64_t m,
                               int64_t* out_shape, int64_t* out_stride) {
    TS_GUARD(return put(sp::complement(mk(shape, stride, n), m), out_shape, out_stride));
}
int tesserae_layout_flat_divide(const int64_t* shape, const int64_t* stride, int n, int64_t divisor,
                                int64_t* out_shape, int64_t* out_stride) {
    TS_GUARD(return put(sp::flat_divide(mk(shape, stride, n), divisor), out_shape, out_stride));
}
int tesserae_layout_logical_divide(const int64_t* shape, const int64_t* stride, int n, const int64_t* tile_shape,
                                   int64_t* out_shape, int64_t* out_stride) {
    TS_GUARD(return put(sp::logical_divide(mk(shape, stride, n), sp::Ints(tile_shape, tile_shape + n)), out_shape, out_stride));
}

int64_t tesserae_pipeline_smem_bytes(int depth, int64_t tile_bytes) {
    TS_GUARD(return sp::pipeline_make(depth, tile_bytes).smem_bytes);
}
int tesserae_pipeline_stage_of(int64_t iter, int depth) { return depth > 0 ? sp::stage_of(iter, depth) : fail("depth must be > 0"); }
int tesserae_pipeline_phase_of(int64_t iter, int depth) { return depth > 0 ? sp::phase_of(iter, depth) : fail("depth must be > 0"); }
int64_t tesserae_pipeline_smem_offset_of(int64_t tile_bytes, int stage) { return sp::smem_offset_of(tile_bytes, stage); }
int64_t tesserae_pipeline_b_smem_offset_of(int64_t tile_bytes, int stage, int bm, int bk, int elem_bytes) {
    return sp::b_smem_offset_of(tile_bytes, stage, bm, bk, elem_bytes);
}

int tesserae_tmem_validate(int cta_group, int num_cols, int num_rows) {
    TS_GUARD({ sp::tmem_make(cta_group, num_cols, num_rows); return 0; });
}
int64_t tesserae_tmem_address(int row, int col) { return sp::tmem_address(row, col); }
int tesserae_tmem_warp_row_offset(int warp_id) { return sp::tmem_warp_row_offset(warp_id); }
int tesserae_tmem_num_loads_per_warp(int num_cols) { return sp::tmem_num_loads_per_warp(num_cols); }
int tesserae_tmem_buf_col_offset(int buf_id) { return sp::tmem_buf_col_offset(buf_id); }

int64_t tesserae_smem_desc_encode(int64_t base_addr, int64_t leading_off, int64_t stride_off, int swizzle_mode_bits) {
    return sp::smem_desc_encode(base_addr, leading_off, stride_off, swizzle_mode_bits);
}
uint64_t tesserae_umma_smem_desc(uint32_t smem_addr, int swizzle_b) {
    if (swizzle_b < 0 || swizzle_b > 3) { fail("swizzle_b must be 0..3"); return 0; }
    return sp::umma_smem_desc(smem_addr, swizzle_b);
}
uint32_t tesserae_umma_instr_desc(int elem, int umma_m, int umma_n) {
    try { return sp::umma_instr_desc(elem, umma_m, umma_n); }
    catch (const std::exception& e) { fail(e.what()); return 0; }
}

int64_t tesserae_tile_io_bytes_a(int elem, int bm, int bk) { return sp::bytes_per_load_a(elem, bm, bk); }
int64_t tesserae_tile_io_bytes_b(int elem, int bn, int bk, int cta_group) { return sp::bytes_per_load_b(elem, bn, bk, cta_group); }
int64_t tesserae_tile_io_expect_tx(int elem, int strategy, int bm, int bn, int bk) { return sp::expect_tx(elem, strategy, bm, bn, bk); }

int64_t tesserae_predicate_count_valid(const int64_t* shape, const int64_t* bounds, int n) {
    TS_GUARD(return sp::predicate_count_valid(sp::Ints(shape, shape + n), sp::Ints(bounds, bounds + n)));
}
int tesserae_predicate_residue(const int64_t* shape, const int64_t* bounds, int n, int64_t* out) {
    TS_GUARD({
        sp::Ints r = sp::predicate_residue(sp::Ints(shape, shape + n), sp::Ints(bounds, bounds + n));
        for (int i = 0; i < n; ++i) out[i] = r[i];
        return 0;
    });
}

// ------------------------------------------------------------------ Memspace / atoms / Tiled_* / Tile_op
static int put_string(const std::string& s, char* buf, size_t buf_size) {
    if (!buf || buf_size == 0) return fail("output buffer is null");
    if (s.size() + 1 > buf_size) return fail("output buffer too small: need " + std::to_string(s.size() + 1) + " bytes");
    std::memcpy(buf, s.c_str(), s.size() + 1);
    return 0;
}
static sp::MmaAtom atom_from_c(const tesserae_mma_atom* a) {
    sp::MmaAtom r;
    r.arch = a->arch; r.m = a->m; r.n = a->n; r.k = a->k;
    r.a_type = a->a_type; r.b_type = a->b_type; r.c_type = a->c_type; r.d_type = a->d_type;
    r.a_major = a->a_major; r.b_major = a->b_major;
    r.threads = sp::mma_atom_thread_count(r);
    return r;
}
static sp::CopyAtom copy_from_c(const tesserae_copy_atom* a) {
    return sp::CopyAtom{a->kind, a->src_space, a->dst_space, a->elem, a->vec_width, a->bulk_bytes};
}
static sp::TileOp tile_op_from_c(const tesserae_tile_op* t) {
    sp::TiledMma tm = sp::tiled_mma_make(atom_from_c(&t->atom), t->thread_layout_size, t->warp_layout_size, t->tiler_m, t->tiler_n);
    sp::Tmem tmem{t->tmem_cta_group, t->tmem_cols, t->tmem_rows};
    return sp::tile_op_make(tm, t->accum_loc, t->has_tmem ? &tmem : nullptr, t->double_buf != 0);
}

int tesserae_memspace_can_transfer(int src, int dst) { return sp::memspace_can_transfer(src, dst) ? 1 : 0; }
const char* tesserae_memspace_name(int space) { return sp::memspace_name(space); }

int tesserae_mma_atom_make(int which, int a_major, int b_major, tesserae_mma_atom* out) {
    if (!out) return fail("mma_atom_make: null output");
    TS_GUARD({
        const sp::MmaAtom a = sp::mma_atom_make(which, a_major, b_major);
        out->arch = a.arch; out->m = a.m; out->n = a.n; out->k = a.k;
        out->a_type = a.a_type; out->b_type = a.b_type; out->c_type = a.c_type; out->d_type = a.d_type;
        out->a_major = a.a_major; out->b_major = a.b_major;
        return 0;
    });
}
int tesserae_mma_atom_thread_count(const tesserae_mma_atom* a) { return a ? sp::mma_atom_thread_count(atom_from_c(a)) : -1; }
int tesserae_mma_atom_is_wgmma(const tesserae_mma_atom* a) { return a ? (sp::mma_atom_is_wgmma(atom_from_c(a)) ? 1 : 0) : -1; }
int tesserae_mma_atom_emit_cpp(const tesserae_mma_atom* a, char* buf, size_t buf_size) {
    if (!a) return fail("mma_atom_emit_cpp: null atom");
    return put_string(sp::mma_atom_emit_cpp(atom_from_c(a)), buf, buf_size);
}

int tesserae_copy_atom_make(int kind, int elem, int src_space, int dst_space, tesserae_copy_atom* out) {
    if (!out) return fail("copy_atom_make: null output");
    TS_GUARD({
        const sp::CopyAtom a = sp::copy_atom_make(kind, elem, src_space, dst_space);
        out->kind = a.kind; out->src_space = a.src_space; out->dst_space = a.dst_space; out->elem = a.elem;
        out->vec_width = a.vec_width; out->bulk_bytes = a.bulk_bytes;
        return 0;
    });
}
int tesserae_copy_atom_is_async(const tesserae_copy_atom* a) { return a ? (sp::copy_atom_is_async(copy_from_c(a)) ? 1 : 0) : -1; }
int tesserae_copy_atom_is_tma(const tesserae_copy_atom* a) { return a ? (sp::copy_atom_is_tma(copy_from_c(a)) ? 1 : 0) : -1; }
int tesserae_copy_atom_requires_mbar(const tesserae_copy_atom* a) { return a ? (sp::copy_atom_requires_mbar(copy_from_c(a)) ? 1 : 0) : -1; }
int tesserae_copy_atom_emit_cpp(const tesserae_copy_atom* a, char* buf, size_t buf_size) {
    if (!a) return fail("copy_atom_emit_cpp: null atom");
    return put_string(sp::copy_atom_emit_cpp(copy_from_c(a)), buf, buf_size);
}

int tesserae_tiled_mma_make(const tesserae_mma_atom* atom, int64_t thread_layout_size, int64_t warp_layout_size,
                            int64_t tiler_m, int64_t tiler_n, tesserae_tiled_mma* out) {
    if (!atom || !out) return fail("tiled_mma_make: null argument");
    TS_GUARD({
        const sp::TiledMma t = sp::tiled_mma_make(atom_from_c(atom), thread_layout_size, warp_layout_size, tiler_m, tiler_n);
        out->thread_count = sp::tiled_mma_thread_count(t);
        out->warp_count = sp::tiled_mma_warp_count(t);
        out->tile_m = t.tiler_m; out->tile_n = t.tiler_n; out->tile_k = t.atom.k;
        out->partition_a = sp::tiled_mma_partition_a(t);
        out->partition_b = sp::tiled_mma_partition_b(t);
        out->partition_c = sp::tiled_mma_partition_c(t);
        return 0;
    });
}

int tesserae_tiled_copy_make(const tesserae_copy_atom* atom, int64_t thread_layout_size, int64_t val_layout_size,
                             tesserae_tiled_copy* out) {
    if (!atom || !out) return fail("tiled_copy_make: null argument");
    TS_GUARD({
        const sp::TiledCopy t = sp::tiled_copy_make(copy_from_c(atom), thread_layout_size, val_layout_size);
        out->thread_count = t.thread_layout_size;
        out->elements_per_thread = t.val_layout_size;
        out->tile_size = sp::tiled_copy_tile_size(t);
        out->is_tma = sp::copy_atom_is_tma(t.atom) ? 1 : 0;
        out->requires_mbar = sp::copy_atom_requires_mbar(t.atom) ? 1 : 0;
        return 0;
    });
}
int tesserae_tiled_copy_partition(int64_t thread_count, const int64_t* shape, const int64_t* stride, int n,
                                  int64_t* out_shape, int64_t* out_stride) {
    TS_GUARD({
        const sp::Layout d = sp::flat_divide(mk(shape, stride, n), thread_count);
        if (out_shape) *out_shape = d.shape[1];
        if (out_stride) *out_stride = d.stride[1];
        return 1;
    });
}

int tesserae_tile_op_check(const tesserae_tile_op* t) {
    if (!t) return fail("tile_op_check: null argument");
    TS_GUARD({ (void)tile_op_from_c(t); return 0; });
}
int tesserae_tile_op_is_tmem(const tesserae_tile_op* t) { TS_GUARD(return t ? (sp::tile_op_is_tmem(tile_op_from_c(t)) ? 1 : 0) : -1); }
int tesserae_tile_op_is_wgmma(const tesserae_tile_op* t) { TS_GUARD(return t ? (sp::tile_op_is_wgmma(tile_op_from_c(t)) ? 1 : 0) : -1); }
int64_t tesserae_tile_op_accum_elems_per_thread(const tesserae_tile_op* t) {
    TS_GUARD(return t ? sp::tile_op_accum_elems_per_thread(tile_op_from_c(t)) : -1);
}
int tesserae_tile_op_emit(const tesserae_tile_op* t, int what, const char* arg0, const char* arg1, int flag,
                          char* buf, size_t buf_size) {
    if (!t) return fail("tile_op_emit: null argument");
    const std::string a0 = arg0 ? arg0 : "", a1 = arg1 ? arg1 : "";
    TS_GUARD({
        const sp::TileOp op = tile_op_from_c(t);
        switch (what) {
            case TESSERAE_TILE_OP_MMA: return put_string(sp::tile_op_emit_mma(op, a0, a1, flag != 0), buf, buf_size);
            case TESSERAE_TILE_OP_COMMIT: return put_string(sp::tile_op_emit_commit(op, a0, flag), buf, buf_size);
            case TESSERAE_TILE_OP_ACCUM_DECL: return put_string(sp::tile_op_emit_accum_decl(op, a0), buf, buf_size);
            case TESSERAE_TILE_OP_TMEM_ALLOC: return put_string(sp::tile_op_emit_tmem_alloc(op, a0), buf, buf_size);
            case TESSERAE_TILE_OP_TMEM_DEALLOC: return put_string(sp::tile_op_emit_tmem_dealloc(op, a0), buf, buf_size);
            default: return fail("tile_op_emit: unknown text selector");
        }
    });
}

// Shard `index` of `parts` over [0, total): contiguous ranges whose boundaries are multiples of `align`
// (the last range takes the remainder).  N-split shards align to 128 columns so that no 128x128 weight
// scale block or 128-row scale chunk straddles two GPUs; K-split shards align to one smem stage.
int tesserae_shard_range(int64_t total, int parts, int index, int64_t align, int64_t* begin, int64_t* length) {
    if (total < 0 || parts < 1 || index < 0 || index >= parts || align < 1) return fail("shard_range: bad argument");
    const int64_t units = (total + align - 1) / align;
    const int64_t base = units / parts, extra = units % parts;
    const int64_t u0 = base * index + (index < extra ? index : extra);
    const int64_t un = base + (index < extra ? 1 : 0);
    int64_t b = u0 * align, e = (u0 + un) * align;
    if (b > total) b = total;
    if (e > total) e = total;
    if (begin) *begin = b;
    if (length) *length = e - b;
    return 0;
}

}  // extern "C"
