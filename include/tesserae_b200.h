/* tesserae_b200 — C ABI of the B200-native backend/runtime for tesserae's dense GEMM path.
 *
 * Every entry point is plain C (pointers, sizes, ints).  It is the symbol set that the
 * OCaml `external`s of the reference bind to, re-stated one level below the OCaml
 * runtime: each `caml_*` stub of the reference becomes a thin wrapper over the
 * `tesserae_*` function of the same name declared here (the reference already uses that
 * split for NVRTC, lib/runtime/nvrtc_stub.h:23-55).  Paths cited below are relative to
 * the reference project root.
 *
 * Conventions: functions returning int return 0 on success and non-zero on failure;
 * tesserae_last_error() then holds a message for the calling thread (the reference
 * turns the same messages into OCaml `Failure`, lib/kernel/kernel_launch_stubs.c:8-19).
 * Nothing aborts the process.  Device pointers are raw CUDA device addresses.  Streams
 * are CUstream/cudaStream_t handles passed as void* (NULL = default stream).
 * There is no CPU fallback anywhere: GPU entry points fail on a machine without a
 * CUDA driver.
 */
#ifndef TESSERAE_B200_H
#define TESSERAE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ errors */
const char* tesserae_last_error(void);
/* Library version string, e.g. "tesserae_b200 0.1 (sm_100a)". */
const char* tesserae_version(void);

/* ------------------------------------------------------------------ enums */
/* Kernel_ast.arch (lib/kernel/kernel_ast.ml:3-6) */
enum { TESSERAE_SM80 = 0, TESSERAE_SM90 = 1, TESSERAE_SM100 = 2 };
/* Kernel_ast.elem (lib/kernel/kernel_ast.ml:8-13) = Elemtype.t (lib/core/elemtype.ml:9-14),
 * extended with the two narrow float formats the reference lacks. */
enum {
    TESSERAE_F16 = 0, TESSERAE_BF16 = 1, TESSERAE_F32 = 2, TESSERAE_S8 = 3, TESSERAE_S32 = 4,
    TESSERAE_F8E4M3 = 5, TESSERAE_F4E2M1 = 6
};
/* Kernel_desc.family (lib/kernel/kernel_desc.ml:7-10) */
enum { TESSERAE_AMPERE = 0, TESSERAE_HOPPER = 1, TESSERAE_BLACKWELL = 2 };
/* Tile_io.strategy (lib/pipeline/tile_io.ml:5-8).  TMA_PAIR stands for the reference's third tag (its SM100
 * strategy): a CTA pair in which each CTA loads its own rows of A and its own half of the B tile. */
enum { TESSERAE_CP_ASYNC = 0, TESSERAE_TMA_LOAD = 1, TESSERAE_TMA_PAIR = 2 };
/* Cluster.warp_role (lib/pipeline/cluster.ml:9-13); -1 = no role */
enum { TESSERAE_ROLE_PRODUCER = 0, TESSERAE_ROLE_CONSUMER = 1, TESSERAE_ROLE_EPILOGUE = 2, TESSERAE_ROLE_SCHEDULER = 3 };
/* Lower.error (lib/kernel/lower.ml:11-16); returned by tesserae_lower */
enum {
    TESSERAE_LOWER_OK = 0, TESSERAE_LOWER_UNSUPPORTED_ARCH = 1, TESSERAE_LOWER_UNSUPPORTED_ELEM = 2,
    TESSERAE_LOWER_INCOMPATIBLE_TILE = 3, TESSERAE_LOWER_MISSING_ARG = 4, TESSERAE_LOWER_INVALID_PIPELINE = 5
};
/* Scaling of the operands (new surface; the reference has no scale-factor concept). */
enum {
    TESSERAE_SCALE_NONE = 0,
    TESSERAE_SCALE_FP8_BLOCK = 1,  /* A: fp32 per 1x128 (row, K-block); B: fp32 per 128x128 block */
    TESSERAE_SCALE_NVFP4 = 2       /* UE4M3 per 16 K-elements + one fp32 per tensor */
};

/* ------------------------------------------------------------------ integer layout maps
 * Bit-exact restatements of the reference's CPU-evaluable functions.  Shapes, strides and
 * coordinates are passed flattened (the reference flattens before every computation,
 * lib/core/layout.ml:17-32).  Functions that the reference makes raise return -1 and set
 * tesserae_last_error() to the reference's exception message. */

/* Swizzle.apply (lib/core/swizzle.ml:15-17): x ^ ((x & (((1<<b)-1) << (m+s))) >> s) */
int64_t tesserae_swizzle_apply(int b, int m, int s, int64_t offset);
/* Swizzle.apply_to_layout (lib/core/swizzle.ml:36-43): the swizzle applied to every stride leaf (flattened, n leaves);
 * shapes are unchanged.  Returns 0, or -1 on a negative parameter. */
int tesserae_swizzle_apply_to_strides(int b, int m, int s, const int64_t* stride, int n, int64_t* out_stride);
/* Swizzle.smem_selector (lib/core/swizzle.ml:46-56); writes b,m,s */
int tesserae_swizzle_smem_selector(int elem, int tile_m, int tile_k, int* b, int* m, int* s);
/* Elemtype.byte_width / bits / vec_width (lib/core/elemtype.ml:24-57); -1 for a bad code.
 * F4E2M1 reports 0 bytes, 4 bits. */
int tesserae_elem_byte_width(int elem);
int tesserae_elem_bits(int elem);
int tesserae_elem_vec_width(int elem);
/* Layout.size / cosize / idx (lib/core/layout.ml:15-32) */
int64_t tesserae_layout_size(const int64_t* shape, int n);
int64_t tesserae_layout_cosize(const int64_t* shape, const int64_t* stride, int n);
int64_t tesserae_layout_idx(const int64_t* stride, const int64_t* coord, int n);
/* Compose.compose (lib/core/compose.ml:3-21): result has the inner layout's flat shape;
 * writes n_inner strides. */
int tesserae_layout_compose(const int64_t* outer_shape, const int64_t* outer_stride, int n_outer,
                            const int64_t* inner_shape, const int64_t* inner_stride, int n_inner,
                            int64_t* out_stride);
/* Compose.tile (lib/core/compose.ml:24-47): out_* get 2n entries, the n "within" modes
 * then the n "across" modes. */
int tesserae_layout_tile(const int64_t* shape, const int64_t* stride, int n, const int64_t* tile,
                         int64_t* out_shape, int64_t* out_stride);
/* Algebra.sort / coalesce / is_admissible / complement / flat_divide
 * (lib/core/algebra.ml:6-112).  Output arrays hold at least n+1 entries; the functions
 * return the number of output modes (or -1). */
int tesserae_layout_sort(const int64_t* shape, const int64_t* stride, int n, int64_t* out_shape, int64_t* out_stride);
int tesserae_layout_coalesce(const int64_t* shape, const int64_t* stride, int n, int64_t* out_shape, int64_t* out_stride);
int tesserae_layout_is_admissible(const int64_t* shape, const int64_t* stride, int n, int64_t m);
int tesserae_layout_complement(const int64_t* shape, const int64_t* stride, int n, int64_t m,
                               int64_t* out_shape, int64_t* out_stride);
int tesserae_layout_flat_divide(const int64_t* shape, const int64_t* stride, int n, int64_t divisor,
                                int64_t* out_shape, int64_t* out_stride);
/* Algebra.logical_divide (lib/core/algebra.ml:114-120): divisibility check, then Compose.tile */
int tesserae_layout_logical_divide(const int64_t* shape, const int64_t* stride, int n, const int64_t* tile_shape,
                                   int64_t* out_shape, int64_t* out_stride);
/* Pipeline (lib/pipeline/pipeline.ml:9-31) */
int64_t tesserae_pipeline_smem_bytes(int depth, int64_t tile_bytes);
int tesserae_pipeline_stage_of(int64_t iter, int depth);
int tesserae_pipeline_phase_of(int64_t iter, int depth);
int64_t tesserae_pipeline_smem_offset_of(int64_t tile_bytes, int stage);
int64_t tesserae_pipeline_b_smem_offset_of(int64_t tile_bytes, int stage, int bm, int bk, int elem_bytes);
/* Tmem (lib/pipeline/tmem.ml:24-110) */
int tesserae_tmem_validate(int cta_group, int num_cols, int num_rows);
int64_t tesserae_tmem_address(int row, int col);
int tesserae_tmem_warp_row_offset(int warp_id);
int tesserae_tmem_num_loads_per_warp(int num_cols);
int tesserae_tmem_buf_col_offset(int buf_id);
/* Smem_desc.encode (lib/pipeline/smem_desc.ml:38-43): the reference's packing, kept
 * bit-exact; it is not the sm_100 hardware descriptor (tesserae_umma_smem_desc is). */
int64_t tesserae_smem_desc_encode(int64_t base_addr, int64_t leading_off, int64_t stride_off, int swizzle_mode_bits);
/* Hardware descriptors the kernels use (new): shared-memory matrix descriptor of a
 * K-major tile with 128-byte rows under `swizzle_b` (0..3), and the 32-bit instruction
 * descriptor of a dense MMA. */
uint64_t tesserae_umma_smem_desc(uint32_t smem_addr, int swizzle_b);
uint32_t tesserae_umma_instr_desc(int elem, int umma_m, int umma_n);
/* Tile_io byte counts (lib/pipeline/tile_io.ml:75-87,119-127) */
int64_t tesserae_tile_io_bytes_a(int elem, int bm, int bk);
int64_t tesserae_tile_io_bytes_b(int elem, int bn, int bk, int cta_group);
int64_t tesserae_tile_io_expect_tx(int elem, int strategy, int bm, int bn, int bk);
/* Predicate.count_valid / residue (lib/pipeline/predicate.ml:21-41) over a flat shape */
int64_t tesserae_predicate_count_valid(const int64_t* shape, const int64_t* bounds, int n);
int tesserae_predicate_residue(const int64_t* shape, const int64_t* bounds, int n, int64_t* out);

/* ------------------------------------------------------------------ Memspace, atoms, tiled atoms, Tile_op
 * Plain-integer restatements of lib/core/memspace.ml, lib/atoms/{mma_atom,copy_atom,tiled_mma,tiled_copy}.ml and
 * lib/pipeline/tile_op.ml.  The reference's phantom types (arch, element, memory space) become integer codes. */
/* Memspace.space (lib/core/memspace.ml:8-12) */
enum { TESSERAE_SPACE_GLOBAL = 0, TESSERAE_SPACE_SHARED = 1, TESSERAE_SPACE_REGISTER = 2, TESSERAE_SPACE_TENSOR = 3 };
/* Memspace.can_transfer (lib/core/memspace.ml:26-47): 1 / 0 */
int tesserae_memspace_can_transfer(int src_space, int dst_space);
/* Memspace.name (lib/core/memspace.ml:14-20) */
const char* tesserae_memspace_name(int space);

/* Mma_atom.t (lib/atoms/mma_atom.ml:17-28); `arch` is a TESSERAE_SM* code, the types are element codes */
enum { TESSERAE_ROW_MAJOR = 0, TESSERAE_COL_MAJOR = 1 };
enum {  /* the reference's atom constructors, lib/atoms/mma_atom.ml:32-112, in file order */
    TESSERAE_MMA_SM80_16x8x8_F32F16F16F32 = 0, TESSERAE_MMA_SM80_16x8x16_F32F16F16F32 = 1,
    TESSERAE_MMA_SM80_16x8x16_F32BF16BF16F32 = 2, TESSERAE_MMA_SM80_16x8x32_S32S8S8S32 = 3,
    TESSERAE_MMA_SM90_64x64x16_F32F16F16F32 = 4, TESSERAE_MMA_SM90_64x128x16_F32F16F16F32 = 5,
    TESSERAE_MMA_SM90_64x64x16_F32BF16BF16F32 = 6, TESSERAE_MMA_SM100_64x64x16_F32F16F16F32 = 7,
    TESSERAE_MMA_SM100_128x128x16_F32F16F16F32 = 8, TESSERAE_MMA_SM100_64x64x32_S32S8S8S32 = 9
};
typedef struct tesserae_mma_atom {
    int arch, m, n, k;
    int a_type, b_type, c_type, d_type;
    int a_major, b_major;
} tesserae_mma_atom;
int tesserae_mma_atom_make(int which, int a_major, int b_major, tesserae_mma_atom* out);
/* Mma_atom.thread_count / is_wgmma / emit_cpp (lib/atoms/mma_atom.ml:118-156) */
int tesserae_mma_atom_thread_count(const tesserae_mma_atom* atom);
int tesserae_mma_atom_is_wgmma(const tesserae_mma_atom* atom);
int tesserae_mma_atom_emit_cpp(const tesserae_mma_atom* atom, char* buf, size_t buf_size);

/* Copy_atom.kind (lib/atoms/copy_atom.ml:4-12).  TMA_LOAD_PAIR is the reference's fifth kind (its SM100
 * cluster-wide TMA load), which this backend lowers to the per-CTA loads of a CTA pair. */
enum {
    TESSERAE_COPY_ASYNC_GLOBAL = 0, TESSERAE_COPY_ASYNC_CACHED = 1, TESSERAE_COPY_TMA_LOAD = 2,
    TESSERAE_COPY_TMA_STORE = 3, TESSERAE_COPY_TMA_LOAD_PAIR = 4, TESSERAE_COPY_LDMATRIX = 5,
    TESSERAE_COPY_LDMATRIX_TRANS = 6, TESSERAE_COPY_UNIVERSAL = 7
};
typedef struct tesserae_copy_atom { int kind, src_space, dst_space, elem, vec_width, bulk_bytes; } tesserae_copy_atom;
/* The reference's constructors (lib/atoms/copy_atom.ml:23-104); src/dst spaces are read for UNIVERSAL only. */
int tesserae_copy_atom_make(int kind, int elem, int src_space, int dst_space, tesserae_copy_atom* out);
/* Copy_atom.is_async / is_tma / requires_mbar / emit_cpp (lib/atoms/copy_atom.ml:106-137) */
int tesserae_copy_atom_is_async(const tesserae_copy_atom* atom);
int tesserae_copy_atom_is_tma(const tesserae_copy_atom* atom);
int tesserae_copy_atom_requires_mbar(const tesserae_copy_atom* atom);
int tesserae_copy_atom_emit_cpp(const tesserae_copy_atom* atom, char* buf, size_t buf_size);

/* Tiled_mma (lib/atoms/tiled_mma.ml:12-53).  The reference reads only the sizes of the thread and warp
 * layouts; partition_a/b/c are the sizes of the `n:1` fragments it returns.  Fails with the reference's
 * message when the thread layout does not match the atom. */
typedef struct tesserae_tiled_mma {
    int64_t thread_count, warp_count;
    int64_t tile_m, tile_n, tile_k;                 /* tile_shape_mnk */
    int64_t partition_a, partition_b, partition_c;
} tesserae_tiled_mma;
int tesserae_tiled_mma_make(const tesserae_mma_atom* atom, int64_t thread_layout_size, int64_t warp_layout_size,
                            int64_t tiler_m, int64_t tiler_n, tesserae_tiled_mma* out);
/* Tiled_copy (lib/atoms/tiled_copy.ml:10-50) */
typedef struct tesserae_tiled_copy {
    int64_t thread_count, elements_per_thread, tile_size;
    int is_tma, requires_mbar;
} tesserae_tiled_copy;
int tesserae_tiled_copy_make(const tesserae_copy_atom* atom, int64_t thread_layout_size, int64_t val_layout_size,
                             tesserae_tiled_copy* out);
/* Tiled_copy.partition_src / partition_dst (lib/atoms/tiled_copy.ml:38-50): Algebra.flat_divide by the thread
 * count, "across" mode kept.  Writes one mode; returns 1 (the mode count) or -1. */
int tesserae_tiled_copy_partition(int64_t thread_count, const int64_t* shape, const int64_t* stride, int n,
                                  int64_t* out_shape, int64_t* out_stride);

/* Tile_op.t (lib/pipeline/tile_op.ml:9-16): a tiled MMA plus where its accumulator lives. */
enum { TESSERAE_ACCUM_REGISTERS = 0, TESSERAE_ACCUM_TENSOR_MEM = 1 };
typedef struct tesserae_tile_op {
    tesserae_mma_atom atom;
    int64_t thread_layout_size, warp_layout_size, tiler_m, tiler_n;
    int accum_loc;                                  /* TESSERAE_ACCUM_* */
    int has_tmem, tmem_cta_group, tmem_cols, tmem_rows;
    int double_buf;
} tesserae_tile_op;
/* Tile_op.make's checks (lib/pipeline/tile_op.ml:18-37): "TensorMem requires a tmem descriptor" */
int tesserae_tile_op_check(const tesserae_tile_op* op);
/* Tile_op.is_tmem / is_wgmma / accum_elems_per_thread (lib/pipeline/tile_op.ml:39-50) */
int tesserae_tile_op_is_tmem(const tesserae_tile_op* op);
int tesserae_tile_op_is_wgmma(const tesserae_tile_op* op);
int64_t tesserae_tile_op_accum_elems_per_thread(const tesserae_tile_op* op);
/* Tile_op.emit_* (lib/pipeline/tile_op.ml:52-107), the reference's instruction text.  `what` selects the
 * emitter; arg0/arg1/flag are (a_desc, b_desc, enable_accum) for MMA, (mbar_var, -, cta_mask) for COMMIT,
 * (var name, -, -) for the rest.  The text is descriptive: the kernels of this library are built from the
 * working PTX wrappers, not from these strings. */
enum { TESSERAE_TILE_OP_MMA = 0, TESSERAE_TILE_OP_COMMIT = 1, TESSERAE_TILE_OP_ACCUM_DECL = 2,
       TESSERAE_TILE_OP_TMEM_ALLOC = 3, TESSERAE_TILE_OP_TMEM_DEALLOC = 4 };
int tesserae_tile_op_emit(const tesserae_tile_op* op, int what, const char* arg0, const char* arg1, int flag,
                          char* buf, size_t buf_size);

/* ------------------------------------------------------------------ kernel spec -> descriptor */
/* Kernel_ast.kernel (lib/kernel/kernel_ast.ml:64-72).  `args` and `body` of the reference
 * record are DSL statements that its lowering never reads (lib/kernel/lower.ml:61-83), so
 * they are not carried.  Fields after `stages` are extensions; 0 selects the reference's
 * behaviour (CTA pair, fp32 output, no bias, no scales). */
typedef struct tesserae_kernel_spec {
    const char* name;
    int arch;        /* TESSERAE_SM* */
    int elem;        /* TESSERAE_* element code of A and B */
    int tile_m, tile_n, tile_k;   /* 128 rows per CTA; tile_n a multiple of 16 per CTA (and of the 128-byte store chunk) up
                                     to 256, or 512 for an unscaled CTA-pair kernel; tile_k elements spanning 32, 64 or
                                     128 bytes (128 for the block-scaled kernels) */
    int stages;      /* ignored by Lower.lower, like the reference; 0 = choose by smem */
    int cta_group;   /* 0 or 2: CTA pair (reference), 1: single CTA */
    int out_elem;    /* 0 or TESSERAE_F32: fp32 C (reference); TESSERAE_BF16: bf16 C */
    int has_bias;    /* add bf16 bias[n] in the epilogue */
    int scale_mode;  /* TESSERAE_SCALE_* */
    int scatter;     /* row-scattered output for tesserae_gemm_ksplit_scatter (unscaled kernels, fp32 out, no bias):
                        1 = each tile is stored to the owner's slot, 2 = each tile is added into the owner's buffer */
    /* Optional overrides of the kernel's tuning choices, "NAME=VALUE;NAME=VALUE" (NULL or "" = the defaults).
     * The kernel a plan runs is a function of its spec alone; nothing is read from the environment.  Names:
     *   GROUP_M=1..64          M-tiles per raster group of the persistent tile order (default: sized per launch so
     *                          that a group's panel of A, group_m x 128*cta_group rows x K, is about 32 MB)
     *   STORE_BUFS=2..4        dense kernel: staging buffers per epilogue warp
     *   FP8_PROMO_WARPS=8|16   block-scaled FP8: promotion warps
     *   FP8_SPLIT=0|1          block-scaled FP8: one MMA chain per tile width / per 128 columns
     *   TAIL_SPLITS=0..64      block-scaled FP8: stream-K tail (tesserae_gemm_run_scaled_ws); 0 or 1 = none
     *   CLC=0|1                unscaled kernels without scatter: tile order by cluster launch control.  The grid has
     *                          one cluster per tile; a seventh warp (the Scheduler role of lib/pipeline/cluster.mli:17-21)
     *                          cancels clusters that have not started and feeds their tiles to the running ones, so
     *                          tiles of unequal length are balanced dynamically.  Results are bit-identical to the
     *                          static order's.
     * An unknown name or a value out of range fails with IncompatibleTile. */
    const char* tuning;
    int grouped;     /* 1: the kernel walks a list of problems (tesserae_gemm_run_grouped); unscaled kernels, no scatter */
} tesserae_kernel_spec;

/* Kernel_desc.t (lib/kernel/kernel_desc.ml:12-26), flattened to integers. */
typedef struct tesserae_kernel_desc {
    int family;
    char name[64];
    int bm, bn, bk;
    int elem;
    int swizzle_b, swizzle_m, swizzle_s;            /* Swizzle.smem_selector elem bm bk */
    int cluster_x, cluster_y, cluster_z;
    int num_warps;
    int warp_roles[8];                              /* role of warp i, -1 beyond num_warps */
    int pipeline_depth;
    int64_t tile_bytes;                             /* (bm+bn)*bk*byte_width */
    int64_t smem_bytes;                             /* depth*tile_bytes */
    int strategy;                                   /* TESSERAE_TMA_PAIR for Blackwell */
    int copy_bulk_bytes, copy_vec;                  /* 128, 128/byte_width */
    int atom_m, atom_n, atom_k, atom_threads;       /* sm100_128x128x16: 128,128,16,128 */
    int tmem_cta_group, tmem_rows, tmem_cols, tmem_double_buf;
    int64_t pred_a_bounds[2], pred_b_bounds[2], pred_c_bounds[2];
    int sm_count;
    int64_t m, n, k;                                /* Lower.infer_*: tile*32 */
} tesserae_kernel_desc;

/* Lower.lower (lib/kernel/lower.ml:61-97).  Returns a TESSERAE_LOWER_* code; only
 * SM100 with F16/BF16/S8 (reference) or F8E4M3/F4E2M1 (extension) lowers. */
int tesserae_lower(const tesserae_kernel_spec* spec, tesserae_kernel_desc* out);
/* Kernel_desc.validate (lib/kernel/kernel_desc.ml:167-190); message = reference's Error text. */
int tesserae_kernel_desc_validate(const tesserae_kernel_desc* d);
/* Kernel_desc.arithmetic_intensity (lib/kernel/kernel_desc.ml:193-202) */
double tesserae_kernel_desc_arithmetic_intensity(const tesserae_kernel_desc* d);
/* Kernel_desc.emit_launch_config's grid (lib/kernel/kernel_desc.ml:222-239) */
int tesserae_kernel_desc_grid(const tesserae_kernel_desc* d, int64_t m, int64_t n, int* gx, int* gy, int* threads);

/* ------------------------------------------------------------------ backend: descriptor -> CUDA source */
/* Backend_cute.output (lib/backend/backend_cute.mli:10-21).  Strings are owned by the
 * record; release with tesserae_backend_output_free. */
typedef struct tesserae_backend_output {
    char* filename;
    char* includes;
    char* helpers;
    char* shared_storage;
    char* producer_body;
    char* consumer_body;
    char* epilogue_body;
    char* kernel_func;
    char* host_launcher;
    char* full_source;
} tesserae_backend_output;
/* Backend_cute.emit (lib/backend/backend_cute.ml:431-453) for the Blackwell family. */
int tesserae_backend_emit(const tesserae_kernel_spec* spec, tesserae_backend_output* out);
void tesserae_backend_output_free(tesserae_backend_output* out);

/* ------------------------------------------------------------------ Tirix: the IR between descriptor and source
 * The reference's second emission path goes descriptor -> Tirix IR -> source (lib/tirix/desc_to_tirix.ml:466-508,
 * lib/tirix/tirix_emit.ml:481-501) with a scope / structure verifier in between (lib/tirix/tirix_verify.ml:9-183).
 * Here the IR states, role by role, the structure of the sm_100a mainloop a spec selects, in the reference's
 * statement forms (let / assign / op / if / for / pipeline / warpgroup / pragma / seq) and operations, extended by
 * what the working kernels need (bounded waits only, TMA stores and reduce-adds, TMEM stores, the fp32 promotion).
 * It has a line-oriented text form that prints and parses back, so a host can inspect or edit it as text.
 * Emission goes through the IR: the program must verify and must have the structure of the mainloop its `origin`
 * line selects; the emitted source carries the program's listing in its header. */
typedef struct tesserae_tirix tesserae_tirix;
/* Desc_to_tirix.lower after Lower.lower; returns a TESSERAE_LOWER_* code. */
int tesserae_tirix_lower(const tesserae_kernel_spec* spec, tesserae_tirix** out);
/* Text -> program; -1 with a message naming the line on a malformed text. */
int tesserae_tirix_parse(const char* text, tesserae_tirix** out);
void tesserae_tirix_free(tesserae_tirix* program);
/* Program -> text (malloc'ed; caller frees). */
char* tesserae_tirix_print(const tesserae_tirix* program);
/* Tirix_verify.verify: number of errors (0 = Ok); *errors gets the messages, newline-separated (malloc'ed; caller
 * frees), the reference's wording: "undefined variable 'x'", "unknown tensor 't' in copy.src", "SFor 'i' has zero
 * step", "SPipeline has invalid stage count 0", "SWarpGroup role not in cluster warp_roles", ... */
int tesserae_tirix_verify(const tesserae_tirix* program, char** errors);
/* How many operations of the named kind ("Copy", "Mma", "MbarWaitParity", "TmemAlloc", ...) the program holds. */
int tesserae_tirix_count_ops(const tesserae_tirix* program, const char* op_name);
/* Tirix_emit.emit: program -> the record of source sections (release with tesserae_backend_output_free). */
int tesserae_tirix_emit(const tesserae_tirix* program, tesserae_backend_output* out);

/* Compile.result (lib/runtime/compile.ml:4-9), with a cubin image instead of PTX. */
typedef struct tesserae_compile_result {
    char* kernel_name;
    char* source;
    void* cubin;          /* NULL for to_source */
    size_t cubin_size;
    double duration_ms;   /* wall time of emit (+ compile) */
    int cache_hit;        /* cubin came from the on-disk cache */
} tesserae_compile_result;
/* Compile.to_source / Compile.to_ptx (lib/runtime/compile.ml:36-75) */
int tesserae_compile_to_source(const tesserae_kernel_spec* spec, tesserae_compile_result* out);
int tesserae_compile_to_cubin(const tesserae_kernel_spec* spec, tesserae_compile_result* out);
void tesserae_compile_result_free(tesserae_compile_result* r);

/* ------------------------------------------------------------------ NVRTC (lib/runtime/nvrtc_stub.h:6-55) */
typedef struct tesserae_nvrtc_program {
    char* source;
    char* name;
    char* ptx;        /* NULL until compiled (and when the target produced a cubin only) */
    char* log;
    int compiled;
    int valid;
    void* handle;
    void* cubin;      /* extension: device image when compiled for a real architecture */
    size_t cubin_size;
} tesserae_nvrtc_program;
tesserae_nvrtc_program* tesserae_nvrtc_create(const char* source, const char* name);
void tesserae_nvrtc_destroy(tesserae_nvrtc_program* prog);
int tesserae_nvrtc_is_valid(tesserae_nvrtc_program* prog);
int tesserae_nvrtc_compile(tesserae_nvrtc_program* prog, const char** opts, int n_opts);
char* tesserae_nvrtc_get_ptx(tesserae_nvrtc_program* prog);   /* caller frees */
char* tesserae_nvrtc_get_log(tesserae_nvrtc_program* prog);   /* caller frees */
const char* tesserae_nvrtc_get_source(tesserae_nvrtc_program* prog);
const char* tesserae_nvrtc_get_name(tesserae_nvrtc_program* prog);
/* Extension: borrowed pointer to the cubin (valid until destroy). */
int tesserae_nvrtc_get_cubin(tesserae_nvrtc_program* prog, const void** image, size_t* size);
/* Extension: compile `source` for sm_100a to a cubin through the on-disk cache
 * (directory $TESSERAE_CACHE_DIR, default "_cubin_cache" beside the library).  The image
 * is malloc'ed; caller frees.  *cache_hit tells whether NVRTC ran. */
int tesserae_compile_cached(const char* source, const char* name, const char** opts, int n_opts,
                            void** image, size_t* size, int* cache_hit);
const char* tesserae_cache_dir(void);

/* ------------------------------------------------------------------ device buffers (lib/runtime/gpu_buffer_stubs.c:26-83) */
int tesserae_gpu_alloc(size_t n_bytes, void** dptr);                 /* cudaMalloc + zero fill */
int tesserae_gpu_free(void* dptr);                                   /* NULL is a no-op */
int tesserae_gpu_copy_to_device(void* dptr, const void* src, size_t n_bytes);
int tesserae_gpu_copy_to_host(void* dst, const void* dptr, size_t n_bytes);

/* ------------------------------------------------------------------ modules and launch (lib/kernel/kernel_launch_stubs.c:21-107) */
int tesserae_cuinit(void);
int tesserae_set_device(int device);
int tesserae_module_load(const void* image, void** module);          /* PTX text or cubin */
int tesserae_module_unload(void* module);
int tesserae_get_function(void* module, const char* name, void** function);
/* caml_launch_kernel: every argument is one 8-byte slot passed by address; default stream. */
int tesserae_launch_kernel(void* function, int gx, int gy, int gz, int bx, int by, int bz,
                           int smem_bytes, const int64_t* args, int n_args);
/* Extension: cuLaunchKernelEx with cluster dimensions, a stream and arguments of any size
 * (a 128-byte tensor map does not fit the 8-byte slots above). */
typedef struct tesserae_launch_arg { const void* data; size_t size; } tesserae_launch_arg;
int tesserae_launch_kernel_ex(void* function, const int grid[3], const int block[3], const int cluster[3],
                              int smem_bytes, void* stream, const tesserae_launch_arg* args, int n_args);
int tesserae_device_synchronize(void);
/* caml_device_info: "NAME (sm_XY)" of device 0 */
int tesserae_device_info(char* buf, size_t buf_size);
int tesserae_device_sm_count(int* sm_count);
/* Extension: 128-byte tensor map of a row-major 2-D array for tiled TMA access.
 * swizzle_b is Swizzle.b (0..3 = none/32B/64B/128B, lib/pipeline/smem_desc.ml:17-23). */
int tesserae_tensor_map_2d(void* out_map128, int elem, const void* gptr, uint64_t inner, uint64_t outer,
                           uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_b);

/* ------------------------------------------------------------------ GEMM plans and Runtime.run */
typedef struct tesserae_gemm_plan tesserae_gemm_plan;
/* Emit + compile (cached) + load the kernel a spec names.  One plan serves any M, N, K.
 * A plan belongs to the device that was current when it was made (calls with another device current are refused).
 * Calls on one plan may come from any host thread but not from two at once: the plan holds per-call host state (the
 * status word's owner, the pinned staging copy of a grouped launch's problem table, the host-buffer entry points'
 * workspaces).  Different plans are independent. */
int tesserae_gemm_plan_create(const tesserae_kernel_spec* spec, tesserae_gemm_plan** plan);
void tesserae_gemm_plan_destroy(tesserae_gemm_plan* plan);
int tesserae_gemm_plan_info(const tesserae_gemm_plan* plan, int* cta_group, int* block_n, int* stages,
                            int* smem_bytes, int* cache_hit, double* compile_ms);
/* C = alpha * A . B^T (+ bias).  A is M x K row-major, B is N x K row-major ("column-major
 * K x N"), C is M x N row-major; all device pointers; asynchronous on `stream`.
 * K*elem_bytes and N*out_bytes must be multiples of 16. */
int tesserae_gemm_run(tesserae_gemm_plan* plan, const void* a, const void* b, void* c, const void* bias,
                      float alpha, int64_t m, int64_t n, int64_t k, void* stream);
/* Scale factors of a block-scaled GEMM (device pointers).
 *  TESSERAE_SCALE_FP8_BLOCK: scale_a = fp32 [M][K/128] (one per row and 128-wide K block),
 *                            scale_b = fp32 [ceil(N/128)][K/128] (one per 128x128 block); K % 128 == 0.
 *  TESSERAE_SCALE_NVFP4: A and B hold E2M1 values, two per byte along K (even k in the low nibble);
 *      scale_a / scale_b hold one UE4M3 byte per row and 16 K-elements, stored in the order the
 *      tensor core reads them: 512-byte chunks [row block rb of 128 rows][K group kg of 64 elements],
 *      chunk byte (r % 32) * 16 + (r / 32) * 4 + j = scale of row 128*rb + r, K block 4*kg + j; the
 *      row count is padded up to a multiple of 128 with zero bytes; K % 256 == 0.
 *      global_a / global_b: the per-tensor fp32 scales (multiplied into alpha). */
typedef struct tesserae_gemm_scales {
    const void* scale_a;
    const void* scale_b;
    float global_a;
    float global_b;
} tesserae_gemm_scales;
/* tesserae_gemm_run for a plan whose spec has a scale_mode: C = alpha * dequant(A) . dequant(B)^T (+ bias). */
int tesserae_gemm_run_scaled(tesserae_gemm_plan* plan, const void* a, const void* b, void* c,
                             const tesserae_gemm_scales* scales, const void* bias,
                             float alpha, int64_t m, int64_t n, int64_t k, void* stream);
/* ------------------------------------------------------------------ stream-K tail (FP8 block-scaled)
 * tesserae_gemm_run_scaled with a workspace, for plans whose spec's tuning has TAIL_SPLITS=n (n >= 2; the kernel is
 * then compiled with the unit logic below; opt-in, because on the shapes measured it wins nothing over running the
 * left-over tiles as a last wave):
 * when tiles are left over after the last whole wave and fill at most half the resident clusters, each of them is
 * split into at most n ranges of K blocks that all CTAs share; the fp32 partial sums are added into the workspace and
 * a closing kernel adds the bias, casts into C and clears the workspace again.  The role is the one the reference
 * reserves for a scheduler (lib/pipeline/cluster.mli:17-21); it has no counterpart there.
 *   tesserae_gemm_tail_workspace_bytes: bytes the call below needs for this problem on this plan (0: no tail is used,
 *   the workspace may be NULL; always 0 for plans without TAIL_SPLITS).
 *   The workspace must be 128-byte aligned and ZERO-FILLED before its first use; every call leaves it zero-filled.
 *   After a call whose tesserae_gemm_status is not 0, clear it again.
 * The additions into the workspace happen in no fixed order: the tail tiles' results can differ in the last bit from
 * run to run and from tesserae_gemm_run_scaled; all other tiles are bit-identical. */
size_t tesserae_gemm_tail_workspace_bytes(const tesserae_gemm_plan* plan, int64_t m, int64_t n, int64_t k);
int tesserae_gemm_run_scaled_ws(tesserae_gemm_plan* plan, const void* a, const void* b, void* c,
                                const tesserae_gemm_scales* scales, const void* bias,
                                float alpha, int64_t m, int64_t n, int64_t k,
                                void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ grouped GEMM
 * Many independent problems C_i = alpha * A_i . B_i^T (+ bias_i) in one launch (the role the reference reserves for
 * its scheduler warp, lib/pipeline/cluster.mli:17-21, lib/kernel/kernel_desc.ml:135; it builds none).  The plan's spec
 * must have grouped = 1.  The tiles of all problems are numbered consecutively and dealt to the persistent CTAs, so a
 * wave holds tiles of several problems and a list of small or ragged problems is not quantised one by one.
 * Layouts per problem as for tesserae_gemm_run; sizes may differ from problem to problem.
 * `workspace` is device memory of tesserae_gemm_grouped_workspace_bytes(n_problems) bytes (the problem table: tensor
 * maps and sizes, written by this call with an asynchronous copy on `stream`); it must stay untouched until the launch
 * has finished.  Asynchronous on `stream`. */
typedef struct tesserae_gemm_problem {
    const void* a;      /* M x K, row-major */
    const void* b;      /* N x K, row-major */
    void* c;            /* M x N, row-major */
    const void* bias;   /* bf16[N] or NULL (must be given when the kernel was built with a bias) */
    int64_t m, n, k;
} tesserae_gemm_problem;
size_t tesserae_gemm_grouped_workspace_bytes(int n_problems);
int tesserae_gemm_run_grouped(tesserae_gemm_plan* plan, const tesserae_gemm_problem* problems, int n_problems,
                              float alpha, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ quantisers (the step before a block-scaled GEMM)
 * fp32 device source -> the operand and scale layouts tesserae_gemm_run_scaled takes.  New surface: the
 * reference has no narrow float element.  Asynchronous on `stream` unless noted.  Recipes:
 *   FP8 rows   : scale = absmax(row, 128-wide K block) / 448 (1 for an all-zero block), q = sat_rne_e4m3(x / scale)
 *   FP8 blocks : the same per 128x128 block of w (rows beyond N count as zeros)
 *   NVFP4      : global = absmax(x) / (448*6) (1 if zero), s = rne_ue4m3(absmax16 / (6*global)),
 *                q = sat_rne_e2m1(x / (s*global)); scales in the chunked order described at tesserae_gemm_scales */
int tesserae_quantize_fp8_rows(const float* x, void* q_e4m3, float* scale, int64_t m, int64_t k, void* stream);
int tesserae_quantize_fp8_blocks(const float* w, void* q_e4m3, float* scale, int64_t n, int64_t k, void* stream);
/* Bytes of an NVFP4 scale table for `rows` x `k` (rows padded to a multiple of 128). */
size_t tesserae_nvfp4_scale_bytes(int64_t rows, int64_t k);
/* q: rows x k/2 bytes; scale_chunks: tesserae_nvfp4_scale_bytes(rows, k) bytes; workspace4: 4 device bytes.
 * Writes the per-tensor scale to *global_scale (host) and therefore synchronises `stream` before returning. */
int tesserae_quantize_nvfp4(const float* x, void* q_e2m1, void* scale_chunks, float* global_scale, void* workspace4,
                            int64_t rows, int64_t k, void* stream);

/* ------------------------------------------------------------------ sharding across the GPUs of one node */
/* Range [begin, begin+length) that shard `index` of `parts` owns out of [0, total), with boundaries at
 * multiples of `align`.  N-split (columns of C / rows of B, no collective): align 128; K-split (columns of A
 * and B, reduce-scatter of the fp32 partials afterwards): align = K elements of one smem stage. */
int tesserae_shard_range(int64_t total, int parts, int index, int64_t align, int64_t* begin, int64_t* length);

/* NCCL for hosts that have no other route to it (the reference has no collective; new exports).  libnccl.so.2 is
 * opened on first use — the copy already in the process if there is one, else $TESSERAE_NCCL_LIB, else the loader's
 * search path; tesserae_nccl_load(path) opens a specific file first.  One communicator per GPU, created with that
 * GPU current: rank 0 makes the 128-byte id, the host carries it to the other ranks by its own means, every rank
 * calls comm_init.  The collectives are asynchronous on `stream`; counts are fp32 elements per rank.  The K-split
 * path's exchange is tesserae_nccl_reduce_scatter_f32(comm, partial[M x N], mine[M/G x N], M/G * N, stream). */
int tesserae_nccl_load(const char* path_or_null);
int tesserae_nccl_version(int* version);
int tesserae_nccl_unique_id(void* id128);
int tesserae_nccl_comm_init(void** comm, int world, int rank, const void* id128);
/* comm_init that gives up: the communicator is created non-blocking and polled; if it is not ready after
 * `timeout_ms` (a rank never joined, a peer died during set-up) it is aborted, *comm is NULL and the call fails
 * with a message that names the timeout.  Needs NCCL 2.14 or later.  Collectives on such a communicator are
 * settled inside the wrappers below, so callers see the same 0 / non-zero contract. */
int tesserae_nccl_comm_init_deadline(void** comm, int world, int rank, const void* id128, int timeout_ms);
/* ncclCommAbort: tears a communicator down without waiting for its peers or for work in flight; the call for
 * the path where a rank has failed and ncclCommDestroy would block.  NULL is a no-op. */
int tesserae_nccl_comm_abort(void* comm);
int tesserae_nccl_comm_destroy(void* comm);
int tesserae_nccl_reduce_scatter_f32(void* comm, const void* send, void* recv, size_t recv_count, void* stream);
int tesserae_nccl_all_reduce_f32(void* comm, const void* send, void* recv, size_t count, void* stream);

/* ------------------------------------------------------------------ K-split: fp32 partials, then sum + bf16 cast */
/* out[i] = bf16(alpha * sum_p parts[p * part_stride_elems + i]): the pass that follows the fp32
 * partial products of a K-split GEMM (on one GPU, or after the reduce-scatter between GPUs).
 * Buffers 16-byte aligned; asynchronous on `stream`. */
int tesserae_reduce_cast_bf16(const void* parts_f32, int n_parts, size_t part_stride_elems, float alpha,
                              void* out_bf16, size_t n_elems, void* stream);
/* out[i] = bf16(alpha * acc[i]) and acc[i] = 0, in one pass: the step after a K-split GEMM whose epilogue ADDED the
 * partial tiles into `acc` (spec.scatter = 2); the buffer is left holding the zeros its next use needs.
 * Buffers 16-byte aligned; asynchronous on `stream`. */
int tesserae_cast_clear_bf16(void* acc_f32, float alpha, void* out_bf16, size_t n_elems, void* stream);
/* Scratch (global memory beyond inputs and outputs) the K-split entry points need: k_splits fp32 M x N partials. */
size_t tesserae_gemm_ksplit_scratch_bytes(int64_t m, int64_t n, int k_splits);
/* Partial products only: slice s of K (K/k_splits wide) -> scratch[s] (fp32 M x N).  The plan must be an
 * unscaled kernel with fp32 output and no bias.  With one slice per GPU this is each GPU's share of a
 * K-split across GPUs; the caller then reduce-scatters the partials. */
int tesserae_gemm_ksplit_partials(tesserae_gemm_plan* plan, const void* a, const void* b, void* scratch,
                                  size_t scratch_bytes, int64_t m, int64_t n, int64_t k, int k_splits, void* stream);
/* Whole K-split GEMM on one GPU: partials into `scratch`, then sum + alpha + bf16 cast into c_bf16. */
int tesserae_gemm_ksplit_run(tesserae_gemm_plan* plan, const void* a, const void* b, void* c_bf16, void* scratch,
                             size_t scratch_bytes, float alpha, int64_t m, int64_t n, int64_t k, int k_splits,
                             void* stream);
/* K-split partial product with the reduce-scatter fused into the GEMM's epilogue.  The plan's spec must
 * have scatter = 1, fp32 output, no bias, no scales.  Rows [g*rows_per_owner, (g+1)*rows_per_owner) of this
 * GPU's fp32 partial C are stored to dst[g] (an M/G x N fp32 array, row pitch N), g = 0..n_dst-1 <= 8;
 * rows_per_owner is a multiple of 128 and n_dst * rows_per_owner >= m.  With dst[g] pointing into GPU g's
 * memory (peer mapping of a staging slot reserved for this source GPU) the partial tiles cross NVLink as
 * plain TMA stores while the mainloop runs; after a barrier between the GPUs each owner sums its slots with
 * tesserae_reduce_cast_bf16.  Only stores go to peer memory; every load is local.
 * With scatter = 2 in the spec the tiles are not stored but ADDED (fp32, by the memory system of the GPU that owns
 * dst[g]; a TMA reduce, still a store-type operation): every source GPU passes the SAME dst[g] for owner g, the
 * buffers must hold zeros when the first contribution arrives, and after the barrier dst[own] already is the
 * reduce-scattered fp32 sum, so only tesserae_reduce_cast_bf16 with n_parts = 1 remains.  The contributions of
 * more than two GPUs meet in no fixed order: the sum may differ in the last place between runs.
 * start_owner: the owner whose rows this GPU computes (and sends) first; the others follow round robin.  Give every
 * source GPU a different one (its own rank): GPUs that walk the tiles in the same order would all send to the same
 * owner at the same time and queue up on that owner's NVLink ingress.  0 is always valid. */
int tesserae_gemm_ksplit_scatter(tesserae_gemm_plan* plan, const void* a, const void* b, void* const* dst, int n_dst,
                                 int64_t rows_per_owner, int start_owner, int64_t m, int64_t n, int64_t k, void* stream);
/* tesserae_gemm_ksplit_run without caller scratch and without any allocation.  It has no counterpart in
 * the reference.  It is for hosts that cannot call cudaMalloc at the moment they need the GEMM: a process
 * whose own allocator already owns nearly all GPU memory (a raw cudaMalloc would fail there), or a serving
 * loop that cannot take the device-wide synchronisation an allocation or free implies.  The fp32 partials
 * go to a fixed array inside the library image (TESSERAE_NOALLOC_MAX_ELEMS floats = 32 MiB per GPU).
 *   - Limit: m * n * k_splits <= TESSERAE_NOALLOC_MAX_ELEMS, otherwise the call fails with a message naming
 *     both numbers; nothing is launched.
 *   - The first call on each device is the set-up call: it looks up the array's device address (with that
 *     device current), and because CUDA loads device code lazily that lookup is also the moment the driver
 *     reserves the 32 MiB on that device (they are then held until the process exits).  Make that first call
 *     at start-up, before the host's own allocator takes the remaining memory and before any stream capture;
 *     a call that is refused for its size still performs the set-up, so a start-up call needs no real work.
 *     From the second call on a device nothing is allocated or reserved: free device memory is the same
 *     before and after a call.
 *   - The looked-up address is cached per device ordinal.  If the host resets a device's primary context
 *     (cudaDeviceReset) the cached address is stale; the library is not meant to outlive such a reset.
 *   - All calls share the one array, which keeps the previous call's partials.  Nothing needs clearing (the
 *     GEMM overwrites every element it later sums), but two calls that overlap on the GPU (different
 *     streams, no ordering between them) race on it.
 *   - Neither this call nor anything under it calls cudaMalloc, cudaFree or an allocating library routine;
 *     the plan is created beforehand, and must be used with the device it was created on current. */
#define TESSERAE_NOALLOC_MAX_ELEMS 8388608
size_t tesserae_gemm_ksplit_noalloc_max_elems(void);
int tesserae_gemm_ksplit_run_noalloc(tesserae_gemm_plan* plan, const void* a, const void* b, void* c_bf16,
                                     float alpha, int64_t m, int64_t n, int64_t k, int k_splits, void* stream);
/* Reads (and clears) the device status word the kernels write when a bounded wait ran out;
 * synchronises the device.  0 = healthy. */
int tesserae_gemm_status(tesserae_gemm_plan* plan, uint32_t* status);
/* Self-test of the bounded wait the kernels are built on: one warp waits, with a budget of
 * `budget_cycles` SM cycles (1e3..2e9), on a barrier that nothing signals.  On return *status_out
 * holds the bits the kernel recorded (0x40 = the wait gave up, as it must; 0 would mean the barrier
 * completed) and *waited_cycles_out the cycles the wait took.  The kernel returns normally and the
 * context stays usable.  No counterpart in the reference, whose waits are unbounded. */
int tesserae_wait_selftest(int64_t budget_cycles, uint32_t* status_out, int64_t* waited_cycles_out);
/* Same call with host buffers in the operand's own element type: copies A, B (and bias) to
 * the device, runs, copies C back, all inside the call.  Synchronous. */
int tesserae_gemm_run_host(tesserae_gemm_plan* plan, const void* a, const void* b, void* c, const void* bias,
                           float alpha, int64_t m, int64_t n, int64_t k);
/* The block-scaled call with host buffers: A, B, both scale tables (in `scales`, HOST pointers here) and the bias
 * go up, C comes back, inside the call; same chunked pipeline as tesserae_gemm_run_host.  Synchronous. */
int tesserae_gemm_run_scaled_host(tesserae_gemm_plan* plan, const void* a, const void* b, void* c,
                                  const tesserae_gemm_scales* scales, const void* bias,
                                  float alpha, int64_t m, int64_t n, int64_t k);
/* Runtime.run (lib/runtime/runtime.ml:15-75): fp32 host arrays in, fp32 host array out;
 * A and B are rounded to the spec's element type on the host (the reference uploads fp32
 * bits unconverted, lib/runtime/gpu_buffer.ml:32-40, which its kernels then misread). */
int tesserae_runtime_run(const tesserae_kernel_spec* spec, int64_t m, int64_t n, int64_t k,
                         const float* a, const float* b, float* c);
/* Runtime.is_available / Runtime.device_info (lib/runtime/runtime.ml:7-13,77-80) */
int tesserae_runtime_is_available(void);

#ifdef __cplusplus
}
#endif
#endif /* TESSERAE_B200_H */
