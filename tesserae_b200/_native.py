"""ctypes loader for libtesserae_b200.so (the in-tree C-ABI library).

There is no fallback: if the library is missing the import fails with the build command to
run, and every GPU entry point fails loudly when no CUDA driver is present.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_PKG = Path(__file__).resolve().parent
LIB_PATH = _PKG / "libtesserae_b200.so"


class KernelSpecC(C.Structure):
    _fields_ = [("name", C.c_char_p), ("arch", C.c_int), ("elem", C.c_int),
                ("tile_m", C.c_int), ("tile_n", C.c_int), ("tile_k", C.c_int), ("stages", C.c_int),
                ("cta_group", C.c_int), ("out_elem", C.c_int), ("has_bias", C.c_int), ("scale_mode", C.c_int),
                ("scatter", C.c_int), ("tuning", C.c_char_p), ("grouped", C.c_int)]


class KernelDescC(C.Structure):
    _fields_ = [("family", C.c_int), ("name", C.c_char * 64), ("bm", C.c_int), ("bn", C.c_int), ("bk", C.c_int),
                ("elem", C.c_int), ("swizzle_b", C.c_int), ("swizzle_m", C.c_int), ("swizzle_s", C.c_int),
                ("cluster_x", C.c_int), ("cluster_y", C.c_int), ("cluster_z", C.c_int), ("num_warps", C.c_int),
                ("warp_roles", C.c_int * 8), ("pipeline_depth", C.c_int), ("tile_bytes", C.c_int64),
                ("smem_bytes", C.c_int64), ("strategy", C.c_int), ("copy_bulk_bytes", C.c_int),
                ("copy_vec", C.c_int), ("atom_m", C.c_int), ("atom_n", C.c_int), ("atom_k", C.c_int),
                ("atom_threads", C.c_int), ("tmem_cta_group", C.c_int), ("tmem_rows", C.c_int),
                ("tmem_cols", C.c_int), ("tmem_double_buf", C.c_int), ("pred_a_bounds", C.c_int64 * 2),
                ("pred_b_bounds", C.c_int64 * 2), ("pred_c_bounds", C.c_int64 * 2), ("sm_count", C.c_int),
                ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64)]


class BackendOutputC(C.Structure):
    _fields_ = [(f, C.c_void_p) for f in ("filename", "includes", "helpers", "shared_storage", "producer_body",
                                          "consumer_body", "epilogue_body", "kernel_func", "host_launcher",
                                          "full_source")]


class CompileResultC(C.Structure):
    _fields_ = [("kernel_name", C.c_void_p), ("source", C.c_void_p), ("cubin", C.c_void_p),
                ("cubin_size", C.c_size_t), ("duration_ms", C.c_double), ("cache_hit", C.c_int)]


class NvrtcProgramC(C.Structure):
    _fields_ = [("source", C.c_void_p), ("name", C.c_void_p), ("ptx", C.c_void_p), ("log", C.c_void_p),
                ("compiled", C.c_int), ("valid", C.c_int), ("handle", C.c_void_p), ("cubin", C.c_void_p),
                ("cubin_size", C.c_size_t)]


class GemmScalesC(C.Structure):
    _fields_ = [("scale_a", C.c_void_p), ("scale_b", C.c_void_p), ("global_a", C.c_float), ("global_b", C.c_float)]


class MmaAtomC(C.Structure):
    _fields_ = [(f, C.c_int) for f in ("arch", "m", "n", "k", "a_type", "b_type", "c_type", "d_type", "a_major", "b_major")]


class CopyAtomC(C.Structure):
    _fields_ = [(f, C.c_int) for f in ("kind", "src_space", "dst_space", "elem", "vec_width", "bulk_bytes")]


class TiledMmaC(C.Structure):
    _fields_ = [(f, C.c_int64) for f in ("thread_count", "warp_count", "tile_m", "tile_n", "tile_k", "partition_a",
                                         "partition_b", "partition_c")]


class TiledCopyC(C.Structure):
    _fields_ = [("thread_count", C.c_int64), ("elements_per_thread", C.c_int64), ("tile_size", C.c_int64),
                ("is_tma", C.c_int), ("requires_mbar", C.c_int)]


class TileOpC(C.Structure):
    _fields_ = [("atom", MmaAtomC), ("thread_layout_size", C.c_int64), ("warp_layout_size", C.c_int64),
                ("tiler_m", C.c_int64), ("tiler_n", C.c_int64), ("accum_loc", C.c_int), ("has_tmem", C.c_int),
                ("tmem_cta_group", C.c_int), ("tmem_cols", C.c_int), ("tmem_rows", C.c_int), ("double_buf", C.c_int)]


class GemmProblemC(C.Structure):
    _fields_ = [("a", C.c_void_p), ("b", C.c_void_p), ("c", C.c_void_p), ("bias", C.c_void_p),
                ("m", C.c_int64), ("n", C.c_int64), ("k", C.c_int64)]


class LaunchArgC(C.Structure):
    _fields_ = [("data", C.c_void_p), ("size", C.c_size_t)]


_I64P = C.POINTER(C.c_int64)
_IP = C.POINTER(C.c_int)

# name -> (restype, argtypes); must list every symbol include/tesserae_b200.h declares.
SIGNATURES = {
    "tesserae_last_error": (C.c_char_p, []),
    "tesserae_version": (C.c_char_p, []),
    "tesserae_swizzle_apply": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int64]),
    "tesserae_swizzle_smem_selector": (C.c_int, [C.c_int, C.c_int, C.c_int, _IP, _IP, _IP]),
    "tesserae_elem_byte_width": (C.c_int, [C.c_int]),
    "tesserae_elem_bits": (C.c_int, [C.c_int]),
    "tesserae_elem_vec_width": (C.c_int, [C.c_int]),
    "tesserae_layout_size": (C.c_int64, [_I64P, C.c_int]),
    "tesserae_swizzle_apply_to_strides": (C.c_int, [C.c_int, C.c_int, C.c_int, _I64P, C.c_int, _I64P]),
    "tesserae_layout_cosize": (C.c_int64, [_I64P, _I64P, C.c_int]),
    "tesserae_layout_idx": (C.c_int64, [_I64P, _I64P, C.c_int]),
    "tesserae_layout_compose": (C.c_int, [_I64P, _I64P, C.c_int, _I64P, _I64P, C.c_int, _I64P]),
    "tesserae_layout_tile": (C.c_int, [_I64P, _I64P, C.c_int, _I64P, _I64P, _I64P]),
    "tesserae_layout_sort": (C.c_int, [_I64P, _I64P, C.c_int, _I64P, _I64P]),
    "tesserae_layout_coalesce": (C.c_int, [_I64P, _I64P, C.c_int, _I64P, _I64P]),
    "tesserae_layout_is_admissible": (C.c_int, [_I64P, _I64P, C.c_int, C.c_int64]),
    "tesserae_layout_complement": (C.c_int, [_I64P, _I64P, C.c_int, C.c_int64, _I64P, _I64P]),
    "tesserae_layout_flat_divide": (C.c_int, [_I64P, _I64P, C.c_int, C.c_int64, _I64P, _I64P]),
    "tesserae_layout_logical_divide": (C.c_int, [_I64P, _I64P, C.c_int, _I64P, _I64P, _I64P]),
    "tesserae_pipeline_smem_bytes": (C.c_int64, [C.c_int, C.c_int64]),
    "tesserae_pipeline_stage_of": (C.c_int, [C.c_int64, C.c_int]),
    "tesserae_pipeline_phase_of": (C.c_int, [C.c_int64, C.c_int]),
    "tesserae_pipeline_smem_offset_of": (C.c_int64, [C.c_int64, C.c_int]),
    "tesserae_pipeline_b_smem_offset_of": (C.c_int64, [C.c_int64, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tesserae_tmem_validate": (C.c_int, [C.c_int, C.c_int, C.c_int]),
    "tesserae_tmem_address": (C.c_int64, [C.c_int, C.c_int]),
    "tesserae_tmem_warp_row_offset": (C.c_int, [C.c_int]),
    "tesserae_tmem_num_loads_per_warp": (C.c_int, [C.c_int]),
    "tesserae_tmem_buf_col_offset": (C.c_int, [C.c_int]),
    "tesserae_smem_desc_encode": (C.c_int64, [C.c_int64, C.c_int64, C.c_int64, C.c_int]),
    "tesserae_umma_smem_desc": (C.c_uint64, [C.c_uint32, C.c_int]),
    "tesserae_umma_instr_desc": (C.c_uint32, [C.c_int, C.c_int, C.c_int]),
    "tesserae_tile_io_bytes_a": (C.c_int64, [C.c_int, C.c_int, C.c_int]),
    "tesserae_tile_io_bytes_b": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "tesserae_tile_io_expect_tx": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]),
    "tesserae_predicate_count_valid": (C.c_int64, [_I64P, _I64P, C.c_int]),
    "tesserae_predicate_residue": (C.c_int, [_I64P, _I64P, C.c_int, _I64P]),
    "tesserae_memspace_can_transfer": (C.c_int, [C.c_int, C.c_int]),
    "tesserae_memspace_name": (C.c_char_p, [C.c_int]),
    "tesserae_mma_atom_make": (C.c_int, [C.c_int, C.c_int, C.c_int, C.POINTER(MmaAtomC)]),
    "tesserae_mma_atom_thread_count": (C.c_int, [C.POINTER(MmaAtomC)]),
    "tesserae_mma_atom_is_wgmma": (C.c_int, [C.POINTER(MmaAtomC)]),
    "tesserae_mma_atom_emit_cpp": (C.c_int, [C.POINTER(MmaAtomC), C.c_char_p, C.c_size_t]),
    "tesserae_copy_atom_make": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(CopyAtomC)]),
    "tesserae_copy_atom_is_async": (C.c_int, [C.POINTER(CopyAtomC)]),
    "tesserae_copy_atom_is_tma": (C.c_int, [C.POINTER(CopyAtomC)]),
    "tesserae_copy_atom_requires_mbar": (C.c_int, [C.POINTER(CopyAtomC)]),
    "tesserae_copy_atom_emit_cpp": (C.c_int, [C.POINTER(CopyAtomC), C.c_char_p, C.c_size_t]),
    "tesserae_tiled_mma_make": (C.c_int, [C.POINTER(MmaAtomC), C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.POINTER(TiledMmaC)]),
    "tesserae_tiled_copy_make": (C.c_int, [C.POINTER(CopyAtomC), C.c_int64, C.c_int64, C.POINTER(TiledCopyC)]),
    "tesserae_tiled_copy_partition": (C.c_int, [C.c_int64, _I64P, _I64P, C.c_int, _I64P, _I64P]),
    "tesserae_tile_op_check": (C.c_int, [C.POINTER(TileOpC)]),
    "tesserae_tile_op_is_tmem": (C.c_int, [C.POINTER(TileOpC)]),
    "tesserae_tile_op_is_wgmma": (C.c_int, [C.POINTER(TileOpC)]),
    "tesserae_tile_op_accum_elems_per_thread": (C.c_int64, [C.POINTER(TileOpC)]),
    "tesserae_tile_op_emit": (C.c_int, [C.POINTER(TileOpC), C.c_int, C.c_char_p, C.c_char_p, C.c_int, C.c_char_p, C.c_size_t]),
    "tesserae_lower": (C.c_int, [C.POINTER(KernelSpecC), C.POINTER(KernelDescC)]),
    "tesserae_kernel_desc_validate": (C.c_int, [C.POINTER(KernelDescC)]),
    "tesserae_kernel_desc_arithmetic_intensity": (C.c_double, [C.POINTER(KernelDescC)]),
    "tesserae_kernel_desc_grid": (C.c_int, [C.POINTER(KernelDescC), C.c_int64, C.c_int64, _IP, _IP, _IP]),
    "tesserae_backend_emit": (C.c_int, [C.POINTER(KernelSpecC), C.POINTER(BackendOutputC)]),
    "tesserae_backend_output_free": (None, [C.POINTER(BackendOutputC)]),
    "tesserae_tirix_lower": (C.c_int, [C.POINTER(KernelSpecC), C.POINTER(C.c_void_p)]),
    "tesserae_tirix_parse": (C.c_int, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "tesserae_tirix_free": (None, [C.c_void_p]),
    "tesserae_tirix_print": (C.c_void_p, [C.c_void_p]),
    "tesserae_tirix_verify": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "tesserae_tirix_count_ops": (C.c_int, [C.c_void_p, C.c_char_p]),
    "tesserae_tirix_emit": (C.c_int, [C.c_void_p, C.POINTER(BackendOutputC)]),
    "tesserae_compile_to_source": (C.c_int, [C.POINTER(KernelSpecC), C.POINTER(CompileResultC)]),
    "tesserae_compile_to_cubin": (C.c_int, [C.POINTER(KernelSpecC), C.POINTER(CompileResultC)]),
    "tesserae_compile_result_free": (None, [C.POINTER(CompileResultC)]),
    "tesserae_nvrtc_create": (C.POINTER(NvrtcProgramC), [C.c_char_p, C.c_char_p]),
    "tesserae_nvrtc_destroy": (None, [C.POINTER(NvrtcProgramC)]),
    "tesserae_nvrtc_is_valid": (C.c_int, [C.POINTER(NvrtcProgramC)]),
    "tesserae_nvrtc_compile": (C.c_int, [C.POINTER(NvrtcProgramC), C.POINTER(C.c_char_p), C.c_int]),
    "tesserae_nvrtc_get_ptx": (C.c_void_p, [C.POINTER(NvrtcProgramC)]),
    "tesserae_nvrtc_get_log": (C.c_void_p, [C.POINTER(NvrtcProgramC)]),
    "tesserae_nvrtc_get_source": (C.c_char_p, [C.POINTER(NvrtcProgramC)]),
    "tesserae_nvrtc_get_name": (C.c_char_p, [C.POINTER(NvrtcProgramC)]),
    "tesserae_nvrtc_get_cubin": (C.c_int, [C.POINTER(NvrtcProgramC), C.POINTER(C.c_void_p), C.POINTER(C.c_size_t)]),
    "tesserae_compile_cached": (C.c_int, [C.c_char_p, C.c_char_p, C.POINTER(C.c_char_p), C.c_int,
                                          C.POINTER(C.c_void_p), C.POINTER(C.c_size_t), _IP]),
    "tesserae_cache_dir": (C.c_char_p, []),
    "tesserae_gpu_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "tesserae_gpu_free": (C.c_int, [C.c_void_p]),
    "tesserae_gpu_copy_to_device": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "tesserae_gpu_copy_to_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t]),
    "tesserae_cuinit": (C.c_int, []),
    "tesserae_set_device": (C.c_int, [C.c_int]),
    "tesserae_module_load": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "tesserae_module_unload": (C.c_int, [C.c_void_p]),
    "tesserae_get_function": (C.c_int, [C.c_void_p, C.c_char_p, C.POINTER(C.c_void_p)]),
    "tesserae_launch_kernel": (C.c_int, [C.c_void_p] + [C.c_int] * 7 + [_I64P, C.c_int]),
    "tesserae_launch_kernel_ex": (C.c_int, [C.c_void_p, _IP, _IP, _IP, C.c_int, C.c_void_p,
                                            C.POINTER(LaunchArgC), C.c_int]),
    "tesserae_device_synchronize": (C.c_int, []),
    "tesserae_device_info": (C.c_int, [C.c_char_p, C.c_size_t]),
    "tesserae_device_sm_count": (C.c_int, [_IP]),
    "tesserae_tensor_map_2d": (C.c_int, [C.c_void_p, C.c_int, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64,
                                         C.c_uint32, C.c_uint32, C.c_int]),
    "tesserae_gemm_plan_create": (C.c_int, [C.POINTER(KernelSpecC), C.POINTER(C.c_void_p)]),
    "tesserae_gemm_plan_destroy": (None, [C.c_void_p]),
    "tesserae_gemm_plan_info": (C.c_int, [C.c_void_p, _IP, _IP, _IP, _IP, _IP, C.POINTER(C.c_double)]),
    "tesserae_gemm_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                                    C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "tesserae_gemm_run_scaled": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(GemmScalesC),
                                           C.c_void_p, C.c_float, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "tesserae_gemm_tail_workspace_bytes": (C.c_size_t, [C.c_void_p, C.c_int64, C.c_int64, C.c_int64]),
    "tesserae_gemm_run_scaled_ws": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(GemmScalesC), C.c_void_p,
                                              C.c_float, C.c_int64, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tesserae_gemm_grouped_workspace_bytes": (C.c_size_t, [C.c_int]),
    "tesserae_gemm_run_grouped": (C.c_int, [C.c_void_p, C.POINTER(GemmProblemC), C.c_int, C.c_float, C.c_void_p, C.c_size_t,
                                            C.c_void_p]),
    "tesserae_quantize_fp8_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "tesserae_quantize_fp8_blocks": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_void_p]),
    "tesserae_nvfp4_scale_bytes": (C.c_size_t, [C.c_int64, C.c_int64]),
    "tesserae_quantize_nvfp4": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_float), C.c_void_p, C.c_int64,
                                          C.c_int64, C.c_void_p]),
    "tesserae_nccl_load": (C.c_int, [C.c_char_p]),
    "tesserae_nccl_version": (C.c_int, [C.POINTER(C.c_int)]),
    "tesserae_nccl_unique_id": (C.c_int, [C.c_void_p]),
    "tesserae_nccl_comm_init": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p]),
    "tesserae_nccl_comm_init_deadline": (C.c_int, [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_void_p, C.c_int]),
    "tesserae_nccl_comm_abort": (C.c_int, [C.c_void_p]),
    "tesserae_nccl_comm_destroy": (C.c_int, [C.c_void_p]),
    "tesserae_nccl_reduce_scatter_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tesserae_nccl_all_reduce_f32": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tesserae_wait_selftest": (C.c_int, [C.c_int64, C.POINTER(C.c_uint32), C.POINTER(C.c_int64)]),
    "tesserae_shard_range": (C.c_int, [C.c_int64, C.c_int, C.c_int, C.c_int64, _I64P, _I64P]),
    "tesserae_reduce_cast_bf16": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_float, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tesserae_cast_clear_bf16": (C.c_int, [C.c_void_p, C.c_float, C.c_void_p, C.c_size_t, C.c_void_p]),
    "tesserae_gemm_ksplit_scratch_bytes": (C.c_size_t, [C.c_int64, C.c_int64, C.c_int]),
    "tesserae_gemm_ksplit_partials": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int64,
                                                C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "tesserae_gemm_ksplit_scatter": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int, C.c_int64,
                                               C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "tesserae_gemm_ksplit_run": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t,
                                           C.c_float, C.c_int64, C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "tesserae_gemm_ksplit_noalloc_max_elems": (C.c_size_t, []),
    "tesserae_gemm_ksplit_run_noalloc": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float, C.c_int64,
                                                   C.c_int64, C.c_int64, C.c_int, C.c_void_p]),
    "tesserae_gemm_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "tesserae_gemm_run_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_float,
                                         C.c_int64, C.c_int64, C.c_int64]),
    "tesserae_gemm_run_scaled_host": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(GemmScalesC),
                                                C.c_void_p, C.c_float, C.c_int64, C.c_int64, C.c_int64]),
    "tesserae_runtime_run": (C.c_int, [C.POINTER(KernelSpecC), C.c_int64, C.c_int64, C.c_int64,
                                       C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "tesserae_runtime_is_available": (C.c_int, []),
}

_lib = None


def lib() -> C.CDLL:
    """The loaded library with argument types set; raises if it has not been built."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise ImportError(f"{LIB_PATH} is missing: run `python -m tesserae_b200.build` (needs nvcc); "
                              "tesserae_b200 has no fallback path")
        handle = C.CDLL(str(LIB_PATH))
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)   # AttributeError here = header and library out of step
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def last_error() -> str:
    return (lib().tesserae_last_error() or b"").decode("utf-8", "replace")


class TesseraeError(RuntimeError):
    """A C-ABI call returned non-zero; the message is tesserae_last_error()."""


def check(rc: int, what: str = "") -> None:
    if rc != 0:
        raise TesseraeError(f"{what}: {last_error()}" if what else last_error())


def take_string(ptr) -> str:
    """Copy a char* the library handed out (owned by the caller), then free it."""
    if not ptr:
        return ""
    s = C.string_at(ptr).decode("utf-8", "replace")
    C.CDLL(None).free(C.c_void_p(ptr))
    return s
