"""Python view of the C ABI, named after the reference's OCaml modules so that tests read like
the reference's own (Kernel_ast.make -> KernelSpec, Lower.lower -> lower, Compile.to_source ->
compile_to_source, Runtime.run -> runtime_run).  This layer only marshals arguments; all logic
is in libtesserae_b200.so.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

from . import _native as N
from ._native import TesseraeError, check  # noqa: F401

# Kernel_ast.arch / elem (lib/kernel/kernel_ast.ml:3-13)
SM80, SM90, SM100 = 0, 1, 2
F16, BF16, F32, S8, S32, F8E4M3, F4E2M1 = 0, 1, 2, 3, 4, 5, 6
SCALE_NONE, SCALE_FP8_BLOCK, SCALE_NVFP4 = 0, 1, 2
ROLE_PRODUCER, ROLE_CONSUMER, ROLE_EPILOGUE, ROLE_SCHEDULER = 0, 1, 2, 3
TMA_PAIR = 2
LOWER_ERRORS = {0: "Ok", 1: "UnsupportedArch", 2: "UnsupportedElem", 3: "IncompatibleTile", 4: "MissingArg",
                5: "InvalidPipeline"}


@dataclass
class KernelSpec:
    """Kernel_ast.kernel (lib/kernel/kernel_ast.ml:64-72) plus the extension fields."""
    name: str = "gemm"
    arch: int = SM100
    elem: int = BF16
    tile: tuple = (128, 256, 64)
    stages: int = 0
    cta_group: int = 0
    out_elem: int = 0
    has_bias: int = 0
    scale_mode: int = 0
    scatter: int = 0
    tuning: str = ""
    grouped: int = 0
    _keep: list = field(default_factory=list, repr=False, compare=False)

    def to_c(self) -> N.KernelSpecC:
        name = self.name.encode()
        self._keep.append(name)
        tuning = self.tuning.encode() if self.tuning else None
        self._keep.append(tuning)
        return N.KernelSpecC(name, self.arch, self.elem, self.tile[0], self.tile[1], self.tile[2], self.stages,
                             self.cta_group, self.out_elem, self.has_bias, self.scale_mode, self.scatter, tuning, self.grouped)


class LowerError(Exception):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{LOWER_ERRORS.get(code, code)}: {msg}")
        self.code = code
        self.kind = LOWER_ERRORS.get(code, str(code))


def lower(spec: KernelSpec) -> N.KernelDescC:
    """Lower.lower_exn (lib/kernel/lower.ml:99-104)."""
    d = N.KernelDescC()
    rc = N.lib().tesserae_lower(C.byref(spec.to_c()), C.byref(d))
    if rc != 0:
        raise LowerError(rc, N.last_error())
    return d


@dataclass
class BackendOutput:
    filename: str
    includes: str
    helpers: str
    shared_storage: str
    producer_body: str
    consumer_body: str
    epilogue_body: str
    kernel_func: str
    host_launcher: str
    full_source: str


def backend_emit(spec: KernelSpec) -> BackendOutput:
    """Backend_cute.emit (lib/backend/backend_cute.ml:431-453)."""
    out = N.BackendOutputC()
    rc = N.lib().tesserae_backend_emit(C.byref(spec.to_c()), C.byref(out))
    if rc != 0:
        raise TesseraeError(N.last_error())
    vals = {f: (C.string_at(getattr(out, f)).decode() if getattr(out, f) else "") for f, _ in out._fields_}
    N.lib().tesserae_backend_output_free(C.byref(out))
    return BackendOutput(**vals)


class Tirix:
    """A Tirix program (tesserae_tirix_*): lowered from a spec or parsed from its text form."""

    def __init__(self, handle):
        self._h = handle

    @classmethod
    def lower(cls, spec: KernelSpec) -> "Tirix":
        """Desc_to_tirix.lower (lib/tirix/desc_to_tirix.ml:466-508) after Lower.lower."""
        h = C.c_void_p()
        rc = N.lib().tesserae_tirix_lower(C.byref(spec.to_c()), C.byref(h))
        if rc != 0:
            raise LowerError(rc, N.last_error())
        return cls(h)

    @classmethod
    def parse(cls, text: str) -> "Tirix":
        h = C.c_void_p()
        if N.lib().tesserae_tirix_parse(text.encode(), C.byref(h)) != 0:
            raise ValueError(N.last_error())
        return cls(h)

    def text(self) -> str:
        return N.take_string(N.lib().tesserae_tirix_print(self._h))

    def verify(self) -> list:
        """Tirix_verify.verify (lib/tirix/tirix_verify.ml:9-183): [] when Ok, else the error messages."""
        e = C.c_void_p()
        n = N.lib().tesserae_tirix_verify(self._h, C.byref(e))
        msgs = N.take_string(e.value).split("\n") if e.value else []
        assert n == len(msgs)
        return msgs

    def count_ops(self, name: str) -> int:
        return N.lib().tesserae_tirix_count_ops(self._h, name.encode())

    def emit(self) -> "BackendOutput":
        """Tirix_emit.emit (lib/tirix/tirix_emit.ml:481-501)."""
        out = N.BackendOutputC()
        rc = N.lib().tesserae_tirix_emit(self._h, C.byref(out))
        if rc != 0:
            raise TesseraeError(N.last_error())
        vals = {f: (C.string_at(getattr(out, f)).decode() if getattr(out, f) else "") for f, _ in out._fields_}
        N.lib().tesserae_backend_output_free(C.byref(out))
        return BackendOutput(**vals)

    def __del__(self):
        try:
            if self._h:
                N.lib().tesserae_tirix_free(self._h)
                self._h = None
        except Exception:
            pass


@dataclass
class CompileResult:
    kernel_name: str
    source: str
    cubin: bytes
    cubin_size: int
    duration_ms: float
    cache_hit: bool


def _compile(spec: KernelSpec, fn) -> CompileResult:
    r = N.CompileResultC()
    rc = fn(C.byref(spec.to_c()), C.byref(r))
    if rc != 0:
        raise TesseraeError(N.last_error())
    res = CompileResult(C.string_at(r.kernel_name).decode(), C.string_at(r.source).decode(),
                        C.string_at(r.cubin, r.cubin_size) if r.cubin else b"", r.cubin_size, r.duration_ms,
                        bool(r.cache_hit))
    N.lib().tesserae_compile_result_free(C.byref(r))
    return res


def compile_to_source(spec: KernelSpec) -> CompileResult:
    """Compile.to_source (lib/runtime/compile.ml:36-45)."""
    return _compile(spec, N.lib().tesserae_compile_to_source)


def compile_to_cubin(spec: KernelSpec) -> CompileResult:
    """Compile.to_ptx (lib/runtime/compile.ml:54-75), producing a cached sm_100a cubin."""
    return _compile(spec, N.lib().tesserae_compile_to_cubin)


def _ptr(x) -> C.c_void_p:
    """Device or host address of a torch tensor / numpy array / int."""
    if x is None:
        return C.c_void_p(0)
    if isinstance(x, int):
        return C.c_void_p(x)
    if hasattr(x, "data_ptr"):
        return C.c_void_p(x.data_ptr())
    if hasattr(x, "ctypes"):
        return C.c_void_p(x.ctypes.data)
    raise TypeError(f"cannot take the address of {type(x)}")


class GemmPlan:
    """One compiled GEMM kernel (tesserae_gemm_plan_*).  Needs a GPU."""

    def __init__(self, spec: KernelSpec):
        self.spec = spec
        self._h = C.c_void_p()
        check(N.lib().tesserae_gemm_plan_create(C.byref(spec.to_c()), C.byref(self._h)), "gemm_plan_create")
        cg, bn, st, sm, hit = (C.c_int() for _ in range(5))
        ms = C.c_double()
        check(N.lib().tesserae_gemm_plan_info(self._h, cg, bn, st, sm, hit, ms))
        self.cta_group, self.block_n, self.stages, self.smem_bytes = cg.value, bn.value, st.value, sm.value
        self.cache_hit, self.compile_ms = bool(hit.value), ms.value

    def run(self, a, b, c, bias=None, alpha: float = 1.0, m=None, n=None, k=None, stream=None) -> None:
        """C = alpha * A @ B.T (+ bias) on device buffers; asynchronous on `stream` (a CUDA stream handle)."""
        check(N.lib().tesserae_gemm_run(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(bias), alpha, m, n, k,
                                        C.c_void_p(stream or 0)), "gemm_run")

    def run_scaled(self, a, b, c, scale_a, scale_b, bias=None, alpha: float = 1.0, m=None, n=None, k=None,
                   stream=None, global_a: float = 1.0, global_b: float = 1.0) -> None:
        """Block-scaled variant: scale_a / scale_b are device buffers in the layout the spec's scale_mode names."""
        sc = N.GemmScalesC(_ptr(scale_a), _ptr(scale_b), global_a, global_b)
        check(N.lib().tesserae_gemm_run_scaled(self._h, _ptr(a), _ptr(b), _ptr(c), C.byref(sc), _ptr(bias), alpha,
                                               m, n, k, C.c_void_p(stream or 0)), "gemm_run_scaled")

    def tail_workspace_bytes(self, m: int, n: int, k: int) -> int:
        """Bytes of zero-filled workspace run_scaled_ws wants for this problem (0: no stream-K tail is used)."""
        return N.lib().tesserae_gemm_tail_workspace_bytes(self._h, m, n, k)

    def run_scaled_ws(self, a, b, c, scale_a, scale_b, workspace, workspace_bytes: int, bias=None, alpha: float = 1.0,
                      m=None, n=None, k=None, stream=None) -> None:
        """FP8 block-scaled GEMM with a stream-K tail through `workspace` (zero-filled before first use)."""
        sc = N.GemmScalesC(_ptr(scale_a), _ptr(scale_b), 1.0, 1.0)
        check(N.lib().tesserae_gemm_run_scaled_ws(self._h, _ptr(a), _ptr(b), _ptr(c), C.byref(sc), _ptr(bias), alpha, m, n, k,
                                                  _ptr(workspace), workspace_bytes, C.c_void_p(stream or 0)), "gemm_run_scaled_ws")

    def run_grouped(self, problems, workspace, workspace_bytes: int, alpha: float = 1.0, stream=None) -> None:
        """Grouped GEMM: `problems` is a list of (a, b, c, bias, m, n, k) with device buffers; one launch."""
        arr = (N.GemmProblemC * len(problems))()
        for i, (a, b, c, bias, m, n, k) in enumerate(problems):
            arr[i] = N.GemmProblemC(_ptr(a), _ptr(b), _ptr(c), _ptr(bias), m, n, k)
        check(N.lib().tesserae_gemm_run_grouped(self._h, arr, len(problems), alpha, _ptr(workspace), workspace_bytes,
                                                C.c_void_p(stream or 0)), "gemm_run_grouped")

    def ksplit_partials(self, a, b, scratch, scratch_bytes, m, n, k, k_splits=1, stream=None) -> None:
        """fp32 partial products of each K slice into scratch[s] (device buffers)."""
        check(N.lib().tesserae_gemm_ksplit_partials(self._h, _ptr(a), _ptr(b), _ptr(scratch), scratch_bytes, m, n, k,
                                                    k_splits, C.c_void_p(stream or 0)), "gemm_ksplit_partials")

    def ksplit_scatter(self, a, b, dst_ptrs, rows_per_owner, m, n, k, stream=None, start_owner: int = 0) -> None:
        """fp32 partial product with rows [g*rows_per_owner, ...) stored to dst_ptrs[g] (device addresses, local or
        peer-mapped): the K-split GEMM with the scatter half of the reduce-scatter in its epilogue."""
        arr = (C.c_void_p * len(dst_ptrs))(*[int(p) for p in dst_ptrs])
        check(N.lib().tesserae_gemm_ksplit_scatter(self._h, _ptr(a), _ptr(b), arr, len(dst_ptrs), rows_per_owner, start_owner,
                                                   m, n, k, C.c_void_p(stream or 0)), "gemm_ksplit_scatter")

    def ksplit_run(self, a, b, c, scratch, scratch_bytes, m, n, k, k_splits=1, alpha: float = 1.0, stream=None) -> None:
        """K-split GEMM on one GPU: partials into scratch, then sum + bf16 cast into c."""
        check(N.lib().tesserae_gemm_ksplit_run(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(scratch), scratch_bytes, alpha,
                                               m, n, k, k_splits, C.c_void_p(stream or 0)), "gemm_ksplit_run")

    def run_host(self, a, b, c, bias=None, alpha: float = 1.0, m=None, n=None, k=None) -> None:
        """Same with host buffers: H2D copies, launch, D2H copy inside the call."""
        check(N.lib().tesserae_gemm_run_host(self._h, _ptr(a), _ptr(b), _ptr(c), _ptr(bias), alpha, m, n, k),
              "gemm_run_host")

    def run_scaled_host(self, a, b, c, scale_a, scale_b, bias=None, alpha: float = 1.0, m=None, n=None, k=None,
                        global_a: float = 1.0, global_b: float = 1.0) -> None:
        """Block-scaled GEMM with host buffers (operands, scale tables, bias up; C back) inside the call."""
        sc = N.GemmScalesC(_ptr(scale_a), _ptr(scale_b), global_a, global_b)
        check(N.lib().tesserae_gemm_run_scaled_host(self._h, _ptr(a), _ptr(b), _ptr(c), C.byref(sc), _ptr(bias), alpha,
                                                    m, n, k), "gemm_run_scaled_host")

    def status(self) -> int:
        s = C.c_uint32()
        check(N.lib().tesserae_gemm_status(self._h, C.byref(s)), "gemm_status")
        return s.value

    def close(self) -> None:
        if self._h:
            N.lib().tesserae_gemm_plan_destroy(self._h)
            self._h = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def runtime_run(spec: KernelSpec, m: int, n: int, k: int, a, b):
    """Runtime.run (lib/runtime/runtime.ml:15-75): float arrays in, float array out (numpy)."""
    import numpy as np
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    if a.size != m * k or b.size != n * k:
        raise ValueError("a must hold m*k and b must hold n*k floats")
    c = np.empty(m * n, dtype=np.float32)
    fp = C.POINTER(C.c_float)
    check(N.lib().tesserae_runtime_run(C.byref(spec.to_c()), m, n, k, a.ctypes.data_as(fp), b.ctypes.data_as(fp),
                                       c.ctypes.data_as(fp)), "runtime_run")
    return c


def reduce_cast_bf16(parts, n_parts: int, part_stride: int, out, n: int, alpha: float = 1.0, stream=None) -> None:
    """out[i] = bf16(alpha * sum_p parts[p * part_stride + i]) on device buffers."""
    check(N.lib().tesserae_reduce_cast_bf16(_ptr(parts), n_parts, part_stride, alpha, _ptr(out), n,
                                            C.c_void_p(stream or 0)), "reduce_cast_bf16")


def cast_clear_bf16(acc, out, n: int, alpha: float = 1.0, stream=None) -> None:
    """out[i] = bf16(alpha * acc[i]); acc[i] = 0 (device buffers)."""
    check(N.lib().tesserae_cast_clear_bf16(_ptr(acc), alpha, _ptr(out), n, C.c_void_p(stream or 0)), "cast_clear_bf16")


def quantize_fp8_rows(x, q, scale, m: int, k: int, stream=None) -> None:
    check(N.lib().tesserae_quantize_fp8_rows(_ptr(x), _ptr(q), _ptr(scale), m, k, C.c_void_p(stream or 0)), "quantize_fp8_rows")


def quantize_fp8_blocks(w, q, scale, n: int, k: int, stream=None) -> None:
    check(N.lib().tesserae_quantize_fp8_blocks(_ptr(w), _ptr(q), _ptr(scale), n, k, C.c_void_p(stream or 0)), "quantize_fp8_blocks")


def nvfp4_scale_bytes(rows: int, k: int) -> int:
    return N.lib().tesserae_nvfp4_scale_bytes(rows, k)


def quantize_nvfp4(x, q, scale_chunks, workspace4, rows: int, k: int, stream=None) -> float:
    """Returns the per-tensor scale (host float); synchronises the stream."""
    g = C.c_float()
    check(N.lib().tesserae_quantize_nvfp4(_ptr(x), _ptr(q), _ptr(scale_chunks), C.byref(g), _ptr(workspace4), rows, k,
                                          C.c_void_p(stream or 0)), "quantize_nvfp4")
    return g.value


class NcclComm:
    """NCCL communicator through the C ABI (one per GPU, created with that GPU current)."""

    def __init__(self, world: int, rank: int, unique_id: bytes):
        assert len(unique_id) == 128
        self._buf = C.create_string_buffer(unique_id, 128)
        self._h = C.c_void_p()
        check(N.lib().tesserae_nccl_comm_init(C.byref(self._h), world, rank, self._buf), "nccl_comm_init")
        self.world, self.rank = world, rank

    def reduce_scatter_f32(self, send, recv, recv_count: int, stream=None) -> None:
        check(N.lib().tesserae_nccl_reduce_scatter_f32(self._h, _ptr(send), _ptr(recv), recv_count, C.c_void_p(stream or 0)),
              "nccl_reduce_scatter_f32")

    def all_reduce_f32(self, send, recv, count: int, stream=None) -> None:
        check(N.lib().tesserae_nccl_all_reduce_f32(self._h, _ptr(send), _ptr(recv), count, C.c_void_p(stream or 0)),
              "nccl_all_reduce_f32")

    def close(self) -> None:
        if self._h:
            check(N.lib().tesserae_nccl_comm_destroy(self._h), "nccl_comm_destroy")
            self._h = C.c_void_p()


def nccl_load(path: str | None = None) -> None:
    check(N.lib().tesserae_nccl_load(path.encode() if path else None), "nccl_load")


def nccl_version() -> int:
    v = C.c_int()
    check(N.lib().tesserae_nccl_version(C.byref(v)), "nccl_version")
    return v.value


def nccl_unique_id() -> bytes:
    buf = C.create_string_buffer(128)
    check(N.lib().tesserae_nccl_unique_id(buf), "nccl_unique_id")
    return buf.raw


def wait_selftest(budget_cycles: int = 200_000):
    """(status bits, cycles waited) of a wait on a barrier that nothing signals; status must be 0x40."""
    st, w = C.c_uint32(), C.c_int64()
    check(N.lib().tesserae_wait_selftest(budget_cycles, C.byref(st), C.byref(w)), "wait_selftest")
    return st.value, w.value


def shard_range(total: int, parts: int, index: int, align: int = 1):
    """(begin, length) of shard `index` of `parts` over [0, total), boundaries at multiples of `align`."""
    b, n = C.c_int64(), C.c_int64()
    check(N.lib().tesserae_shard_range(total, parts, index, align, C.byref(b), C.byref(n)), "shard_range")
    return b.value, n.value


def grouped_workspace_bytes(n_problems: int) -> int:
    return N.lib().tesserae_gemm_grouped_workspace_bytes(n_problems)


def ksplit_scratch_bytes(m: int, n: int, k_splits: int = 1) -> int:
    return N.lib().tesserae_gemm_ksplit_scratch_bytes(m, n, k_splits)


def is_available() -> bool:
    """Runtime.is_available (lib/runtime/runtime.ml:7-9)."""
    return bool(N.lib().tesserae_runtime_is_available())


def device_info() -> str:
    buf = C.create_string_buffer(256)
    check(N.lib().tesserae_device_info(buf, 256), "device_info")
    return buf.value.decode()


# ---------------------------------------------------------------- integer maps
def _arr(xs):
    xs = list(xs)
    return (C.c_int64 * max(len(xs), 1))(*xs), len(xs)


def swizzle_apply(b: int, m: int, s: int, offset: int) -> int:
    r = N.lib().tesserae_swizzle_apply(b, m, s, offset)
    if r == -1 and (b < 0 or m < 0 or s < 0):
        raise ValueError(N.last_error())
    return r


def swizzle_smem_selector(elem: int, tile_m: int, tile_k: int):
    b, m, s = C.c_int(), C.c_int(), C.c_int()
    check(N.lib().tesserae_swizzle_smem_selector(elem, tile_m, tile_k, b, m, s))
    return b.value, m.value, s.value


def swizzle_apply_to_strides(b: int, m: int, s: int, stride):
    """Swizzle.apply_to_layout on the flattened strides of a layout (its shape does not change)."""
    d, n = _arr(stride)
    out = (C.c_int64 * max(n, 1))()
    check(N.lib().tesserae_swizzle_apply_to_strides(b, m, s, d, n, out), "swizzle_apply_to_strides")
    return [out[i] for i in range(n)]


def layout_cosize(shape, stride) -> int:
    s, n = _arr(shape)
    d, _ = _arr(stride)
    return N.lib().tesserae_layout_cosize(s, d, n)


def layout_idx(stride, coord) -> int:
    d, n = _arr(stride)
    c, _ = _arr(coord)
    return N.lib().tesserae_layout_idx(d, c, n)


def _layout_out(rc, os, od):
    if rc < 0:
        raise ValueError(N.last_error())
    return list(os[:rc]), list(od[:rc])


def layout_compose(outer, inner):
    os_, no = _arr(outer[0]); od_, _ = _arr(outer[1])
    is_, ni = _arr(inner[0]); id_, _ = _arr(inner[1])
    out = (C.c_int64 * max(ni, 1))()
    rc = N.lib().tesserae_layout_compose(os_, od_, no, is_, id_, ni, out)
    if rc < 0:
        raise ValueError(N.last_error())
    return list(inner[0]), list(out[:rc])


def _unary(fn, shape, stride, *extra, nout=None):
    s, n = _arr(shape)
    d, _ = _arr(stride)
    cap = nout or (n + 1)
    os_ = (C.c_int64 * cap)(); od_ = (C.c_int64 * cap)()
    return _layout_out(fn(s, d, n, *extra, os_, od_), os_, od_)


def layout_tile(shape, stride, tile):
    t, _ = _arr(tile)
    return _unary(N.lib().tesserae_layout_tile, shape, stride, t, nout=2 * len(list(shape)) + 1)


def layout_sort(shape, stride):
    return _unary(N.lib().tesserae_layout_sort, shape, stride)


def layout_coalesce(shape, stride):
    return _unary(N.lib().tesserae_layout_coalesce, shape, stride)


def layout_is_admissible(shape, stride, m: int) -> bool:
    s, n = _arr(shape)
    d, _ = _arr(stride)
    return bool(N.lib().tesserae_layout_is_admissible(s, d, n, m))


def layout_complement(shape, stride, m: int):
    return _unary(N.lib().tesserae_layout_complement, shape, stride, m)


def layout_flat_divide(shape, stride, divisor: int):
    return _unary(N.lib().tesserae_layout_flat_divide, shape, stride, divisor)


def layout_logical_divide(shape, stride, tile_shape):
    t, _ = _arr(tile_shape)
    return _unary(N.lib().tesserae_layout_logical_divide, shape, stride, t, nout=2 * len(list(shape)) + 1)


# ---------------------------------------------------------------- Memspace, atoms, tiled atoms, Tile_op
SPACES = {"global": 0, "shared": 1, "register": 2, "tensor": 3}
ELEMS = {"f16": F16, "bf16": BF16, "f32": F32, "s8": S8, "s32": S32}
MAJORS = {"RowMajor": 0, "ColMajor": 1}
MMA_ATOM_IDS = {name: i for i, name in enumerate([
    "sm80_16x8x8_f32f16f16f32", "sm80_16x8x16_f32f16f16f32", "sm80_16x8x16_f32bf16bf16f32", "sm80_16x8x32_s32s8s8s32",
    "sm90_64x64x16_f32f16f16f32", "sm90_64x128x16_f32f16f16f32", "sm90_64x64x16_f32bf16bf16f32",
    "sm100_64x64x16_f32f16f16f32", "sm100_128x128x16_f32f16f16f32", "sm100_64x64x32_s32s8s8s32"])}
COPY_KINDS = {"AsyncCopyGlobal": 0, "AsyncCopyCached": 1, "TmaLoad": 2, "TmaStore": 3, "TmaLoadPair": 4, "Ldmatrix": 5,
              "LdmatrixTrans": 6, "UniversalCopy": 7}
TILE_OP_TEXT = {"mma": 0, "commit": 1, "accum_decl": 2, "tmem_alloc": 3, "tmem_dealloc": 4}


def _text(fn, *args) -> str:
    buf = C.create_string_buffer(4096)
    if fn(*args, buf, 4096) != 0:
        raise ValueError(N.last_error())
    return buf.value.decode()


def memspace_can_transfer(src: str, dst: str) -> bool:
    """Memspace.can_transfer (lib/core/memspace.ml:26-47)."""
    return bool(N.lib().tesserae_memspace_can_transfer(SPACES[src], SPACES[dst]))


def memspace_name(space: str) -> str:
    return N.lib().tesserae_memspace_name(SPACES[space]).decode()


def mma_atom(name: str, a_major: str = "ColMajor", b_major: str = "RowMajor") -> N.MmaAtomC:
    """One of the reference's Mma_atom constructors (lib/atoms/mma_atom.ml:32-112)."""
    a = N.MmaAtomC()
    if N.lib().tesserae_mma_atom_make(MMA_ATOM_IDS[name], MAJORS[a_major], MAJORS[b_major], C.byref(a)) != 0:
        raise ValueError(N.last_error())
    return a


def mma_atom_thread_count(a) -> int:
    return N.lib().tesserae_mma_atom_thread_count(C.byref(a))


def mma_atom_is_wgmma(a) -> bool:
    return bool(N.lib().tesserae_mma_atom_is_wgmma(C.byref(a)))


def mma_atom_emit_cpp(a) -> str:
    return _text(N.lib().tesserae_mma_atom_emit_cpp, C.byref(a))


def copy_atom(kind: str, elem: str, src: str = "global", dst: str = "shared") -> N.CopyAtomC:
    """One of the reference's Copy_atom constructors (lib/atoms/copy_atom.ml:23-104)."""
    a = N.CopyAtomC()
    if N.lib().tesserae_copy_atom_make(COPY_KINDS[kind], ELEMS[elem], SPACES[src], SPACES[dst], C.byref(a)) != 0:
        raise ValueError(N.last_error())
    return a


def copy_atom_is_async(a) -> bool:
    return bool(N.lib().tesserae_copy_atom_is_async(C.byref(a)))


def copy_atom_is_tma(a) -> bool:
    return bool(N.lib().tesserae_copy_atom_is_tma(C.byref(a)))


def copy_atom_requires_mbar(a) -> bool:
    return bool(N.lib().tesserae_copy_atom_requires_mbar(C.byref(a)))


def copy_atom_emit_cpp(a) -> str:
    return _text(N.lib().tesserae_copy_atom_emit_cpp, C.byref(a))


def tiled_mma(atom, thread_layout_size: int, warp_layout_size: int, tiler_m: int, tiler_n: int) -> N.TiledMmaC:
    """Tiled_mma.make and its derived numbers (lib/atoms/tiled_mma.ml:12-53)."""
    t = N.TiledMmaC()
    if N.lib().tesserae_tiled_mma_make(C.byref(atom), thread_layout_size, warp_layout_size, tiler_m, tiler_n, C.byref(t)) != 0:
        raise ValueError(N.last_error())
    return t


def tiled_copy(atom, thread_layout_size: int, val_layout_size: int) -> N.TiledCopyC:
    """Tiled_copy.make and its derived numbers (lib/atoms/tiled_copy.ml:10-36)."""
    t = N.TiledCopyC()
    if N.lib().tesserae_tiled_copy_make(C.byref(atom), thread_layout_size, val_layout_size, C.byref(t)) != 0:
        raise ValueError(N.last_error())
    return t


def tiled_copy_partition(thread_count: int, shape, stride):
    """Tiled_copy.partition_src / partition_dst (lib/atoms/tiled_copy.ml:38-50): (shape, stride) of the one mode."""
    s, n = _arr(shape)
    d, _ = _arr(stride)
    os_, od_ = C.c_int64(), C.c_int64()
    if N.lib().tesserae_tiled_copy_partition(thread_count, s, d, n, C.byref(os_), C.byref(od_)) < 0:
        raise ValueError(N.last_error())
    return os_.value, od_.value


def tile_op(atom, thread_layout_size: int, warp_layout_size: int, tiler_m: int, tiler_n: int, accum: str,
            tmem=None, double_buf: bool = False) -> N.TileOpC:
    """Tile_op.make (lib/pipeline/tile_op.ml:18-37); tmem = (cta_group, num_cols, num_rows) or None."""
    t = N.TileOpC()
    t.atom = atom
    t.thread_layout_size, t.warp_layout_size, t.tiler_m, t.tiler_n = thread_layout_size, warp_layout_size, tiler_m, tiler_n
    t.accum_loc = {"Registers": 0, "TensorMem": 1}[accum]
    t.has_tmem = int(tmem is not None)
    if tmem is not None:
        t.tmem_cta_group, t.tmem_cols, t.tmem_rows = tmem
    t.double_buf = int(double_buf)
    if N.lib().tesserae_tile_op_check(C.byref(t)) != 0:
        raise ValueError(N.last_error())
    return t


def tile_op_is_tmem(t) -> bool:
    return bool(N.lib().tesserae_tile_op_is_tmem(C.byref(t)))


def tile_op_is_wgmma(t) -> bool:
    return bool(N.lib().tesserae_tile_op_is_wgmma(C.byref(t)))


def tile_op_accum_elems_per_thread(t) -> int:
    return N.lib().tesserae_tile_op_accum_elems_per_thread(C.byref(t))


def tile_op_emit(t, what: str, arg0: str = "", arg1: str = "", flag: int = 0) -> str:
    """Tile_op.emit_mma / emit_commit / emit_accum_decl / emit_tmem_alloc / emit_tmem_dealloc (lib/pipeline/tile_op.ml:52-107)."""
    return _text(N.lib().tesserae_tile_op_emit, C.byref(t), TILE_OP_TEXT[what], arg0.encode(), arg1.encode(), flag)
