/* OCaml-runtime glue between tesserae's `external` declarations and libtesserae_b200.
 *
 * One file replaces the reference's three stub files (lib/runtime/nvrtc_stub.c:109-192,
 * lib/runtime/gpu_buffer_stubs.c:26-83, lib/kernel/kernel_launch_stubs.c:21-107): every caml_* symbol the
 * OCaml side names (lib/runtime/nvrtc.ml:15-31, lib/runtime/gpu_buffer.ml:9-13, lib/kernel/kernel_launch.ml:12-30)
 * is a few lines over the plain-C function of the same name in include/tesserae_b200.h.  The last section adds
 * the externals of the new GEMM plan path.
 *
 * Status: NOT linked against an OCaml runtime.  No OCaml toolchain exists where this library is built, so this
 * file is only checked to parse and type-check (gcc -fsyntax-only -Wall -Wextra -Werror) against a minimal
 * stand-in for <caml/...> kept with the tests; what it proves is that the glue calls tesserae_* with the right
 * argument types.  A maintainer with the toolchain adds it as `foreign_stubs` in the dune files of lib/runtime and lib/kernel.
 *
 * Conventions kept from the reference: a failing call raises Failure with the library's message
 * (kernel_launch_stubs.c:8-19); `compile` is the one call that returns a result instead of raising
 * (nvrtc_stub.c:137-169); handles are custom blocks whose finaliser releases the native object; nothing
 * releases the runtime lock.
 */
#include <string.h>

#include <caml/mlvalues.h>
#include <caml/memory.h>
#include <caml/alloc.h>
#include <caml/fail.h>
#include <caml/custom.h>

#include "tesserae_b200.h"

#define TS_CHECK(rc) do { if ((rc) != 0) caml_failwith(tesserae_last_error()); } while (0)
#define TS_PTR(v) (*(void**)Data_custom_val(v))

/* ------------------------------------------------------------------ lib/kernel/kernel_launch.ml:12-30 */
CAMLprim value caml_cuinit(value unit) {
    CAMLparam1(unit);
    TS_CHECK(tesserae_cuinit());
    CAMLreturn(Val_unit);
}

CAMLprim value caml_module_load_ptx(value image) {           /* PTX text or cubin bytes */
    CAMLparam1(image);
    void* m = NULL;
    TS_CHECK(tesserae_module_load(String_val(image), &m));
    CAMLreturn(caml_copy_nativeint((intnat)m));
}

CAMLprim value caml_module_unload(value m) {
    CAMLparam1(m);
    TS_CHECK(tesserae_module_unload((void*)Nativeint_val(m)));
    CAMLreturn(Val_unit);
}

CAMLprim value caml_get_function(value m, value name) {
    CAMLparam2(m, name);
    void* f = NULL;
    TS_CHECK(tesserae_get_function((void*)Nativeint_val(m), String_val(name), &f));
    CAMLreturn(caml_copy_nativeint((intnat)f));
}

CAMLprim value caml_launch_kernel(value fn, value gx, value gy, value gz, value bx, value by, value bz,
                                  value smem, value args) {
    CAMLparam5(fn, gx, gy, gz, bx);
    CAMLxparam4(by, bz, smem, args);
    int64_t slots[64];
    mlsize_t n = Wosize_val(args), i;
    if (n > 64) caml_failwith("launch_kernel: too many arguments");
    for (i = 0; i < n; i++) slots[i] = (int64_t)Nativeint_val(Field(args, i));
    TS_CHECK(tesserae_launch_kernel((void*)Nativeint_val(fn), Int_val(gx), Int_val(gy), Int_val(gz),
                                    Int_val(bx), Int_val(by), Int_val(bz), Int_val(smem), slots, (int)n));
    CAMLreturn(Val_unit);
}

CAMLprim value caml_launch_kernel_bytecode(value* argv, int argc) {
    (void)argc;
    return caml_launch_kernel(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7], argv[8]);
}

CAMLprim value caml_device_synchronize(value unit) {
    CAMLparam1(unit);
    TS_CHECK(tesserae_device_synchronize());
    CAMLreturn(Val_unit);
}

CAMLprim value caml_device_info(value unit) {
    CAMLparam1(unit);
    char buf[256];
    TS_CHECK(tesserae_device_info(buf, sizeof buf));
    CAMLreturn(caml_copy_string(buf));
}

/* ------------------------------------------------------------------ lib/runtime/gpu_buffer.ml:9-13 */
static void ts_buffer_finalize(value v) { tesserae_gpu_free(TS_PTR(v)); }

static struct custom_operations ts_buffer_ops = {
    "tesserae_b200.gpu_buffer", ts_buffer_finalize, custom_compare_default, custom_hash_default,
    custom_serialize_default, custom_deserialize_default, custom_compare_ext_default, custom_fixed_length_default
};

CAMLprim value caml_gpu_alloc(value n_bytes) {
    CAMLparam1(n_bytes);
    CAMLlocal1(block);
    void* p = NULL;
    TS_CHECK(tesserae_gpu_alloc((size_t)Long_val(n_bytes), &p));
    block = caml_alloc_custom(&ts_buffer_ops, sizeof(void*), 0, 1);
    TS_PTR(block) = p;
    CAMLreturn(block);
}

CAMLprim value caml_gpu_free(value h) {                      /* idempotent */
    CAMLparam1(h);
    TS_CHECK(tesserae_gpu_free(TS_PTR(h)));
    TS_PTR(h) = NULL;
    CAMLreturn(Val_unit);
}

CAMLprim value caml_gpu_copy_to_device(value h, value src, value n_bytes) {
    CAMLparam3(h, src, n_bytes);
    TS_CHECK(tesserae_gpu_copy_to_device(TS_PTR(h), Bytes_val(src), (size_t)Long_val(n_bytes)));
    CAMLreturn(Val_unit);
}

CAMLprim value caml_gpu_copy_to_host(value dst, value h, value n_bytes) {
    CAMLparam3(dst, h, n_bytes);
    TS_CHECK(tesserae_gpu_copy_to_host(Bytes_val(dst), TS_PTR(h), (size_t)Long_val(n_bytes)));
    CAMLreturn(Val_unit);
}

CAMLprim value caml_gpu_ptr(value h) {
    CAMLparam1(h);
    CAMLreturn(caml_copy_nativeint((intnat)TS_PTR(h)));
}

/* The reference's gpu_buffer.ml:9 spells its first external "ocaml_gpu_alloc"; keep that name alive too. */
CAMLprim value ocaml_gpu_alloc(value n_bytes) { return caml_gpu_alloc(n_bytes); }

/* ------------------------------------------------------------------ lib/runtime/nvrtc.ml:15-31 */
static void ts_program_finalize(value v) {
    tesserae_nvrtc_destroy((tesserae_nvrtc_program*)TS_PTR(v));
    TS_PTR(v) = NULL;
}

static struct custom_operations ts_program_ops = {
    "tesserae_b200.nvrtc_program", ts_program_finalize, custom_compare_default, custom_hash_default,
    custom_serialize_default, custom_deserialize_default, custom_compare_ext_default, custom_fixed_length_default
};

CAMLprim value caml_nvrtc_create(value source, value name) {
    CAMLparam2(source, name);
    CAMLlocal1(block);
    tesserae_nvrtc_program* p = tesserae_nvrtc_create(String_val(source), String_val(name));   /* copies both */
    if (p == NULL) caml_failwith("nvrtc_create: allocation failed");
    block = caml_alloc_custom(&ts_program_ops, sizeof(void*), 0, 1);
    TS_PTR(block) = p;
    CAMLreturn(block);
}

CAMLprim value caml_nvrtc_destroy(value prog) {              /* idempotent: the pointer is cleared */
    CAMLparam1(prog);
    tesserae_nvrtc_destroy((tesserae_nvrtc_program*)TS_PTR(prog));
    TS_PTR(prog) = NULL;
    CAMLreturn(Val_unit);
}

CAMLprim value caml_nvrtc_is_valid(value prog) {
    CAMLparam1(prog);
    tesserae_nvrtc_program* p = (tesserae_nvrtc_program*)TS_PTR(prog);
    CAMLreturn(Val_bool(p != NULL && tesserae_nvrtc_is_valid(p)));
}

/* program -> string list -> (unit, string) result: Ok () is a block of tag 0, Error log a block of tag 1. */
CAMLprim value caml_nvrtc_compile(value prog, value opts) {
    CAMLparam2(prog, opts);
    CAMLlocal3(result, log, cell);
    const char* argv[64];
    int argc = 0, rc;
    tesserae_nvrtc_program* p = (tesserae_nvrtc_program*)TS_PTR(prog);
    if (p == NULL) caml_failwith("nvrtc_compile: program was destroyed");
    for (cell = opts; cell != Val_emptylist && argc < 64; cell = Field(cell, 1))
        argv[argc++] = String_val(Field(cell, 0));           /* valid until the next allocation; none happens before the call returns */
    rc = tesserae_nvrtc_compile(p, argv, argc);
    if (rc == 0) {
        result = caml_alloc(1, 0);
        Store_field(result, 0, Val_unit);
    } else {
        char* text = tesserae_nvrtc_get_log(p);              /* malloc'ed copy, or NULL */
        log = caml_copy_string(text != NULL ? text : tesserae_last_error());
        free(text);
        result = caml_alloc(1, 1);
        Store_field(result, 0, log);
    }
    CAMLreturn(result);
}

CAMLprim value caml_nvrtc_get_ptx(value prog) {
    CAMLparam1(prog);
    CAMLlocal1(out);
    tesserae_nvrtc_program* p = (tesserae_nvrtc_program*)TS_PTR(prog);
    char* text = p != NULL ? tesserae_nvrtc_get_ptx(p) : NULL;
    if (text == NULL) caml_failwith("get_ptx: not compiled or failed");
    out = caml_copy_string(text);
    free(text);
    CAMLreturn(out);
}

CAMLprim value caml_nvrtc_get_log(value prog) {
    CAMLparam1(prog);
    CAMLlocal1(out);
    tesserae_nvrtc_program* p = (tesserae_nvrtc_program*)TS_PTR(prog);
    char* text = p != NULL ? tesserae_nvrtc_get_log(p) : NULL;
    out = caml_copy_string(text != NULL ? text : "");
    free(text);
    CAMLreturn(out);
}

/* ------------------------------------------------------------------ new externals: GEMM plans
 *   type plan
 *   external plan_create : name:string -> arch:int -> elem:int -> tile:(int * int * int) -> stages:int ->
 *                          cta_group:int -> out_elem:int -> has_bias:bool -> scale_mode:int -> plan
 *                        = "caml_gemm_plan_create_bytecode" "caml_gemm_plan_create"
 *   external plan_run    : plan -> a:nativeint -> b:nativeint -> c:nativeint -> bias:nativeint -> alpha:float ->
 *                          m:int -> n:int -> k:int -> unit = "caml_gemm_plan_run_bytecode" "caml_gemm_plan_run"
 *   external plan_status : plan -> int = "caml_gemm_plan_status"
 *   external runtime_run : name:string -> elem:int -> tile:(int * int * int) -> m:int -> n:int -> k:int ->
 *                          float array -> float array -> float array = "caml_runtime_run_bytecode" "caml_runtime_run"
 */
static void ts_plan_finalize(value v) {
    tesserae_gemm_plan_destroy((tesserae_gemm_plan*)TS_PTR(v));
    TS_PTR(v) = NULL;
}

static struct custom_operations ts_plan_ops = {
    "tesserae_b200.gemm_plan", ts_plan_finalize, custom_compare_default, custom_hash_default,
    custom_serialize_default, custom_deserialize_default, custom_compare_ext_default, custom_fixed_length_default
};

CAMLprim value caml_gemm_plan_create(value name, value arch, value elem, value tile, value stages,
                                     value cta_group, value out_elem, value has_bias, value scale_mode) {
    CAMLparam5(name, arch, elem, tile, stages);
    CAMLxparam4(cta_group, out_elem, has_bias, scale_mode);
    CAMLlocal1(block);
    tesserae_kernel_spec spec;
    tesserae_gemm_plan* plan = NULL;
    memset(&spec, 0, sizeof spec);
    spec.name = String_val(name);                            /* read before anything below allocates */
    spec.arch = Int_val(arch);
    spec.elem = Int_val(elem);
    spec.tile_m = Int_val(Field(tile, 0));
    spec.tile_n = Int_val(Field(tile, 1));
    spec.tile_k = Int_val(Field(tile, 2));
    spec.stages = Int_val(stages);
    spec.cta_group = Int_val(cta_group);
    spec.out_elem = Int_val(out_elem);
    spec.has_bias = Bool_val(has_bias);
    spec.scale_mode = Int_val(scale_mode);
    TS_CHECK(tesserae_gemm_plan_create(&spec, &plan));
    block = caml_alloc_custom(&ts_plan_ops, sizeof(void*), 0, 1);
    TS_PTR(block) = plan;
    CAMLreturn(block);
}

CAMLprim value caml_gemm_plan_create_bytecode(value* argv, int argc) {
    (void)argc;
    return caml_gemm_plan_create(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7], argv[8]);
}

CAMLprim value caml_gemm_plan_run(value plan, value a, value b, value c, value bias, value alpha,
                                  value m, value n, value k) {
    CAMLparam5(plan, a, b, c, bias);
    CAMLxparam4(alpha, m, n, k);
    tesserae_gemm_plan* p = (tesserae_gemm_plan*)TS_PTR(plan);
    if (p == NULL) caml_failwith("gemm_plan_run: plan was destroyed");
    TS_CHECK(tesserae_gemm_run(p, (const void*)Nativeint_val(a), (const void*)Nativeint_val(b), (void*)Nativeint_val(c),
                               (const void*)Nativeint_val(bias), (float)Double_val(alpha),
                               (int64_t)Long_val(m), (int64_t)Long_val(n), (int64_t)Long_val(k), NULL));
    CAMLreturn(Val_unit);
}

CAMLprim value caml_gemm_plan_run_bytecode(value* argv, int argc) {
    (void)argc;
    return caml_gemm_plan_run(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7], argv[8]);
}

CAMLprim value caml_gemm_plan_status(value plan) {
    CAMLparam1(plan);
    uint32_t status = 0;
    tesserae_gemm_plan* p = (tesserae_gemm_plan*)TS_PTR(plan);
    if (p == NULL) caml_failwith("gemm_plan_status: plan was destroyed");
    TS_CHECK(tesserae_gemm_status(p, &status));
    CAMLreturn(Val_long((long)status));
}

/* Runtime.run (lib/runtime/runtime.ml:15-75) in one call: float arrays in, float array out. */
CAMLprim value caml_runtime_run(value name, value elem, value tile, value m, value n, value k, value a, value b) {
    CAMLparam5(name, elem, tile, m, n);
    CAMLxparam3(k, a, b);
    CAMLlocal1(out);
    const int64_t mi = Long_val(m), ni = Long_val(n), ki = Long_val(k);
    const mlsize_t na = Wosize_val(a) / Double_wosize, nb = Wosize_val(b) / Double_wosize;
    float *fa, *fb, *fc;
    tesserae_kernel_spec spec;
    mlsize_t i;
    int rc;
    if (mi <= 0 || ni <= 0 || ki <= 0 || (int64_t)na != mi * ki || (int64_t)nb != ni * ki)
        caml_failwith("runtime_run: array sizes do not match m, n, k");
    fa = (float*)malloc(sizeof(float) * (size_t)na);
    fb = (float*)malloc(sizeof(float) * (size_t)nb);
    fc = (float*)malloc(sizeof(float) * (size_t)(mi * ni));
    if (fa == NULL || fb == NULL || fc == NULL) { free(fa); free(fb); free(fc); caml_failwith("runtime_run: out of memory"); }
    for (i = 0; i < na; i++) fa[i] = (float)Double_flat_field(a, i);
    for (i = 0; i < nb; i++) fb[i] = (float)Double_flat_field(b, i);
    memset(&spec, 0, sizeof spec);
    spec.name = String_val(name);
    spec.arch = TESSERAE_SM100;
    spec.elem = Int_val(elem);
    spec.tile_m = Int_val(Field(tile, 0));
    spec.tile_n = Int_val(Field(tile, 1));
    spec.tile_k = Int_val(Field(tile, 2));
    rc = tesserae_runtime_run(&spec, mi, ni, ki, fa, fb, fc);   /* no OCaml allocation since String_val above */
    free(fa); free(fb);
    if (rc != 0) { free(fc); caml_failwith(tesserae_last_error()); }
    out = caml_alloc_float_array((mlsize_t)(mi * ni));
    for (i = 0; i < (mlsize_t)(mi * ni); i++) Store_double_flat_field(out, i, (double)fc[i]);
    free(fc);
    CAMLreturn(out);
}

CAMLprim value caml_runtime_run_bytecode(value* argv, int argc) {
    (void)argc;
    return caml_runtime_run(argv[0], argv[1], argv[2], argv[3], argv[4], argv[5], argv[6], argv[7]);
}
