/* Minimal stand-in for the OCaml runtime's <caml/mlvalues.h>: just enough declarations for
 * bindings/tesserae_b200_stubs.c to parse and type-check where no OCaml toolchain exists.  It defines the
 * types and the macro/function names with the real ones' signatures; it is not a runtime and nothing built
 * with it can run.  Used only by tests/test_bindings_syntax.py. */
#ifndef CAML_STANDIN_MLVALUES_H
#define CAML_STANDIN_MLVALUES_H
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
typedef intptr_t intnat;
typedef uintptr_t uintnat;
typedef intnat value;
typedef uintnat mlsize_t;
#define CAMLprim
#define Val_unit ((value)1)
#define Val_emptylist ((value)1)
#define Val_long(x) ((value)(((uintnat)(x) << 1) + 1))
#define Long_val(x) ((x) >> 1)
#define Val_int(x) Val_long(x)
#define Int_val(x) ((int)Long_val(x))
#define Val_bool(x) Val_int((x) != 0)
#define Bool_val(x) Int_val(x)
#define Field(x, i) (((value*)(x))[i])
#define Wosize_val(v) ((mlsize_t)(((uintnat*)(v))[-1] >> 10))
#define String_val(v) ((const char*)(v))
#define Bytes_val(v) ((unsigned char*)(v))
#define Double_wosize ((mlsize_t)(sizeof(double) / sizeof(value)))
double caml_Double_val(value v);
#define Double_val(v) caml_Double_val(v)
#define Double_flat_field(v, i) (((double*)(v))[i])
#define Store_double_flat_field(v, i, d) (((double*)(v))[i] = (d))
#define Nativeint_val(v) (*((intnat*)((value*)(v) + 1)))
#endif
