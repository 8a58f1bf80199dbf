/* Stand-in for <caml/alloc.h> (see mlvalues.h here). */
#ifndef CAML_STANDIN_ALLOC_H
#define CAML_STANDIN_ALLOC_H
#include "mlvalues.h"
value caml_alloc(mlsize_t wosize, int tag);
value caml_copy_string(const char* s);
value caml_copy_nativeint(intnat i);
value caml_alloc_float_array(mlsize_t len);
#endif
