/* Stand-in for <caml/fail.h> (see mlvalues.h here). */
#ifndef CAML_STANDIN_FAIL_H
#define CAML_STANDIN_FAIL_H
#include "mlvalues.h"
void caml_failwith(const char* msg) __attribute__((noreturn));
#endif
