"""bindings/tesserae_b200_stubs.c (the OCaml-runtime glue a maintainer adds as foreign_stubs) must parse and
type-check against include/tesserae_b200.h.  No OCaml toolchain exists here, so <caml/...> is a minimal stand-in
(tests/helpers/caml_standin); the check proves that every tesserae_* call in the glue has the right arity and
argument types, and that the glue defines every caml_* symbol the reference's externals name.  It is not linked
against an OCaml runtime."""
import re
import subprocess
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
STUBS = ROOT / "bindings" / "tesserae_b200_stubs.c"

# The externals of lib/runtime/nvrtc.ml:15-31, lib/runtime/gpu_buffer.ml:9-13 and lib/kernel/kernel_launch.ml:12-30.
REFERENCE_EXTERNALS = [
    "caml_nvrtc_create", "caml_nvrtc_destroy", "caml_nvrtc_is_valid", "caml_nvrtc_compile", "caml_nvrtc_get_ptx",
    "caml_nvrtc_get_log", "caml_gpu_alloc", "caml_gpu_free", "caml_gpu_copy_to_device", "caml_gpu_copy_to_host",
    "caml_gpu_ptr", "caml_cuinit", "caml_module_load_ptx", "caml_module_unload", "caml_get_function",
    "caml_launch_kernel", "caml_launch_kernel_bytecode", "caml_device_synchronize", "caml_device_info"]


def test_glue_parses_and_type_checks():
    cmd = ["gcc", "-std=c11", "-fsyntax-only", "-Wall", "-Wextra", "-Werror",
           "-I", str(ROOT / "tests" / "helpers" / "caml_standin"), "-I", str(ROOT / "include"), str(STUBS)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_glue_defines_every_external_the_reference_names():
    text = STUBS.read_text()
    defined = set(re.findall(r"CAMLprim value (\w+)\(", text))
    assert set(REFERENCE_EXTERNALS) <= defined, sorted(set(REFERENCE_EXTERNALS) - defined)
    # and every library function it calls is declared in the header
    header = (ROOT / "include" / "tesserae_b200.h").read_text()
    for fn in set(re.findall(r"\b(tesserae_\w+)\(", text)):
        assert re.search(r"\b" + fn + r"\(", header), fn
