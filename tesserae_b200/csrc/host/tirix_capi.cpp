// C ABI over the Tirix IR (csrc/tirix): lower a spec to the IR, print / parse its text form, verify, count
// operations, emit.  Counterparts: Desc_to_tirix.lower (lib/tirix/desc_to_tirix.ml:466-508),
// Tirix_verify.verify (lib/tirix/tirix_verify.ml:9-183), Tirix_emit.emit (lib/tirix/tirix_emit.ml:481-501).
#include "../../../include/tesserae_b200.h"
#include "../rt/errors.hpp"
#include "../tirix/tirix.hpp"

#include <cstdlib>
#include <cstring>

using tesserae::fail;
namespace tx = tesserae::tirix;

struct tesserae_tirix { tx::Program program; };

namespace {
char* dup(const std::string& s) {
    char* r = static_cast<char*>(malloc(s.size() + 1));
    if (r) memcpy(r, s.c_str(), s.size() + 1);
    return r;
}
}  // namespace

extern "C" {

int tesserae_tirix_lower(const tesserae_kernel_spec* ks, tesserae_tirix** out) {
    if (!ks || !out) return fail("tirix_lower: null argument");
    *out = nullptr;
    tesserae::KernelConfig cfg;
    std::string msg;
    int rc;
    try { rc = tesserae::derive_config(*ks, &cfg, &msg); }
    catch (const tesserae::spec::SpecError& e) { return fail(std::string("InvalidPipeline: ") + e.what()); }
    if (rc != 0) { fail(msg); return rc; }
    auto* t = new tesserae_tirix();
    try { t->program = tx::lower(cfg, *ks); }
    catch (const std::exception& e) { delete t; return fail(std::string("tirix_lower: ") + e.what()); }
    t->program.origin.name = nullptr;       // the program owns its strings; these pointed into the caller's spec
    t->program.origin.tuning = nullptr;
    *out = t;
    return 0;
}

int tesserae_tirix_parse(const char* text, tesserae_tirix** out) {
    if (!text || !out) return fail("tirix_parse: null argument");
    *out = nullptr;
    auto* t = new tesserae_tirix();
    std::string err;
    if (!tx::parse(text, &t->program, &err)) { delete t; return fail("tirix_parse: " + err); }
    *out = t;
    return 0;
}

void tesserae_tirix_free(tesserae_tirix* t) { delete t; }

char* tesserae_tirix_print(const tesserae_tirix* t) { return t ? dup(tx::print(t->program)) : nullptr; }

int tesserae_tirix_verify(const tesserae_tirix* t, char** errors) {
    if (errors) *errors = nullptr;
    if (!t) { fail("tirix_verify: null program"); return -1; }
    const std::vector<std::string> errs = tx::verify(t->program);
    if (!errs.empty() && errors) {
        std::string all;
        for (size_t i = 0; i < errs.size(); ++i) all += (i ? "\n" : "") + errs[i];
        *errors = dup(all);
    }
    return int(errs.size());
}

int tesserae_tirix_count_ops(const tesserae_tirix* t, const char* op_name) {
    if (!t || !op_name) return -1;
    const int kind = tx::op_kind_from_name(op_name);
    if (kind >= 0) return tx::count_ops(t->program, tx::OpKind(kind));
    fail(std::string("tirix_count_ops: unknown operation '") + op_name + "'");
    return -1;
}

int tesserae_tirix_emit(const tesserae_tirix* t, tesserae_backend_output* out) {
    if (!t || !out) return fail("tirix_emit: null argument");
    memset(out, 0, sizeof *out);
    tesserae::BackendOutput o;
    std::string msg;
    int rc;
    try { rc = tx::emit(t->program, &o, &msg); }
    catch (const std::exception& e) { return fail(std::string("tirix_emit: ") + e.what()); }
    if (rc != 0) { fail(msg); return rc; }
    out->filename = dup(o.filename); out->includes = dup(o.includes); out->helpers = dup(o.helpers);
    out->shared_storage = dup(o.shared_storage); out->producer_body = dup(o.producer_body);
    out->consumer_body = dup(o.consumer_body); out->epilogue_body = dup(o.epilogue_body);
    out->kernel_func = dup(o.kernel_func); out->host_launcher = dup(o.host_launcher); out->full_source = dup(o.full_source);
    return 0;
}

}  // extern "C"
