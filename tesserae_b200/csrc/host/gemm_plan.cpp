// Host side of the GEMM path above the C ABI: spec -> descriptor -> source -> cubin ->
// module -> launch.  C++ mirror of the reference's OCaml modules
//   Lower.lower            lib/kernel/lower.ml:61-97
//   Compile.to_source/ptx  lib/runtime/compile.ml:36-75
//   Runtime.run            lib/runtime/runtime.ml:15-75
// (the OCaml toolchain is not available to build against, and the reference host code is
// compiled code, so the mirror is C++).  A plan owns one compiled kernel and serves any
// problem size; tensor maps are encoded per call from the pointers and sizes given.
#include "../../../include/tesserae_b200.h"
#include "../emit/backend_sm100.hpp"
#include "../rt/driver_api.hpp"
#include "../rt/errors.hpp"

#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <vector>

using tesserae::fail;
using tesserae::KernelConfig;

namespace tesserae {
const DriverApi* driver_with_context(std::string* err);
}

struct tesserae_gemm_plan {
    KernelConfig cfg;
    void* module = nullptr;
    void* function = nullptr;
    uint32_t* d_status = nullptr;
    int device = 0;
    int sm_count = 0;
    int max_clusters = 0;    // co-resident clusters (pairs) or CTAs the persistent grid is sized to
    int cache_hit = 0;
    double compile_ms = 0.0;
    // Device staging for the host-buffer entry point; grown on demand, reused across calls.
    // (slots: 0 A, 1 B, 2 C, 3 bias, 4 scales of A, 5 scales of B)
    void* ws[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t ws_cap[6] = {0, 0, 0, 0, 0, 0};
    // Streams and events of the pipelined host-buffer call (copy in / compute / copy out); created on first use.
    static constexpr int kMaxChunks = 32;
    void* tail_function = nullptr;       // FP8 block-scaled: the kernel that closes a stream-K tail
    // Pinned host copy of the grouped launch's problem table and the event that says the device has taken it.
    void* h_table = nullptr;
    size_t h_table_cap = 0;
    cudaEvent_t ev_table = nullptr;
    cudaStream_t s_in = nullptr, s_cmp = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[kMaxChunks] = {}, ev_cmp[kMaxChunks] = {}, ev_done = nullptr;
};

namespace {

// Device status block of a plan: word 0 is the error word the kernels OR their timeout bits into.
constexpr size_t kStatusBytes = 256;

double now_ms() {
    using namespace std::chrono;
    return duration<double, std::milli>(steady_clock::now().time_since_epoch()).count();
}

char* dup_string(const std::string& s) {
    char* r = static_cast<char*>(malloc(s.size() + 1));
    if (r) memcpy(r, s.c_str(), s.size() + 1);
    return r;
}

int out_bytes(int out_elem) { return out_elem == TESSERAE_F32 ? 4 : 2; }

// The epilogues stage C in 32-row x 128-byte buffers written under Swizzle<3,4,3>, whatever the operand tiles use.
constexpr int kStoreSwizzleB = 3;

// fp32 -> bf16 / f16 bits, round to nearest even (host side of Runtime.run).
uint16_t f32_to_bf16(float f) {
    uint32_t u; memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return uint16_t((u >> 16) | 0x40);
    u += 0x7FFFu + ((u >> 16) & 1u);
    return uint16_t(u >> 16);
}
uint16_t f32_to_f16(float f) {
    uint32_t x; memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    int32_t e = int32_t((x >> 23) & 0xFF) - 127 + 15;
    uint32_t m = x & 0x7FFFFFu;
    if (((x >> 23) & 0xFF) == 0xFF) return uint16_t(sign | 0x7C00u | (m ? 0x200u : 0));
    if (e >= 31) return uint16_t(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10) return uint16_t(sign);
        m |= 0x800000u;
        const int shift = 14 - e;
        uint32_t r = m >> shift;
        const uint32_t rem = m & ((1u << shift) - 1), half = 1u << (shift - 1);
        if (rem > half || (rem == half && (r & 1))) ++r;
        return uint16_t(sign | r);
    }
    uint32_t r = (uint32_t(e) << 10) | (m >> 13);
    const uint32_t rem = m & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (r & 1))) ++r;
    return uint16_t(sign | r);
}

}  // namespace

extern "C" {

// ------------------------------------------------------------------ lower / emit / compile
int tesserae_lower(const tesserae_kernel_spec* ks, tesserae_kernel_desc* out) {
    if (!ks || !out) { fail("lower: null argument"); return TESSERAE_LOWER_MISSING_ARG; }
    namespace sp = tesserae::spec;
    sp::KernelDesc d;
    std::string msg;
    std::string name = (ks->name && *ks->name) ? ks->name : "tesserae_gemm";
    int rc;
    try {
        rc = sp::lower(name, ks->arch, ks->elem, ks->tile_m, ks->tile_n, ks->tile_k, &d, &msg);
    } catch (const sp::SpecError& e) {
        fail(std::string("InvalidPipeline: ") + e.what());
        return TESSERAE_LOWER_INVALID_PIPELINE;
    }
    if (rc != sp::LowerOk) { fail(msg); return rc; }
    memset(out, 0, sizeof *out);
    out->family = d.family;
    snprintf(out->name, sizeof out->name, "%s", d.name.c_str());
    out->bm = d.bm; out->bn = d.bn; out->bk = d.bk; out->elem = d.elem;
    out->swizzle_b = d.swizzle.b; out->swizzle_m = d.swizzle.m; out->swizzle_s = d.swizzle.s;
    out->cluster_x = d.cluster.x; out->cluster_y = d.cluster.y; out->cluster_z = d.cluster.z;
    out->num_warps = d.cluster.num_warps;
    for (int w = 0; w < 8; ++w) out->warp_roles[w] = sp::warp_role_of(d.cluster, w);
    out->pipeline_depth = d.pipeline.depth;
    out->tile_bytes = d.pipeline.tile_bytes;
    out->smem_bytes = d.pipeline.smem_bytes;
    out->strategy = d.strategy;
    out->copy_bulk_bytes = d.copy_bulk_bytes; out->copy_vec = d.copy_vec;
    out->atom_m = d.atom.m; out->atom_n = d.atom.n; out->atom_k = d.atom.k; out->atom_threads = d.atom.threads;
    out->tmem_cta_group = d.tmem.cta_group; out->tmem_rows = d.tmem.num_rows; out->tmem_cols = d.tmem.num_cols;
    out->tmem_double_buf = d.double_buf ? 1 : 0;
    for (int i = 0; i < 2; ++i) {
        out->pred_a_bounds[i] = d.pred_a_bounds[i];
        out->pred_b_bounds[i] = d.pred_b_bounds[i];
        out->pred_c_bounds[i] = d.pred_c_bounds[i];
    }
    out->sm_count = d.sm_count;
    out->m = d.m; out->n = d.n; out->k = d.k;
    return TESSERAE_LOWER_OK;
}

static tesserae::spec::KernelDesc desc_from_c(const tesserae_kernel_desc* c) {
    namespace sp = tesserae::spec;
    sp::KernelDesc d;
    d.family = c->family; d.name = c->name; d.bm = c->bm; d.bn = c->bn; d.bk = c->bk; d.elem = c->elem;
    d.swizzle = sp::Swizzle{c->swizzle_b, c->swizzle_m, c->swizzle_s};
    d.cluster = sp::Cluster{c->cluster_x, c->cluster_y, c->cluster_z, c->num_warps, {}};
    d.pipeline = sp::Pipeline{c->pipeline_depth, c->tile_bytes, c->smem_bytes};
    d.strategy = c->strategy;
    d.atom = sp::MmaAtom{c->atom_m, c->atom_n, c->atom_k, c->atom_threads, ""};
    d.tmem = sp::Tmem{c->tmem_cta_group, c->tmem_cols, c->tmem_rows};
    d.sm_count = c->sm_count;
    return d;
}

int tesserae_kernel_desc_validate(const tesserae_kernel_desc* d) {
    if (!d) return fail("validate: null descriptor");
    const std::string msg = tesserae::spec::validate(desc_from_c(d));
    if (!msg.empty()) return fail(msg);
    return 0;
}

double tesserae_kernel_desc_arithmetic_intensity(const tesserae_kernel_desc* d) {
    if (!d) return 0.0;
    return tesserae::spec::arithmetic_intensity(desc_from_c(d));
}

int tesserae_kernel_desc_grid(const tesserae_kernel_desc* d, int64_t m, int64_t n, int* gx, int* gy, int* threads) {
    if (!d || d->bm <= 0 || d->bn <= 0) return fail("grid: bad descriptor");
    if (gx) *gx = int((m + d->bm - 1) / d->bm);
    if (gy) *gy = int((n + d->bn - 1) / d->bn);
    if (threads) *threads = d->num_warps * 32;
    return 0;
}

int tesserae_backend_emit(const tesserae_kernel_spec* ks, tesserae_backend_output* out) {
    if (!ks || !out) return fail("emit: null argument");
    memset(out, 0, sizeof *out);
    KernelConfig cfg;
    std::string msg;
    int rc;
    try { rc = tesserae::derive_config(*ks, &cfg, &msg); }
    catch (const tesserae::spec::SpecError& e) { return fail(std::string("InvalidPipeline: ") + e.what()); }
    if (rc != 0) { fail(msg); return rc; }
    tesserae::BackendOutput o = tesserae::emit(cfg);
    out->filename = dup_string(o.filename);
    out->includes = dup_string(o.includes);
    out->helpers = dup_string(o.helpers);
    out->shared_storage = dup_string(o.shared_storage);
    out->producer_body = dup_string(o.producer_body);
    out->consumer_body = dup_string(o.consumer_body);
    out->epilogue_body = dup_string(o.epilogue_body);
    out->kernel_func = dup_string(o.kernel_func);
    out->host_launcher = dup_string(o.host_launcher);
    out->full_source = dup_string(o.full_source);
    return 0;
}

void tesserae_backend_output_free(tesserae_backend_output* out) {
    if (!out) return;
    char** f[] = {&out->filename, &out->includes, &out->helpers, &out->shared_storage, &out->producer_body,
                  &out->consumer_body, &out->epilogue_body, &out->kernel_func, &out->host_launcher, &out->full_source};
    for (char** p : f) { free(*p); *p = nullptr; }
}

static int compile_impl(const tesserae_kernel_spec* ks, tesserae_compile_result* out, bool want_cubin, KernelConfig* cfg_out) {
    if (!ks || !out) return fail("compile: null argument");
    memset(out, 0, sizeof *out);
    const double t0 = now_ms();
    KernelConfig cfg;
    std::string msg;
    int rc;
    try { rc = tesserae::derive_config(*ks, &cfg, &msg); }
    catch (const tesserae::spec::SpecError& e) { return fail(std::string("InvalidPipeline: ") + e.what()); }
    if (rc != 0) { fail("Lower_error: " + msg); return rc; }
    tesserae::BackendOutput o = tesserae::emit(cfg);
    out->kernel_name = dup_string(cfg.name);
    out->source = dup_string(o.full_source);
    if (want_cubin) {
        std::vector<std::string> opts = tesserae::nvrtc_options();
        std::vector<const char*> copts;
        for (auto& s : opts) copts.push_back(s.c_str());
        rc = tesserae_compile_cached(o.full_source.c_str(), o.filename.c_str(), copts.data(), (int)copts.size(),
                                     &out->cubin, &out->cubin_size, &out->cache_hit);
        if (rc != 0) {
            const std::string e = std::string("Nvrtc_error: ") + tesserae_last_error();
            tesserae_compile_result_free(out);
            return fail(e);
        }
    }
    out->duration_ms = now_ms() - t0;
    if (cfg_out) *cfg_out = cfg;
    return 0;
}

int tesserae_compile_to_source(const tesserae_kernel_spec* ks, tesserae_compile_result* out) {
    return compile_impl(ks, out, false, nullptr);
}
int tesserae_compile_to_cubin(const tesserae_kernel_spec* ks, tesserae_compile_result* out) {
    return compile_impl(ks, out, true, nullptr);
}
void tesserae_compile_result_free(tesserae_compile_result* r) {
    if (!r) return;
    free(r->kernel_name); r->kernel_name = nullptr;
    free(r->source); r->source = nullptr;
    free(r->cubin); r->cubin = nullptr;
    r->cubin_size = 0;
}

// ------------------------------------------------------------------ plans
int tesserae_gemm_plan_create(const tesserae_kernel_spec* ks, tesserae_gemm_plan** plan_out) {
    if (!ks || !plan_out) return fail("plan_create: null argument");
    *plan_out = nullptr;
    std::string err;
    const tesserae::DriverApi* api = tesserae::driver_with_context(&err);
    if (!api) return fail("plan_create: " + err);

    tesserae_compile_result cr;
    KernelConfig cfg;
    int rc = compile_impl(ks, &cr, true, &cfg);
    if (rc != 0) return rc;

    auto* p = new tesserae_gemm_plan();
    p->cfg = cfg;
    p->cache_hit = cr.cache_hit;
    p->compile_ms = cr.duration_ms;
    rc = tesserae_module_load(cr.cubin, &p->module);
    if (rc == 0) rc = tesserae_get_function(p->module, cfg.name.c_str(), &p->function);
    if (rc == 0 && cfg.scale_mode == TESSERAE_SCALE_FP8_BLOCK)
        rc = tesserae_get_function(p->module, (cfg.name + "_tail").c_str(), &p->tail_function);
    tesserae_compile_result_free(&cr);
    if (rc != 0) { tesserae_gemm_plan_destroy(p); return rc; }

    CUresult crc = api->cuFuncSetAttribute(static_cast<CUfunction>(p->function),
                                           CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, cfg.smem_bytes);
    if (crc != CUDA_SUCCESS) {
        const std::string e = tesserae::driver_error(api, "cuFuncSetAttribute(max dynamic smem)", crc);
        tesserae_gemm_plan_destroy(p);
        return fail(e);
    }
    if (cfg.scale_mode == TESSERAE_SCALE_FP8_BLOCK) {
        // The FP8 block-scaled kernel moves registers between its warpgroups (setmaxnreg): the promotion warps'
        // increase blocks until the CTA's pool holds enough, and the pool is what the CTA was launched with.  Refuse a
        // binary whose launch allocation is smaller than what the two budgets add up to, rather than let it wait.
        int regs = 0;
        crc = api->cuFuncGetAttribute(&regs, CU_FUNC_ATTRIBUTE_NUM_REGS, static_cast<CUfunction>(p->function));
        const int issue = cfg.promo_warps == 8 ? 40 : 32, promo = cfg.promo_warps == 8 ? 232 : 112;   // kRegsIssue / kRegsPromo
        const long long need = 128ll * issue + 32ll * cfg.promo_warps * promo;
        if (crc != CUDA_SUCCESS || (long long)regs * cfg.threads < need) {
            const std::string e = "gemm_plan_create: the FP8 kernel was built with " + std::to_string(regs) + " registers x " +
                                  std::to_string(cfg.threads) + " threads, fewer than the " + std::to_string(need) +
                                  " its register reallocation needs";
            tesserae_gemm_plan_destroy(p);
            return fail(e);
        }
    }
    cudaGetDevice(&p->device);
    if (tesserae_device_sm_count(&p->sm_count) != 0) { tesserae_gemm_plan_destroy(p); return -1; }
    p->max_clusters = p->sm_count / cfg.cta_group;
    if (cfg.cta_group == 2) {
        // How many CTA pairs can be resident at once; the persistent grid is sized to that.
        CUlaunchConfig lc;
        memset(&lc, 0, sizeof lc);
        lc.gridDimX = p->sm_count; lc.gridDimY = 1; lc.gridDimZ = 1;
        lc.blockDimX = cfg.threads; lc.blockDimY = 1; lc.blockDimZ = 1;
        lc.sharedMemBytes = cfg.smem_bytes;
        CUlaunchAttribute at;
        at.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        at.value.clusterDim.x = 2; at.value.clusterDim.y = 1; at.value.clusterDim.z = 1;
        lc.attrs = &at; lc.numAttrs = 1;
        int n = 0;
        if (api->cuOccupancyMaxActiveClusters(&n, static_cast<CUfunction>(p->function), &lc) == CUDA_SUCCESS && n > 0)
            p->max_clusters = n;
    }
    void* st = nullptr;
    if (tesserae_gpu_alloc(kStatusBytes, &st) != 0) { tesserae_gemm_plan_destroy(p); return -1; }
    p->d_status = static_cast<uint32_t*>(st);
    *plan_out = p;
    return 0;
}

void tesserae_gemm_plan_destroy(tesserae_gemm_plan* p) {
    if (!p) return;
    if (p->d_status) tesserae_gpu_free(p->d_status);
    for (void* w : p->ws) tesserae_gpu_free(w);
    for (cudaEvent_t e : p->ev_in) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : p->ev_cmp) if (e) cudaEventDestroy(e);
    if (p->ev_done) cudaEventDestroy(p->ev_done);
    if (p->ev_table) cudaEventDestroy(p->ev_table);
    if (p->h_table) cudaFreeHost(p->h_table);
    if (p->s_in) cudaStreamDestroy(p->s_in);
    if (p->s_cmp) cudaStreamDestroy(p->s_cmp);
    if (p->s_out) cudaStreamDestroy(p->s_out);
    if (p->module) tesserae_module_unload(p->module);
    delete p;
}

int tesserae_gemm_plan_info(const tesserae_gemm_plan* p, int* cta_group, int* block_n, int* stages,
                            int* smem_bytes, int* cache_hit, double* compile_ms) {
    if (!p) return fail("plan_info: null plan");
    if (cta_group) *cta_group = p->cfg.cta_group;
    if (block_n) *block_n = p->cfg.block_n;
    if (stages) *stages = p->cfg.stages;
    if (smem_bytes) *smem_bytes = p->cfg.smem_bytes;
    if (cache_hit) *cache_hit = p->cache_hit;
    if (compile_ms) *compile_ms = p->compile_ms;
    return 0;
}

// A plan's module, status word and staging live on the device that was current when it was created; a launch
// with another device current would end in an opaque driver error (or tensor maps over the wrong memory).
static int check_plan_device(const tesserae_gemm_plan* p, const char* what) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) return fail(std::string(what) + ": cannot read the current device");
    if (cur != p->device)
        return fail(std::string(what) + ": the plan was created on device " + std::to_string(p->device) +
                    " but device " + std::to_string(cur) + " is current");
    return 0;
}

// Height of the raster groups in M-tiles.  All tiles of a group read the group's panel of A (group_m M-tiles x K)
// again for every N-tile while B streams through once per group, so the panel should stay resident in L2: it is sized
// to about a quarter of the 126 MB L2 (the rest holds the B tiles in flight and the output on its way out).  Larger
// groups re-read B fewer times: with 8-tile groups the NVFP4 case (1 MB of A per M-tile) fetched B eight times.
// When K is so long that not even 8 M-tiles of A fit that budget, residency is out of reach and what is left is the
// reuse between the tiles in flight together, which march through K in step: about 74 clusters = 8 M-tiles x 9 N-tiles
// minimises the rows of A and B they touch, so the group height never goes below 8.
static int pick_group_m(const KernelConfig& cfg, int64_t m, int64_t k) {
    const int64_t tile_m = 128 * cfg.cta_group;
    const int64_t num_m = (m + tile_m - 1) / tile_m;
    if (cfg.group_m > 0) return int(cfg.group_m < num_m ? cfg.group_m : (num_m > 0 ? num_m : 1));
    const int64_t panel = tile_m * (k * tesserae::spec::elem_bits(cfg.elem) / 8);     // bytes of A per M-tile
    int64_t g = (int64_t(32) << 20) / (panel > 0 ? panel : 1);
    if (g < 8) g = 8;
    if (cfg.block_n > 256) g *= 2;       // a wave of 512-column tiles spans half as many tile columns: keep its footprint near square
    if (g > 64) g = 64;
    if (g > num_m) g = num_m;
    return int(g < 1 ? 1 : g);
}

// Stream-K tail of the FP8 block-scaled kernel: which tiles are computed whole and into how many ranges of K blocks
// each of the rest is split.  Only plans whose spec asks for it (TAIL_SPLITS=n, n >= 2, in the tuning string) carry
// the unit logic in their kernel, because what it wins is small.  Measured on a B200, 8192 x 1792 x 4096 (74 clusters,
// 2 tiles left over after 3 whole waves): 72.7 us per call with the tail against 72.5 us without; per kernel (profiler,
// cold caches): 65.1 us + the closing kernel against 70.0 us.  The left-over wave of two tiles costs 11.5 us, not a
// whole wave's 19 us (two tiles alone have the memory system to themselves), the tail's units cost 6.6 us (pipeline
// fill, one pass through the staging buffers, the adds) and the second launch takes most of the rest.  The same
// problem without left-over tiles runs 2 % slower through a kernel compiled with the unit logic.
// With it, a tail is used whenever tiles are left over after the whole waves and fill at most half the clusters.
struct TailPlan { int64_t full_tiles = 0, tail_tiles = 0; int splits = 1; size_t bytes = 0; };
static TailPlan plan_tail(const tesserae_gemm_plan* p, int64_t m, int64_t n, int64_t k) {
    const KernelConfig& cfg = p->cfg;
    TailPlan t;
    const int64_t tile_m = 128 * cfg.cta_group;
    const int64_t tiles = ((m + tile_m - 1) / tile_m) * ((n + cfg.block_n - 1) / cfg.block_n);
    t.full_tiles = tiles;
    if (cfg.scale_mode != TESSERAE_SCALE_FP8_BLOCK || cfg.tail_splits < 2) return t;
    const int64_t clusters = p->max_clusters, nkb = k / 128;
    const int64_t rest = tiles % clusters;
    if (rest == 0 || nkb < 4 || rest * 2 > clusters) return t;
    int64_t splits = clusters / rest;
    if (splits > nkb / 2) splits = nkb / 2;              // at least two K blocks per unit
    if (splits > cfg.tail_splits) splits = cfg.tail_splits;
    if (splits < 2) return t;
    t.full_tiles = tiles - rest;
    t.tail_tiles = rest;
    t.splits = int(splits);
    t.bytes = size_t(rest) * size_t(tile_m) * size_t(cfg.block_n) * 4;
    return t;
}

// lda / ldb / ldc: row pitch in elements of A (M x K), B (N x K) and C (M x N); 0 = dense.
static int gemm_launch(tesserae_gemm_plan* p, const void* a, int64_t lda, const void* b, int64_t ldb, void* c, int64_t ldc,
                       const tesserae_gemm_scales* scales, const void* bias,
                       float alpha, int64_t m, int64_t n, int64_t k, void* stream,
                       void* tail_ws = nullptr, size_t tail_ws_bytes = 0) {
    if (!p || !a || !b || !c) return fail("gemm_run: null argument");
    if (int drc = check_plan_device(p, "gemm_run")) return drc;
    if (m <= 0 || n <= 0 || k <= 0) return fail("gemm_run: M, N and K must be positive");
    if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return fail("gemm_run: dimension exceeds 2^31-1");
    const KernelConfig& cfg = p->cfg;
    if (cfg.scatter) return fail("gemm_run: this plan stores row-scattered output; use tesserae_gemm_ksplit_scatter");
    if (cfg.grouped) return fail("gemm_run: this plan walks a problem table; use tesserae_gemm_run_grouped");
    if (cfg.has_bias && !bias) return fail("gemm_run: this kernel was built with a bias but none was given");
    if (cfg.has_bias && (reinterpret_cast<uintptr_t>(bias) & 15u)) return fail("gemm_run: bias must be 16-byte aligned");
    const bool scaled = cfg.scale_mode != TESSERAE_SCALE_NONE;
    if (scaled && (!scales || !scales->scale_a || !scales->scale_b))
        return fail("gemm_run: this kernel needs scale factors (use tesserae_gemm_run_scaled)");
    if (!scaled && scales) return fail("gemm_run: this kernel takes no scale factors");
    if (cfg.scale_mode == TESSERAE_SCALE_FP8_BLOCK && k % 128 != 0)
        return fail("gemm_run: K must be a multiple of the 128-wide scale block");
    if (cfg.scale_mode == TESSERAE_SCALE_NVFP4 && k % 256 != 0)
        return fail("gemm_run: NVFP4 needs K to be a multiple of 256 (one 128-byte stage)");
    const int ebits = tesserae::spec::elem_bits(cfg.elem);
    const int ob = out_bytes(cfg.out_elem);
    if ((k * ebits / 8) % 16 != 0 || (k * ebits) % 8 != 0) return fail("gemm_run: K * element size must be a multiple of 16 bytes");
    if ((n * ob) % 16 != 0) return fail("gemm_run: N * output element size must be a multiple of 16 bytes");

    alignas(64) unsigned char tm_a[128], tm_b[128], tm_c[128];
    if (lda == 0) lda = k;
    if (ldb == 0) ldb = k;
    if (ldc == 0) ldc = n;
    if (lda < k || ldb < k || ldc < n) return fail("gemm_run: a leading dimension is smaller than the row it holds");
    if ((lda * ebits / 8) % 16 != 0 || (ldb * ebits / 8) % 16 != 0 || (ldc * ob) % 16 != 0)
        return fail("gemm_run: row pitches must be multiples of 16 bytes");
    const uint64_t row_bytes_a = uint64_t(lda) * ebits / 8, row_bytes_b = uint64_t(ldb) * ebits / 8;
    // For the 4-bit element the map addresses bytes: two values per byte along K.
    const uint64_t inner_ab = (cfg.elem == TESSERAE_F4E2M1) ? uint64_t(k) / 2 : uint64_t(k);
    const uint32_t box_k = (cfg.elem == TESSERAE_F4E2M1) ? 128u : uint32_t(cfg.block_k);
    // Operand tiles land in shared memory under the swizzle the descriptor was lowered with (Swizzle.smem_selector
    // of the spec's tile); the output staging rows are always 128 bytes wide, hence Swizzle<3,4,3> for C.
    const int op_swizzle = cfg.desc.swizzle.b;
    int rc = tesserae_tensor_map_2d(tm_a, cfg.elem, a, inner_ab, uint64_t(m), row_bytes_a, box_k, 128, op_swizzle);
    if (rc == 0) rc = tesserae_tensor_map_2d(tm_b, cfg.elem, b, inner_ab, uint64_t(n), row_bytes_b, box_k,
                                             uint32_t(cfg.b_box_rows), op_swizzle);
    if (rc == 0) rc = tesserae_tensor_map_2d(tm_c, cfg.out_elem, c, uint64_t(n), uint64_t(m), uint64_t(ldc) * ob,
                                             uint32_t(128 / ob), 32, kStoreSwizzleB);
    if (rc != 0) return rc;

    const int64_t tile_m = 128 * cfg.cta_group;
    const int64_t tiles = ((m + tile_m - 1) / tile_m) * ((n + cfg.block_n - 1) / cfg.block_n);
    // Static order: one cluster per SM (pair), each walks every n-th tile.  Launch control: one cluster per tile; those
    // that get to run take over the tiles of those that have not started yet.
    if (cfg.clc && tiles * cfg.cta_group > INT32_MAX) return fail("gemm_run: too many tiles for a launch-control grid");
    const int clusters = cfg.clc ? int(tiles) : int(tiles < p->max_clusters ? tiles : p->max_clusters);
    const int grid[3] = {clusters * cfg.cta_group, 1, 1};
    const int block[3] = {cfg.threads, 1, 1};
    const int cluster[3] = {cfg.cta_group, 1, 1};
    const int mi = int(m), ni = int(n), ki = int(k), gmi = pick_group_m(cfg, m, k);
    if (cfg.scale_mode == TESSERAE_SCALE_NVFP4) {
        // Scale tables: [row blocks * K/64] chunks of 512 bytes, addressed as rows of 128 32-bit words;
        // one stage of one row block is 4 consecutive rows.
        alignas(64) unsigned char tm_sfa[128], tm_sfb[128];
        const uint64_t kg = uint64_t(k) / 64;
        rc = tesserae_tensor_map_2d(tm_sfa, TESSERAE_S32, scales->scale_a, 128, uint64_t((m + 127) / 128) * kg, 512, 128, 4, 0);
        if (rc == 0) rc = tesserae_tensor_map_2d(tm_sfb, TESSERAE_S32, scales->scale_b, 128, uint64_t((n + 127) / 128) * kg, 512, 128, 4, 0);
        if (rc != 0) return rc;
        const float alpha_eff = alpha * scales->global_a * scales->global_b;
        const tesserae_launch_arg args[] = {
            {tm_a, 128}, {tm_b, 128}, {tm_c, 128}, {tm_sfa, 128}, {tm_sfb, 128}, {&bias, sizeof(void*)},
            {&alpha_eff, sizeof(float)}, {&mi, sizeof(int)}, {&ni, sizeof(int)}, {&ki, sizeof(int)}, {&gmi, sizeof(int)},
            {&p->d_status, sizeof(void*)}};
        return tesserae_launch_kernel_ex(p->function, grid, block, cluster, cfg.smem_bytes, stream, args, 12);
    }
    if (cfg.scale_mode == TESSERAE_SCALE_FP8_BLOCK) {
        // Stream-K tail: with a workspace, the tiles past the last whole wave are split into ranges of K blocks.
        TailPlan tp = plan_tail(p, m, n, k);
        alignas(64) unsigned char tm_ws[128];
        if (tp.tail_tiles > 0 && tail_ws) {
            if (tail_ws_bytes < tp.bytes) return fail("gemm_run: tail workspace too small, need " + std::to_string(tp.bytes) + " bytes");
            if (reinterpret_cast<uintptr_t>(tail_ws) & 127u) return fail("gemm_run: tail workspace must be 128-byte aligned");
            rc = tesserae_tensor_map_2d(tm_ws, TESSERAE_F32, tail_ws, uint64_t(cfg.block_n), uint64_t(tp.tail_tiles) * tile_m,
                                        uint64_t(cfg.block_n) * 4, 32, 32, kStoreSwizzleB);
            if (rc != 0) return rc;
        } else {
            tp = TailPlan{};
            tp.full_tiles = tiles;
            memcpy(tm_ws, tm_c, 128);                     // never read: every tile is computed whole
        }
        const int64_t units = tp.full_tiles + tp.tail_tiles * tp.splits;
        const int uclusters = int(units < p->max_clusters ? units : p->max_clusters);
        const int ugrid[3] = {uclusters * cfg.cta_group, 1, 1};
        const int full_i = int(tp.full_tiles), splits_i = tp.splits;
        const tesserae_launch_arg args[] = {
            {tm_a, 128}, {tm_b, 128}, {tm_c, 128}, {tm_ws, 128}, {&scales->scale_a, sizeof(void*)}, {&scales->scale_b, sizeof(void*)},
            {&bias, sizeof(void*)}, {&alpha, sizeof(float)}, {&mi, sizeof(int)}, {&ni, sizeof(int)}, {&ki, sizeof(int)},
            {&gmi, sizeof(int)}, {&full_i, sizeof(int)}, {&splits_i, sizeof(int)}, {&p->d_status, sizeof(void*)}};
        rc = tesserae_launch_kernel_ex(p->function, ugrid, block, cluster, cfg.smem_bytes, stream, args, 15);
        if (rc != 0 || tp.tail_tiles == 0) return rc;
        const int tgrid[3] = {int(tp.tail_tiles), 32, 1};
        const int tblock[3] = {256, 1, 1};
        const int one[3] = {1, 1, 1};
        const long long ldc_ll = ldc;
        const tesserae_launch_arg targs[] = {{&tail_ws, sizeof(void*)}, {&c, sizeof(void*)}, {&bias, sizeof(void*)}, {&mi, sizeof(int)},
                                             {&ni, sizeof(int)}, {&ldc_ll, sizeof(long long)}, {&gmi, sizeof(int)}, {&full_i, sizeof(int)}};
        return tesserae_launch_kernel_ex(p->tail_function, tgrid, tblock, one, 0, stream, targs, 8);
    }
    const tesserae_launch_arg args[] = {
        {tm_a, 128}, {tm_b, 128}, {tm_c, 128}, {&bias, sizeof(void*)}, {&alpha, sizeof(float)},
        {&mi, sizeof(int)}, {&ni, sizeof(int)}, {&ki, sizeof(int)}, {&gmi, sizeof(int)}, {&p->d_status, sizeof(void*)}};
    return tesserae_launch_kernel_ex(p->function, grid, block, cluster, cfg.smem_bytes, stream, args, 10);
}

int tesserae_gemm_run_scaled(tesserae_gemm_plan* p, const void* a, const void* b, void* c,
                             const tesserae_gemm_scales* scales, const void* bias,
                             float alpha, int64_t m, int64_t n, int64_t k, void* stream) {
    return gemm_launch(p, a, 0, b, 0, c, 0, scales, bias, alpha, m, n, k, stream);
}

size_t tesserae_gemm_tail_workspace_bytes(const tesserae_gemm_plan* p, int64_t m, int64_t n, int64_t k) {
    if (!p || m <= 0 || n <= 0 || k <= 0) return 0;
    return plan_tail(p, m, n, k).bytes;
}

int tesserae_gemm_run_scaled_ws(tesserae_gemm_plan* p, const void* a, const void* b, void* c,
                                const tesserae_gemm_scales* scales, const void* bias,
                                float alpha, int64_t m, int64_t n, int64_t k,
                                void* workspace, size_t workspace_bytes, void* stream) {
    return gemm_launch(p, a, 0, b, 0, c, 0, scales, bias, alpha, m, n, k, stream, workspace, workspace_bytes);
}

int tesserae_gemm_run(tesserae_gemm_plan* p, const void* a, const void* b, void* c, const void* bias,
                      float alpha, int64_t m, int64_t n, int64_t k, void* stream) {
    return gemm_launch(p, a, 0, b, 0, c, 0, nullptr, bias, alpha, m, n, k, stream);
}

// ------------------------------------------------------------------ grouped
namespace {
// Row of the problem table as the kernel reads it (TsGroupedProblem in gemm_sm100_dense.cuh).
struct alignas(64) GroupedRow {
    unsigned char a[128], b[128], c[128];
    const void* bias;
    int M, N, K;
    int tile_start, num_m, num_n, group_m;
    int pad[7];
};
static_assert(sizeof(GroupedRow) == 448, "the problem table's row is 448 bytes on both sides");
}  // namespace

size_t tesserae_gemm_grouped_workspace_bytes(int n_problems) {
    return n_problems < 1 ? 0 : size_t(n_problems + 1) * sizeof(GroupedRow);
}

int tesserae_gemm_run_grouped(tesserae_gemm_plan* p, const tesserae_gemm_problem* problems, int n_problems, float alpha,
                              void* workspace, size_t workspace_bytes, void* stream) {
    if (!p || !problems || !workspace) return fail("gemm_run_grouped: null argument");
    if (int drc = check_plan_device(p, "gemm_run_grouped")) return drc;
    const KernelConfig& cfg = p->cfg;
    if (!cfg.grouped) return fail("gemm_run_grouped: the plan's spec must have grouped = 1");
    if (n_problems < 1 || n_problems > 65536) return fail("gemm_run_grouped: n_problems must be in 1..65536");
    const size_t need = tesserae_gemm_grouped_workspace_bytes(n_problems);
    if (workspace_bytes < need) return fail("gemm_run_grouped: workspace too small, need " + std::to_string(need) + " bytes");
    if (reinterpret_cast<uintptr_t>(workspace) & 63u) return fail("gemm_run_grouped: workspace must be 64-byte aligned");
    cudaError_t e = cudaSuccess;
    if (p->h_table_cap < need) {
        if (p->h_table) { if (p->ev_table) cudaEventSynchronize(p->ev_table); cudaFreeHost(p->h_table); p->h_table = nullptr; p->h_table_cap = 0; }
        e = cudaHostAlloc(&p->h_table, need, cudaHostAllocDefault);
        if (e != cudaSuccess) return fail(std::string("gemm_run_grouped: ") + cudaGetErrorString(e));
        p->h_table_cap = need;
    }
    if (!p->ev_table) {
        e = cudaEventCreateWithFlags(&p->ev_table, cudaEventDisableTiming);
        if (e != cudaSuccess) return fail(std::string("gemm_run_grouped: ") + cudaGetErrorString(e));
    } else {
        cudaEventSynchronize(p->ev_table);       // the previous call's copy has left the pinned table
    }
    const int ebits = tesserae::spec::elem_bits(cfg.elem);
    const int ob = out_bytes(cfg.out_elem);
    const int op_swizzle = cfg.desc.swizzle.b;
    const int64_t tile_m = 128 * cfg.cta_group;
    GroupedRow* rows = static_cast<GroupedRow*>(p->h_table);
    memset(rows, 0, need);
    int64_t tiles = 0;
    for (int i = 0; i < n_problems; ++i) {
        const tesserae_gemm_problem& q = problems[i];
        const std::string at = "gemm_run_grouped: problem " + std::to_string(i) + ": ";
        if (!q.a || !q.b || !q.c) return fail(at + "null operand");
        if (q.m <= 0 || q.n <= 0 || q.k <= 0 || q.m > INT32_MAX || q.n > INT32_MAX || q.k > INT32_MAX) return fail(at + "bad dimensions");
        if ((q.k * ebits / 8) % 16 != 0) return fail(at + "K * element size must be a multiple of 16 bytes");
        if ((q.n * ob) % 16 != 0) return fail(at + "N * output element size must be a multiple of 16 bytes");
        if (cfg.has_bias && !q.bias) return fail(at + "this kernel was built with a bias but none was given");
        if (cfg.has_bias && (reinterpret_cast<uintptr_t>(q.bias) & 15u)) return fail(at + "bias must be 16-byte aligned");
        GroupedRow& r = rows[i];
        const uint64_t row_bytes = uint64_t(q.k) * ebits / 8;
        int rc = tesserae_tensor_map_2d(r.a, cfg.elem, q.a, uint64_t(q.k), uint64_t(q.m), row_bytes, uint32_t(cfg.block_k), 128, op_swizzle);
        if (rc == 0) rc = tesserae_tensor_map_2d(r.b, cfg.elem, q.b, uint64_t(q.k), uint64_t(q.n), row_bytes, uint32_t(cfg.block_k),
                                                 uint32_t(cfg.b_box_rows), op_swizzle);
        if (rc == 0) rc = tesserae_tensor_map_2d(r.c, cfg.out_elem, q.c, uint64_t(q.n), uint64_t(q.m), uint64_t(q.n) * ob,
                                                 uint32_t(128 / ob), 32, kStoreSwizzleB);
        if (rc != 0) return rc;
        r.bias = q.bias;
        r.M = int(q.m); r.N = int(q.n); r.K = int(q.k);
        r.num_m = int((q.m + tile_m - 1) / tile_m);
        r.num_n = int((q.n + cfg.block_n - 1) / cfg.block_n);
        r.group_m = pick_group_m(cfg, q.m, q.k);
        r.tile_start = int(tiles);
        tiles += int64_t(r.num_m) * r.num_n;
        if (tiles > INT32_MAX) return fail("gemm_run_grouped: too many tiles");
    }
    rows[n_problems].tile_start = int(tiles);            // the sentinel row the tile search stops at
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    e = cudaMemcpyAsync(workspace, rows, need, cudaMemcpyHostToDevice, st);
    if (e == cudaSuccess) e = cudaEventRecord(p->ev_table, st);
    if (e != cudaSuccess) return fail(std::string("gemm_run_grouped: ") + cudaGetErrorString(e));
    // Static order: one cluster per SM (pair), each walks every n-th tile.  Launch control: one cluster per tile; those
    // that get to run take over the tiles of those that have not started yet.
    if (cfg.clc && tiles * cfg.cta_group > INT32_MAX) return fail("gemm_run_grouped: too many tiles for a launch-control grid");
    const int clusters = cfg.clc ? int(tiles) : int(tiles < p->max_clusters ? tiles : p->max_clusters);
    const int grid[3] = {clusters * cfg.cta_group, 1, 1};
    const int block[3] = {cfg.threads, 1, 1};
    const int cluster[3] = {cfg.cta_group, 1, 1};
    const int total = int(tiles);
    const tesserae_launch_arg args[] = {{&workspace, sizeof(void*)}, {&total, sizeof(int)}, {&alpha, sizeof(float)},
                                        {&p->d_status, sizeof(void*)}};
    return tesserae_launch_kernel_ex(p->function, grid, block, cluster, cfg.smem_bytes, stream, args, 4);
}

// ------------------------------------------------------------------ K-split
size_t tesserae_gemm_ksplit_scratch_bytes(int64_t m, int64_t n, int k_splits) {
    if (m <= 0 || n <= 0 || k_splits < 1) return 0;
    return size_t(m) * size_t(n) * sizeof(float) * size_t(k_splits);
}

int tesserae_gemm_ksplit_partials(tesserae_gemm_plan* p, const void* a, const void* b, void* scratch, size_t scratch_bytes,
                                  int64_t m, int64_t n, int64_t k, int k_splits, void* stream) {
    if (!p || !scratch) return fail("gemm_ksplit: null argument");
    const KernelConfig& cfg = p->cfg;
    if (cfg.out_elem != TESSERAE_F32 || cfg.has_bias || cfg.scale_mode != TESSERAE_SCALE_NONE)
        return fail("gemm_ksplit: the plan must be an unscaled kernel with fp32 output and no bias (the partial-product kernel)");
    if (k_splits < 1 || k_splits > 64) return fail("gemm_ksplit: k_splits must be in 1..64");
    const int64_t kblk = cfg.block_k;
    if (k % (int64_t(k_splits) * kblk) != 0)
        return fail("gemm_ksplit: K must be a multiple of k_splits * " + std::to_string(kblk) + " (whole smem stages per slice)");
    if (scratch_bytes < tesserae_gemm_ksplit_scratch_bytes(m, n, k_splits))
        return fail("gemm_ksplit: scratch too small, need " + std::to_string(tesserae_gemm_ksplit_scratch_bytes(m, n, k_splits)) + " bytes");
    const int eb = tesserae::spec::elem_bits(cfg.elem) / 8;
    const int64_t ks = k / k_splits;
    for (int s = 0; s < k_splits; ++s) {
        const char* as = static_cast<const char*>(a) + size_t(s) * ks * eb;
        const char* bs = static_cast<const char*>(b) + size_t(s) * ks * eb;
        float* cs = static_cast<float*>(scratch) + size_t(s) * m * n;
        int rc = gemm_launch(p, as, k, bs, k, cs, n, nullptr, nullptr, 1.0f, m, n, ks, stream);
        if (rc != 0) return rc;
    }
    return 0;
}

int tesserae_gemm_ksplit_scatter(tesserae_gemm_plan* p, const void* a, const void* b, void* const* dst, int n_dst,
                                 int64_t rows_per_owner, int start_owner, int64_t m, int64_t n, int64_t k, void* stream) {
    if (!p || !a || !b || !dst) return fail("ksplit_scatter: null argument");
    if (int drc = check_plan_device(p, "ksplit_scatter")) return drc;
    const KernelConfig& cfg = p->cfg;
    if (!cfg.scatter) return fail("ksplit_scatter: the plan's spec must have scatter = 1 or 2");
    if (n_dst < 1 || n_dst > 8) return fail("ksplit_scatter: n_dst must be in 1..8");
    if (rows_per_owner <= 0 || rows_per_owner % 128 != 0) return fail("ksplit_scatter: rows_per_owner must be a positive multiple of 128");
    if (m <= 0 || n <= 0 || k <= 0 || m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return fail("ksplit_scatter: bad dimensions");
    if (int64_t(n_dst) * rows_per_owner < m) return fail("ksplit_scatter: n_dst * rows_per_owner must cover M");
    if (start_owner < 0 || start_owner >= n_dst) return fail("ksplit_scatter: start_owner must be in [0, n_dst)");
    const int ebits = tesserae::spec::elem_bits(cfg.elem);
    if ((k * ebits / 8) % 16 != 0 || (n * 4) % 16 != 0) return fail("ksplit_scatter: K * element size and N * 4 must be multiples of 16 bytes");
    alignas(64) unsigned char tm_a[128], tm_b[128];
    struct alignas(64) { unsigned char m[8][128]; } tm_c;
    memset(&tm_c, 0, sizeof tm_c);
    const uint64_t row_bytes = uint64_t(k) * ebits / 8;
    const int op_swizzle = cfg.desc.swizzle.b;
    int rc = tesserae_tensor_map_2d(tm_a, cfg.elem, a, uint64_t(k), uint64_t(m), row_bytes, uint32_t(cfg.block_k), 128, op_swizzle);
    if (rc == 0) rc = tesserae_tensor_map_2d(tm_b, cfg.elem, b, uint64_t(k), uint64_t(n), row_bytes, uint32_t(cfg.block_k),
                                             uint32_t(cfg.b_box_rows), op_swizzle);
    for (int g = 0; g < n_dst && rc == 0; ++g) {
        const int64_t rows = (m - g * rows_per_owner) < rows_per_owner ? (m - g * rows_per_owner) : rows_per_owner;
        if (rows <= 0) break;
        if (!dst[g]) return fail("ksplit_scatter: null destination");
        rc = tesserae_tensor_map_2d(tm_c.m[g], TESSERAE_F32, dst[g], uint64_t(n), uint64_t(rows), uint64_t(n) * 4, 32, 32, kStoreSwizzleB);
    }
    if (rc != 0) return rc;
    const int64_t tile_m = 128 * cfg.cta_group;
    const int64_t tiles = ((m + tile_m - 1) / tile_m) * ((n + cfg.block_n - 1) / cfg.block_n);
    const int clusters = int(tiles < p->max_clusters ? tiles : p->max_clusters);
    const int grid[3] = {clusters * cfg.cta_group, 1, 1};
    const int block[3] = {cfg.threads, 1, 1};
    const int cluster[3] = {cfg.cta_group, 1, 1};
    const int mi = int(m), ni = int(n), ki = int(k), rpo = int(rows_per_owner), gmi = pick_group_m(cfg, m, k);
    const int rot = int((int64_t(start_owner) * rows_per_owner) / (128 * cfg.cta_group));   // M-tiles in front of that owner's rows
    const void* no_bias = nullptr;
    const float one = 1.0f;
    const tesserae_launch_arg args[] = {
        {tm_a, 128}, {tm_b, 128}, {&tm_c, sizeof tm_c}, {&rpo, sizeof(int)}, {&rot, sizeof(int)}, {&no_bias, sizeof(void*)},
        {&one, sizeof(float)}, {&mi, sizeof(int)}, {&ni, sizeof(int)}, {&ki, sizeof(int)}, {&gmi, sizeof(int)},
        {&p->d_status, sizeof(void*)}};
    return tesserae_launch_kernel_ex(p->function, grid, block, cluster, cfg.smem_bytes, stream, args, 12);
}

int tesserae_gemm_ksplit_run(tesserae_gemm_plan* p, const void* a, const void* b, void* c_bf16, void* scratch,
                             size_t scratch_bytes, float alpha, int64_t m, int64_t n, int64_t k, int k_splits, void* stream) {
    if (!c_bf16) return fail("gemm_ksplit: null output");
    int rc = tesserae_gemm_ksplit_partials(p, a, b, scratch, scratch_bytes, m, n, k, k_splits, stream);
    if (rc != 0) return rc;
    return tesserae_reduce_cast_bf16(scratch, k_splits, size_t(m) * size_t(n), alpha, c_bf16, size_t(m) * size_t(n), stream);
}

int tesserae_gemm_status(tesserae_gemm_plan* p, uint32_t* status) {
    if (!p) return fail("gemm_status: null plan");
    uint32_t s = 0;
    cudaError_t rc = cudaDeviceSynchronize();
    if (rc == cudaSuccess) rc = cudaMemcpy(&s, p->d_status, sizeof s, cudaMemcpyDeviceToHost);
    if (rc == cudaSuccess && s != 0) rc = cudaMemset(p->d_status, 0, sizeof s);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    if (status) *status = s;
    return 0;
}

static int ensure_ws(tesserae_gemm_plan* p, int i, size_t bytes) {
    if (p->ws_cap[i] >= bytes) return 0;
    tesserae_gpu_free(p->ws[i]);
    p->ws[i] = nullptr; p->ws_cap[i] = 0;
    void* d = nullptr;
    cudaError_t rc = cudaMalloc(&d, bytes);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    p->ws[i] = d; p->ws_cap[i] = bytes;
    return 0;
}

// Bytes of the scale tables a scaled plan reads for `rows` rows of an operand (0 for an unscaled plan).
static size_t scale_table_bytes(const KernelConfig& cfg, bool operand_a, int64_t rows, int64_t k) {
    if (cfg.scale_mode == TESSERAE_SCALE_FP8_BLOCK)
        return size_t(operand_a ? rows : (rows + 127) / 128) * size_t(k / 128) * sizeof(float);
    if (cfg.scale_mode == TESSERAE_SCALE_NVFP4) return tesserae_nvfp4_scale_bytes(rows, k);
    return 0;
}

// Host-buffer call shared by the unscaled and the block-scaled entry points.  `scales` holds HOST pointers (or is
// NULL for an unscaled plan).
static int run_host_impl(tesserae_gemm_plan* p, const void* a, const void* b, void* c, const tesserae_gemm_scales* scales,
                         const void* bias, float alpha, int64_t m, int64_t n, int64_t k, const char* who) {
    if (!p || !a || !b || !c) return fail(std::string(who) + ": null argument");
    if (m <= 0 || n <= 0 || k <= 0) return fail(std::string(who) + ": M, N and K must be positive");
    if (int drc = check_plan_device(p, who)) return drc;
    const KernelConfig& cfg = p->cfg;
    if (cfg.has_bias && !bias) return fail(std::string(who) + ": this kernel was built with a bias but none was given");
    const bool scaled = cfg.scale_mode != TESSERAE_SCALE_NONE;
    if (scaled && (!scales || !scales->scale_a || !scales->scale_b))
        return fail(std::string(who) + ": this kernel needs scale factors (use tesserae_gemm_run_scaled_host)");
    if (!scaled && scales) return fail(std::string(who) + ": this kernel takes no scale factors");
    if (cfg.scale_mode == TESSERAE_SCALE_FP8_BLOCK && k % 128 != 0) return fail(std::string(who) + ": K must be a multiple of the 128-wide scale block");
    if (cfg.scale_mode == TESSERAE_SCALE_NVFP4 && k % 256 != 0) return fail(std::string(who) + ": NVFP4 needs K to be a multiple of 256");
    const int ebits = tesserae::spec::elem_bits(cfg.elem);
    const size_t a_bytes = size_t(m) * k * ebits / 8, b_bytes = size_t(n) * k * ebits / 8;
    const size_t c_bytes = size_t(m) * n * out_bytes(cfg.out_elem);
    const size_t sa_bytes = scale_table_bytes(cfg, true, m, k), sb_bytes = scale_table_bytes(cfg, false, n, k);
    int rc = ensure_ws(p, 0, a_bytes);
    if (rc == 0) rc = ensure_ws(p, 1, b_bytes);
    if (rc == 0) rc = ensure_ws(p, 2, c_bytes);
    if (rc == 0 && cfg.has_bias) rc = ensure_ws(p, 3, size_t(n) * 2);
    if (rc == 0 && scaled) rc = ensure_ws(p, 4, sa_bytes);
    if (rc == 0 && scaled) rc = ensure_ws(p, 5, sb_bytes);
    if (rc != 0) return rc;
    const int ob = out_bytes(cfg.out_elem);
    const size_t row_a = size_t(k) * ebits / 8, row_c = size_t(n) * ob;
    tesserae_gemm_scales dsc;
    if (scaled) { dsc = *scales; dsc.scale_a = p->ws[4]; dsc.scale_b = p->ws[5]; }
    const void* dbias = cfg.has_bias ? p->ws[3] : nullptr;
    cudaError_t e = cudaSuccess;
    // Large calls are PCIe-bound: B (and the scale tables) go up first, then A in row chunks; each chunk's GEMM starts
    // when its rows have landed and its rows of C go back while the next chunk is still arriving (three streams, both
    // copy directions busy at once).  Small calls take the plain order on the default stream.  Either way the copies
    // only run at full speed when the caller's buffers are page-locked.
    const int64_t chunk_rows = ((m / 16 + 255) / 256) * 256;
    const bool pipelined = a_bytes + b_bytes + c_bytes >= (size_t(32) << 20) && chunk_rows >= 256 && m > chunk_rows;
    if (!pipelined) {
        e = cudaMemcpyAsync(p->ws[0], a, a_bytes, cudaMemcpyHostToDevice, nullptr);
        if (e == cudaSuccess) e = cudaMemcpyAsync(p->ws[1], b, b_bytes, cudaMemcpyHostToDevice, nullptr);
        if (e == cudaSuccess && cfg.has_bias) e = cudaMemcpyAsync(p->ws[3], bias, size_t(n) * 2, cudaMemcpyHostToDevice, nullptr);
        if (e == cudaSuccess && scaled) e = cudaMemcpyAsync(p->ws[4], scales->scale_a, sa_bytes, cudaMemcpyHostToDevice, nullptr);
        if (e == cudaSuccess && scaled) e = cudaMemcpyAsync(p->ws[5], scales->scale_b, sb_bytes, cudaMemcpyHostToDevice, nullptr);
        if (e != cudaSuccess) return fail(cudaGetErrorString(e));
        rc = gemm_launch(p, p->ws[0], 0, p->ws[1], 0, p->ws[2], 0, scaled ? &dsc : nullptr, dbias, alpha, m, n, k, nullptr);
        if (rc != 0) return rc;
        e = cudaMemcpyAsync(c, p->ws[2], c_bytes, cudaMemcpyDeviceToHost, nullptr);
    } else {
        const int chunks = int((m + chunk_rows - 1) / chunk_rows);          // <= 16 by construction
        if (!p->s_in) {
            e = cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->s_cmp, cudaStreamNonBlocking);
            if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking);
            for (int i = 0; i < tesserae_gemm_plan::kMaxChunks && e == cudaSuccess; ++i) {
                e = cudaEventCreateWithFlags(&p->ev_in[i], cudaEventDisableTiming);
                if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->ev_cmp[i], cudaEventDisableTiming);
            }
            if (e == cudaSuccess) e = cudaEventCreateWithFlags(&p->ev_done, cudaEventDisableTiming);
            if (e != cudaSuccess) return fail(std::string(who) + ": " + cudaGetErrorString(e));
        }
        // work queued earlier on the default stream (by this thread) comes first
        e = cudaEventRecord(p->ev_done, nullptr);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_in, p->ev_done, 0);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_cmp, p->ev_done, 0);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_out, p->ev_done, 0);
        if (e == cudaSuccess) e = cudaMemcpyAsync(p->ws[1], b, b_bytes, cudaMemcpyHostToDevice, p->s_in);
        if (e == cudaSuccess && cfg.has_bias) e = cudaMemcpyAsync(p->ws[3], bias, size_t(n) * 2, cudaMemcpyHostToDevice, p->s_in);
        if (e == cudaSuccess && scaled) e = cudaMemcpyAsync(p->ws[5], scales->scale_b, sb_bytes, cudaMemcpyHostToDevice, p->s_in);
        if (e == cudaSuccess && scaled) e = cudaMemcpyAsync(p->ws[4], scales->scale_a, sa_bytes, cudaMemcpyHostToDevice, p->s_in);
        for (int i = 0; i < chunks && e == cudaSuccess; ++i) {
            const int64_t r0 = int64_t(i) * chunk_rows, rows = (m - r0 < chunk_rows) ? (m - r0) : chunk_rows;
            char* da = static_cast<char*>(p->ws[0]) + size_t(r0) * row_a;
            char* dc = static_cast<char*>(p->ws[2]) + size_t(r0) * row_c;
            e = cudaMemcpyAsync(da, static_cast<const char*>(a) + size_t(r0) * row_a, size_t(rows) * row_a, cudaMemcpyHostToDevice, p->s_in);
            if (e == cudaSuccess) e = cudaEventRecord(p->ev_in[i], p->s_in);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_cmp, p->ev_in[i], 0);
            if (e != cudaSuccess) break;
            // the chunk's rows of the A scale table: chunk boundaries are multiples of 256 rows, so they are whole rows
            // of the fp32 table and whole 128-row blocks of the chunked NVFP4 table
            tesserae_gemm_scales csc = dsc;
            if (scaled) csc.scale_a = static_cast<const char*>(p->ws[4]) + scale_table_bytes(cfg, true, r0, k);
            rc = gemm_launch(p, da, 0, p->ws[1], 0, dc, 0, scaled ? &csc : nullptr, dbias, alpha, rows, n, k, p->s_cmp);
            if (rc != 0) { cudaDeviceSynchronize(); return rc; }
            e = cudaEventRecord(p->ev_cmp[i], p->s_cmp);
            if (e == cudaSuccess) e = cudaStreamWaitEvent(p->s_out, p->ev_cmp[i], 0);
            if (e == cudaSuccess) e = cudaMemcpyAsync(static_cast<char*>(c) + size_t(r0) * row_c, dc, size_t(rows) * row_c, cudaMemcpyDeviceToHost, p->s_out);
        }
        // the default stream (status read below, and whatever the caller queues next) continues after the last copy
        if (e == cudaSuccess) e = cudaEventRecord(p->ev_done, p->s_out);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(nullptr, p->ev_done, 0);
    }
    uint32_t st = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&st, p->d_status, sizeof st, cudaMemcpyDeviceToHost, nullptr);
    if (e == cudaSuccess) e = cudaStreamSynchronize(nullptr);
    if (e != cudaSuccess) return fail(cudaGetErrorString(e));
    if (st != 0) {
        cudaMemset(p->d_status, 0, sizeof st);
        return fail(std::string(who) + ": kernel reported a timed-out wait, status=" + std::to_string(st));
    }
    return 0;
}

int tesserae_gemm_run_host(tesserae_gemm_plan* p, const void* a, const void* b, void* c, const void* bias,
                           float alpha, int64_t m, int64_t n, int64_t k) {
    return run_host_impl(p, a, b, c, nullptr, bias, alpha, m, n, k, "gemm_run_host");
}

int tesserae_gemm_run_scaled_host(tesserae_gemm_plan* p, const void* a, const void* b, void* c,
                                  const tesserae_gemm_scales* scales, const void* bias,
                                  float alpha, int64_t m, int64_t n, int64_t k) {
    if (!scales) return fail("gemm_run_scaled_host: null scales");
    return run_host_impl(p, a, b, c, scales, bias, alpha, m, n, k, "gemm_run_scaled_host");
}

int tesserae_runtime_run(const tesserae_kernel_spec* ks, int64_t m, int64_t n, int64_t k,
                         const float* a, const float* b, float* c) {
    if (!ks || !a || !b || !c) return fail("runtime_run: null argument");
    if (ks->elem != TESSERAE_BF16 && ks->elem != TESSERAE_F16)
        return fail("runtime_run: float arrays convert to F16 or BF16 only; use the typed entry points for narrower formats");
    if (m <= 0 || n <= 0 || k <= 0) return fail("runtime_run: M, N and K must be positive");
    tesserae_kernel_spec s = *ks;
    s.out_elem = TESSERAE_F32;   // Runtime.run returns a float array (lib/runtime/runtime.ml:69-72)
    s.has_bias = 0;
    tesserae_gemm_plan* plan = nullptr;
    int rc = tesserae_gemm_plan_create(&s, &plan);
    if (rc != 0) return rc;
    std::vector<uint16_t> ha(size_t(m) * k), hb(size_t(n) * k);
    if (ks->elem == TESSERAE_BF16) {
        for (size_t i = 0; i < ha.size(); ++i) ha[i] = f32_to_bf16(a[i]);
        for (size_t i = 0; i < hb.size(); ++i) hb[i] = f32_to_bf16(b[i]);
    } else {
        for (size_t i = 0; i < ha.size(); ++i) ha[i] = f32_to_f16(a[i]);
        for (size_t i = 0; i < hb.size(); ++i) hb[i] = f32_to_f16(b[i]);
    }
    rc = tesserae_gemm_run_host(plan, ha.data(), hb.data(), c, nullptr, 1.0f, m, n, k);
    const std::string keep = rc != 0 ? tesserae_last_error() : "";
    tesserae_gemm_plan_destroy(plan);
    if (rc != 0) tesserae::set_error(keep);
    return rc;
}

}  // extern "C"
