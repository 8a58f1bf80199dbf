// K-split GEMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc when they need a GEMM: a process whose own
// allocator (a tensor framework's caching pool, a database's buffer manager) already holds
// nearly all of the GPU's memory, so that a raw cudaMalloc fails; or a serving loop that cannot
// accept the device-wide synchronisation cudaMalloc and cudaFree imply.  The ordinary K-split
// entry point (tesserae_gemm_ksplit_run) leaves the fp32 partial products in scratch memory the
// caller passes in; this variant keeps that scratch in a fixed array inside the library image
// instead, so the call allocates nothing.
//
// The array bounds the problem: m * n * k_splits <= TESSERAE_NOALLOC_MAX_ELEMS (32 MiB of fp32).
//
// When the memory is reserved: CUDA loads a library's device code lazily, so the 32 MiB are taken
// on a device when this file's module is first touched there, which is the address lookup of the
// first call on that device, and are held until the process exits.  A host whose allocator is
// about to take the rest of the GPU's memory must therefore make one call (any call: even one
// that is refused for its size resolves the array first) per device at start-up, before its
// allocator grows and before any stream capture.  From then on calls allocate nothing.
#include "../../../include/tesserae_b200.h"
#include "../rt/errors.hpp"

#include <cuda_runtime.h>

#include <mutex>
#include <string>

using tesserae::fail;

namespace {

constexpr size_t kMaxElems = TESSERAE_NOALLOC_MAX_ELEMS;

// The scratch itself.  In host code this name is only a handle for the runtime, not a device
// address; the address a kernel can use comes from cudaGetSymbolAddress below.
static __device__ __align__(256) float g_ksplit_scratch[kMaxElems];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices] = {};   // device address of the array, per device ordinal
std::mutex g_setup_mutex;

// Once per device, with that device current: resolve the array's device address.
int scratch_for_current_device(float** out) {
    int dev = -1;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess) return fail(std::string("ksplit_noalloc: ") + cudaGetErrorString(rc));
    if (dev < 0 || dev >= kMaxDevices) return fail("ksplit_noalloc: device ordinal out of range");
    // A thread that has made no runtime call on this device yet has no context bound; the symbol lookup
    // binds the device's primary context to it, so nothing further down has to create one.
    thread_local int bound_dev = -1;
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[dev] || bound_dev != dev) {
        void* p = nullptr;
        rc = cudaGetSymbolAddress(&p, g_ksplit_scratch);
        if (rc != cudaSuccess) return fail(std::string("ksplit_noalloc: cudaGetSymbolAddress: ") + cudaGetErrorString(rc));
        if (!p) return fail("ksplit_noalloc: the scratch array has no device address");
        g_scratch_addr[dev] = static_cast<float*>(p);
        bound_dev = dev;
    }
    *out = g_scratch_addr[dev];
    return 0;
}

}  // namespace

extern "C" size_t tesserae_gemm_ksplit_noalloc_max_elems(void) { return kMaxElems; }

extern "C" int tesserae_gemm_ksplit_run_noalloc(tesserae_gemm_plan* plan, const void* a, const void* b, void* c_bf16,
                                                float alpha, int64_t m, int64_t n, int64_t k, int k_splits, void* stream) {
    // Resolve the array first: the first call on a device is what makes the driver load this module and reserve
    // the array there, and a start-up call made for that purpose may well carry sizes that are refused below.
    float* scratch = nullptr;
    int rc = scratch_for_current_device(&scratch);
    if (rc != 0) return rc;
    if (m <= 0 || n <= 0 || k <= 0 || k_splits < 1) return fail("ksplit_noalloc: M, N, K and k_splits must be positive");
    const unsigned __int128 need = (unsigned __int128)m * (unsigned __int128)n * (unsigned __int128)k_splits;
    if (need > kMaxElems)
        return fail("ksplit_noalloc: m * n * k_splits = " + std::to_string((unsigned long long)need) +
                    " fp32 partials exceed the built-in scratch of " + std::to_string(kMaxElems) +
                    " elements; use tesserae_gemm_ksplit_run with caller-provided scratch");
    // The GEMM overwrites every partial element it later sums, so nothing has to be cleared first.
    return tesserae_gemm_ksplit_run(plan, a, b, c_bf16, scratch, kMaxElems * sizeof(float), alpha, m, n, k, k_splits, stream);
}
