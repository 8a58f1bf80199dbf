// NCCL behind the C ABI: what an OCaml (or any non-Python) host needs for the one exchange step of the
// K-split path — communicator set-up, reduce-scatter of the fp32 partials, tear-down.  libnccl is opened
// with dlopen on first use (like libcuda), so the library still loads where NCCL is absent.  The
// reference has no collective of any kind; these are new exports in the idiom of its plain-C layer
// (lib/runtime/nvrtc_stub.h:23-65: int status + message).
#include "../../../include/tesserae_b200.h"
#include "errors.hpp"

#include <dlfcn.h>
#include <chrono>
#include <climits>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

using tesserae::fail;

namespace {

struct NcclUniqueId { char internal[128]; };                 // ncclUniqueId: 128 opaque bytes, passed by value
typedef int (*GetVersionFn)(int*);
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(void**, int, NcclUniqueId, int);
typedef int (*CommDestroyFn)(void*);
typedef const char* (*GetErrorStringFn)(int);
typedef int (*ReduceScatterFn)(const void*, void*, size_t, int, int, void*, void*);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, void*);
// ncclConfig_t as NCCL 2.17 laid it out; the library reads `size` and `version` and fills the fields a newer
// layout adds with their defaults.
struct NcclConfig {
    size_t size; unsigned magic; unsigned version;
    int blocking, cga_cluster_size, min_ctas, max_ctas; const char* net_name; int split_share;
};
typedef int (*CommInitRankConfigFn)(void**, int, NcclUniqueId, int, NcclConfig*);
typedef int (*CommGetAsyncErrorFn)(void*, int*);
typedef int (*CommAbortFn)(void*);

struct Api {
    void* handle = nullptr;
    GetVersionFn get_version = nullptr;
    GetUniqueIdFn get_unique_id = nullptr;
    CommInitRankFn comm_init_rank = nullptr;
    CommDestroyFn comm_destroy = nullptr;
    GetErrorStringFn get_error_string = nullptr;
    ReduceScatterFn reduce_scatter = nullptr;
    AllReduceFn all_reduce = nullptr;
    // optional (NCCL >= 2.14): communicators that can be given up on
    CommInitRankConfigFn comm_init_rank_config = nullptr;
    CommGetAsyncErrorFn comm_get_async_error = nullptr;
    CommAbortFn comm_abort = nullptr;
};
Api g;
std::mutex g_mu;

constexpr int kNcclFloat32 = 7, kNcclSum = 0;               // ncclDataType_t / ncclRedOp_t values of nccl.h
constexpr int kNcclInProgress = 7;                          // ncclResult_t of a non-blocking communicator at work

std::string dl_message() {
    const char* e = dlerror();
    return e ? e : "no message from the loader";
}

int load_locked(const char* path) {
    if (g.handle) return 0;
    void* h = nullptr;
    std::string tried;
    if (path && *path) {
        h = dlopen(path, RTLD_NOW | RTLD_GLOBAL);
        if (!h) return fail(std::string("nccl: cannot open ") + path + ": " + dl_message());
    } else {
        if (const char* e = getenv("TESSERAE_NCCL_LIB")) {
            if (*e) {
                h = dlopen(e, RTLD_NOW | RTLD_GLOBAL);
                if (!h) tried = std::string(" ($TESSERAE_NCCL_LIB=") + e + " was tried first and failed: " + dl_message() + ")";
            }
        }
        if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return fail("nccl: cannot open libnccl.so.2: " + dl_message() + tried);
    }
    Api a;
    a.handle = h;
    a.get_version = reinterpret_cast<GetVersionFn>(dlsym(h, "ncclGetVersion"));
    a.get_unique_id = reinterpret_cast<GetUniqueIdFn>(dlsym(h, "ncclGetUniqueId"));
    a.comm_init_rank = reinterpret_cast<CommInitRankFn>(dlsym(h, "ncclCommInitRank"));
    a.comm_destroy = reinterpret_cast<CommDestroyFn>(dlsym(h, "ncclCommDestroy"));
    a.get_error_string = reinterpret_cast<GetErrorStringFn>(dlsym(h, "ncclGetErrorString"));
    a.reduce_scatter = reinterpret_cast<ReduceScatterFn>(dlsym(h, "ncclReduceScatter"));
    a.all_reduce = reinterpret_cast<AllReduceFn>(dlsym(h, "ncclAllReduce"));
    a.comm_init_rank_config = reinterpret_cast<CommInitRankConfigFn>(dlsym(h, "ncclCommInitRankConfig"));
    a.comm_get_async_error = reinterpret_cast<CommGetAsyncErrorFn>(dlsym(h, "ncclCommGetAsyncError"));
    a.comm_abort = reinterpret_cast<CommAbortFn>(dlsym(h, "ncclCommAbort"));
    if (!a.get_version || !a.get_unique_id || !a.comm_init_rank || !a.comm_destroy || !a.get_error_string ||
        !a.reduce_scatter || !a.all_reduce) {
        dlclose(h);
        return fail("nccl: the library lacks a required symbol");
    }
    g = a;
    return 0;
}
int ensure() {
    std::lock_guard<std::mutex> lk(g_mu);
    return load_locked(nullptr);
}
int nccl_fail(const char* what, int rc) {
    return fail(std::string(what) + ": " + (g.get_error_string ? g.get_error_string(rc) : "NCCL error") + " (" + std::to_string(rc) + ")");
}

// A call on a non-blocking communicator (one made by tesserae_nccl_comm_init_deadline) may answer "in progress":
// poll the communicator's state until it settles or `timeout_ms` pass.  Returns the settled NCCL result, or
// kNcclInProgress when the time ran out.
int settle(void* comm, int rc, long long timeout_ms) {
    if (rc != kNcclInProgress || !g.comm_get_async_error) return rc;
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        int state = 0;
        const int q = g.comm_get_async_error(comm, &state);
        if (q != 0) return q;
        if (state != kNcclInProgress) return state;
        if (std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count() > timeout_ms)
            return kNcclInProgress;
        std::this_thread::sleep_for(std::chrono::milliseconds(1));
    }
}
constexpr long long kCollectiveSettleMs = 60000;

}  // namespace

extern "C" {

int tesserae_nccl_load(const char* path) {
    std::lock_guard<std::mutex> lk(g_mu);
    return load_locked(path);
}

int tesserae_nccl_version(int* version) {
    if (!version) return fail("nccl_version: null output");
    if (int rc = ensure()) return rc;
    const int rc = g.get_version(version);
    return rc == 0 ? 0 : nccl_fail("ncclGetVersion", rc);
}

int tesserae_nccl_unique_id(void* id128) {
    if (!id128) return fail("nccl_unique_id: null output");
    if (int rc = ensure()) return rc;
    NcclUniqueId id;
    const int rc = g.get_unique_id(&id);
    if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
    std::memcpy(id128, &id, sizeof id);
    return 0;
}

int tesserae_nccl_comm_init(void** comm, int world, int rank, const void* id128) {
    if (!comm || !id128) return fail("nccl_comm_init: null argument");
    if (world < 1 || rank < 0 || rank >= world) return fail("nccl_comm_init: rank must be in [0, world)");
    if (int rc = ensure()) return rc;
    NcclUniqueId id;
    std::memcpy(&id, id128, sizeof id);
    void* c = nullptr;
    const int rc = g.comm_init_rank(&c, world, id, rank);
    if (rc != 0) return nccl_fail("ncclCommInitRank", rc);
    *comm = c;
    return 0;
}

int tesserae_nccl_comm_init_deadline(void** comm, int world, int rank, const void* id128, int timeout_ms) {
    if (!comm || !id128) return fail("nccl_comm_init_deadline: null argument");
    if (world < 1 || rank < 0 || rank >= world) return fail("nccl_comm_init_deadline: rank must be in [0, world)");
    if (timeout_ms <= 0) return fail("nccl_comm_init_deadline: timeout_ms must be positive");
    if (int rc = ensure()) return rc;
    if (!g.comm_init_rank_config || !g.comm_get_async_error || !g.comm_abort)
        return fail("nccl_comm_init_deadline: this NCCL has no non-blocking communicators (needs 2.14 or later)");
    NcclUniqueId id;
    std::memcpy(&id, id128, sizeof id);
    NcclConfig cfg;
    cfg.size = sizeof cfg; cfg.magic = 0xcafebeefu; cfg.version = 21700;
    cfg.blocking = 0;                                       // return at once; progress is polled below
    cfg.cga_cluster_size = INT_MIN; cfg.min_ctas = INT_MIN; cfg.max_ctas = INT_MIN;   // "undefined": library defaults
    cfg.net_name = nullptr; cfg.split_share = INT_MIN;
    void* c = nullptr;
    int rc = g.comm_init_rank_config(&c, world, id, rank, &cfg);
    if (rc != 0 && rc != kNcclInProgress) return nccl_fail("ncclCommInitRankConfig", rc);
    rc = settle(c, kNcclInProgress, timeout_ms);
    if (rc == 0) { *comm = c; return 0; }
    // A peer never joined (or set-up failed): give the half-made communicator up so that nothing keeps waiting.
    if (c) g.comm_abort(c);
    *comm = nullptr;
    if (rc == kNcclInProgress)
        return fail("nccl_comm_init_deadline: the communicator was not ready after " + std::to_string(timeout_ms) +
                    " ms (a rank did not join); it was aborted");
    return nccl_fail("ncclCommInitRankConfig", rc);
}

int tesserae_nccl_comm_abort(void* comm) {
    if (!comm) return 0;
    if (int rc = ensure()) return rc;
    if (!g.comm_abort) return fail("nccl_comm_abort: this NCCL has no ncclCommAbort");
    const int rc = g.comm_abort(comm);
    return rc == 0 ? 0 : nccl_fail("ncclCommAbort", rc);
}

int tesserae_nccl_comm_destroy(void* comm) {
    if (!comm) return 0;
    if (int rc = ensure()) return rc;
    const int rc = g.comm_destroy(comm);
    return rc == 0 ? 0 : nccl_fail("ncclCommDestroy", rc);
}

int tesserae_nccl_reduce_scatter_f32(void* comm, const void* send, void* recv, size_t recv_count, void* stream) {
    if (!comm || !send || !recv) return fail("nccl_reduce_scatter_f32: null argument");
    if (int rc = ensure()) return rc;
    const int rc = settle(comm, g.reduce_scatter(send, recv, recv_count, kNcclFloat32, kNcclSum, comm, stream), kCollectiveSettleMs);
    return rc == 0 ? 0 : nccl_fail("ncclReduceScatter", rc);
}

int tesserae_nccl_all_reduce_f32(void* comm, const void* send, void* recv, size_t count, void* stream) {
    if (!comm || !send || !recv) return fail("nccl_all_reduce_f32: null argument");
    if (int rc = ensure()) return rc;
    const int rc = settle(comm, g.all_reduce(send, recv, count, kNcclFloat32, kNcclSum, comm, stream), kCollectiveSettleMs);
    return rc == 0 ? 0 : nccl_fail("ncclAllReduce", rc);
}

}  // extern "C"
