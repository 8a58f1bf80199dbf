/* A stand-in for libnccl used by the CPU tests of the communicator failure paths: it exports the handful of
 * NCCL entry points libtesserae_b200 binds and plays a peer that never joins (or joins late), so that the
 * deadline, abort and settle logic can be exercised with no GPU and no second rank.  Behaviour is set through
 * environment variables read at each call:
 *   FAKE_NCCL_READY_AFTER_MS   the communicator reports "in progress" until this many milliseconds after its
 *                              creation; unset or negative = never ready
 * Counters are read back through fake_nccl_counter(which). */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

typedef struct { char internal[128]; } ncclUniqueId;
enum { ncclSuccess = 0, ncclInvalidArgument = 4, ncclInProgress = 7 };

static int g_aborts, g_destroys, g_inits, g_collectives;
static struct timespec g_created;
static int g_fake_comm;

static long long ms_since_creation(void) {
    struct timespec now;
    clock_gettime(CLOCK_MONOTONIC, &now);
    return (now.tv_sec - g_created.tv_sec) * 1000LL + (now.tv_nsec - g_created.tv_nsec) / 1000000LL;
}
static int ready(void) {
    const char* e = getenv("FAKE_NCCL_READY_AFTER_MS");
    if (!e || !*e) return 0;
    const long long after = atoll(e);
    return after >= 0 && ms_since_creation() >= after;
}

int fake_nccl_counter(int which) { return which == 0 ? g_aborts : which == 1 ? g_destroys : which == 2 ? g_inits : g_collectives; }

int ncclGetVersion(int* v) { *v = 22809; return ncclSuccess; }
int ncclGetUniqueId(ncclUniqueId* id) { memset(id, 7, sizeof *id); return ncclSuccess; }
const char* ncclGetErrorString(int rc) { return rc == ncclInProgress ? "operation in progress" : rc == 0 ? "no error" : "fake error"; }
int ncclCommInitRank(void** comm, int n, ncclUniqueId id, int rank) {
    (void)n; (void)id; (void)rank;
    ++g_inits; clock_gettime(CLOCK_MONOTONIC, &g_created); *comm = &g_fake_comm; return ncclSuccess;
}
int ncclCommInitRankConfig(void** comm, int n, ncclUniqueId id, int rank, void* config) {
    (void)n; (void)id; (void)rank;
    /* the caller must ask for a non-blocking communicator: size_t size, unsigned magic, unsigned version, int blocking */
    const unsigned char* c = (const unsigned char*)config;
    unsigned magic; int blocking;
    memcpy(&magic, c + sizeof(size_t), sizeof magic);
    memcpy(&blocking, c + sizeof(size_t) + 2 * sizeof(unsigned), sizeof blocking);
    if (magic != 0xcafebeefu || blocking != 0) return ncclInvalidArgument;
    ++g_inits; clock_gettime(CLOCK_MONOTONIC, &g_created); *comm = &g_fake_comm; return ncclInProgress;
}
int ncclCommGetAsyncError(void* comm, int* state) { (void)comm; *state = ready() ? ncclSuccess : ncclInProgress; return ncclSuccess; }
int ncclCommAbort(void* comm) { (void)comm; ++g_aborts; return ncclSuccess; }
int ncclCommDestroy(void* comm) { (void)comm; ++g_destroys; return ncclSuccess; }
int ncclReduceScatter(const void* s, void* r, size_t n, int dt, int op, void* comm, void* stream) {
    (void)s; (void)r; (void)n; (void)dt; (void)op; (void)comm; (void)stream;
    ++g_collectives; return ncclInProgress;      /* a non-blocking communicator may answer this; the state settles at once */
}
int ncclAllReduce(const void* s, void* r, size_t n, int dt, int op, void* comm, void* stream) {
    (void)s; (void)r; (void)n; (void)dt; (void)op; (void)comm; (void)stream;
    ++g_collectives; return ncclSuccess;
}
