// Tirix: the structured kernel IR between a lowered descriptor and the emitted CUDA source.
//
// The reference routes its second emission path through this IR (lib/tirix/tirix.mli:103-222 data
// types, lib/tirix/desc_to_tirix.ml:466-508 lowering, lib/tirix/tirix_verify.ml:9-183 scope and
// structure checks, lib/tirix/tirix_emit.ml:481-501 emission).  This is the same IR restated for
// the sm_100a kernels of this library: the reference's statement forms (let / assign / op / if /
// for / pipeline / warp group / pragma / seq) and primitive operations (copy, MMA, the mbarrier
// and cluster barriers, TMEM alloc / dealloc / load / commit, shared-memory descriptor set-up),
// plus the operations the working kernels need and the reference's vocabulary lacks: bounded
// waits are the only kind of wait, TMA stores and TMA reduce-adds, TMEM stores (scale factors),
// the fp32 promotion of the block-scaled FP8 kernel, cluster-scope barrier arrivals.
//
// Expressions are kept as C-like text: the verifier only needs the identifiers an expression
// reads, and the emitter prints them as they are.
//
// The IR has a line-oriented text form (print / parse round-trip) so that a host in any language
// can build, inspect or edit a kernel's structure without linking C++ types.
#pragma once
#include "../emit/backend_sm100.hpp"

#include <string>
#include <vector>

namespace tesserae::tirix {

struct Var { std::string name; bool is_mutable = false; };

// Primitive operations (lib/tirix/tirix.mli:105-161, extended).
enum class OpKind {
    Copy,                // sub = CpAsync | TmaLoad | TmaPair | TmaStore | TmaReduceAdd | RegToSmem | SmemToReg; tensors = {src, dst}; var = mbar (optional)
    Mma,                 // sub = Sm100Tcgen05.<kind>; tensors = {a, b, c}; flag = accumulate; imm = cta_group
    CtaSync, WarpSync, MemFence,
    MbarInit,            // var = mbar, imm = count
    MbarArriveExpect,    // var = mbar, expr = bytes
    MbarWaitParity,      // var = mbar, expr = phase; always bounded: on expiry the role records `sub` (a status bit name) and leaves
    MbarArrive,          // var = mbar; flag = arrive on the leader CTA's barrier (cluster scope)
    ClusterArrive, ClusterWait,
    CpAsyncWaitAll, CpAsyncCommitGroup,
    BulkCommit, BulkWaitRead,          // TMA store groups; imm = groups left pending
    Tcgen05WaitLd, Tcgen05WaitSt, Tcgen05FenceBefore, Tcgen05FenceAfter,
    TmemAlloc, TmemDealloc,            // var = address variable, imm = columns
    TmemLoad,            // vars = destination registers, expr = source address, imm = column offset
    TmemStore,           // vars = source registers, expr = destination address, imm = column offset
    TmemCommit,          // var = mbar, imm = CTA mask (0 = this CTA only)
    SmemDescInit,        // var = descriptor, expr = pointer, imm = swizzle B
    ScaleFma,            // vars = {accumulators, partial, scale}: acc += partial * scale (fp32 promotion)
    StoreShared,         // vars = source registers, expr = address
    ClcTryCancel,        // var = mbar the 16-byte answer completes, expr = answer's address (cluster launch control)
    ClcQuery,            // vars = {cancelled, tile}: reads the answer at expr
    StoreCluster,        // var = value, expr = address in a CTA of the cluster (st.shared::cluster), imm = CTA rank
};

struct Op {
    OpKind kind = OpKind::CtaSync;
    std::string sub;
    std::vector<std::string> tensors;
    std::string var;
    std::vector<std::string> vars;
    std::string expr;
    int imm = 0;
    bool flag = false;
};

enum class StmtKind { Let, LetMut, Assign, OpStmt, If, For, Pipeline, WarpGroup, Pragma, Seq, Empty };

struct Stmt {
    StmtKind kind = StmtKind::Empty;
    Var var;                                   // Let / LetMut / Assign / For
    std::string expr, stop, step;              // Let value; If condition; For start / stop / step
    Op op;
    int role = -1;                             // WarpGroup: spec::Role
    int stages = 0;                            // Pipeline
    bool unroll = false;                       // For
    std::string text;                          // Pragma
    std::vector<Stmt> body, body2, body3;      // If: then / else; Pipeline: prologue / mainloop / epilogue
};

struct Tensor { std::string name; int space = 0; int elem = 0; spec::Ints shape, stride; int swizzle_b = 0; };
struct Param { std::string name; bool is_tma = false; };

struct Program {
    std::string name;
    int family = 2;
    std::vector<Param> params;
    std::vector<Tensor> tensors;
    long long smem_bytes = 0;
    spec::Cluster cluster{1, 1, 1, 1, {}};
    int pipeline_depth = 0;
    std::vector<Stmt> body;
    // The spec the program was lowered from (or parsed with): what emission specialises the mainloop on.
    tesserae_kernel_spec origin{};
    std::string origin_name, origin_tuning;    // storage behind origin.name / origin.tuning
};

// Desc_to_tirix.lower (lib/tirix/desc_to_tirix.ml:466-508) for the Blackwell family: the structure of the
// mainloop that `cfg` selects, role by role.
Program lower(const KernelConfig& cfg, const tesserae_kernel_spec& spec);

// Tirix_verify.verify (lib/tirix/tirix_verify.ml:9-183): scope and structure checks; the messages are the
// reference's.  Empty = Ok.
std::vector<std::string> verify(const Program& p);

// Text form (the printer of lib/tirix/tirix_pp.ml in spirit; this one parses back).
std::string print(const Program& p);
// Returns false and sets *err on a malformed text.
bool parse(const std::string& text, Program* out, std::string* err);

// Tirix_emit.emit (lib/tirix/tirix_emit.ml:481-501): IR -> the backend's record of source sections.  The
// program must verify, and its structure must be the structure of one of the hand-written mainloops (the one
// its origin spec selects): emission specialises that mainloop and carries the IR listing in the source header.
// Returns 0 or a TESSERAE_LOWER_* code with *msg set.
int emit(const Program& p, BackendOutput* out, std::string* msg);

// The operation kind with this name in the text form, or -1.
int op_kind_from_name(const std::string& name);

// Number of operations of one kind anywhere in the program (for tests and hosts that inspect structure).
int count_ops(const Program& p, OpKind kind);

}  // namespace tesserae::tirix
