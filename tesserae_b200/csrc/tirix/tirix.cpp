// Tirix IR: lowering from a kernel configuration, verifier, text form, emission.
// See tirix.hpp for what corresponds to which reference file.
#include "tirix.hpp"

#include <cctype>
#include <cstdlib>
#include <cstring>
#include <set>
#include <sstream>

namespace tesserae::tirix {

namespace {

// ---------------------------------------------------------------- names
const char* const kOpNames[] = {
    "Copy", "Mma", "CtaSync", "WarpSync", "MemFence", "MbarInit", "MbarArriveExpect", "MbarWaitParity", "MbarArrive",
    "ClusterArrive", "ClusterWait", "CpAsyncWaitAll", "CpAsyncCommitGroup", "BulkCommit", "BulkWaitRead",
    "Tcgen05WaitLd", "Tcgen05WaitSt", "Tcgen05FenceBefore", "Tcgen05FenceAfter", "TmemAlloc", "TmemDealloc", "TmemLoad",
    "TmemStore", "TmemCommit", "SmemDescInit", "ScaleFma", "StoreShared", "ClcTryCancel", "ClcQuery", "StoreCluster"};
constexpr int kNumOps = int(sizeof kOpNames / sizeof kOpNames[0]);
const char* const kRoleNames[] = {"Producer", "Consumer", "Epilogue", "Scheduler"};

int op_from_name(const std::string& s) {
    for (int i = 0; i < kNumOps; ++i) if (s == kOpNames[i]) return i;
    return -1;
}
int role_from_name(const std::string& s) {
    for (int i = 0; i < 4; ++i) if (s == kRoleNames[i]) return i;
    return -1;
}

// ---------------------------------------------------------------- builders
Stmt let(const std::string& name, const std::string& expr, bool mut = false) {
    Stmt s; s.kind = mut ? StmtKind::LetMut : StmtKind::Let; s.var = Var{name, mut}; s.expr = expr; return s;
}
Stmt assign(const std::string& name, const std::string& expr) {
    Stmt s; s.kind = StmtKind::Assign; s.var = Var{name, true}; s.expr = expr; return s;
}
Stmt opstmt(Op o) { Stmt s; s.kind = StmtKind::OpStmt; s.op = std::move(o); return s; }
Op mk(OpKind k) { Op o; o.kind = k; return o; }
Stmt barrier(OpKind k, const std::string& var = "", const std::string& expr = "", int imm = 0, const std::string& sub = "",
             bool flag = false) {
    Op o = mk(k); o.var = var; o.expr = expr; o.imm = imm; o.sub = sub; o.flag = flag; return opstmt(o);
}
Stmt copy(const std::string& kind, const std::string& src, const std::string& dst, const std::string& mbar = "") {
    Op o = mk(OpKind::Copy); o.sub = kind; o.tensors = {src, dst}; o.var = mbar; return opstmt(o);
}
Stmt iff(const std::string& cond, std::vector<Stmt> thn, std::vector<Stmt> els = {}) {
    Stmt s; s.kind = StmtKind::If; s.expr = cond; s.body = std::move(thn); s.body2 = std::move(els); return s;
}
Stmt forr(const std::string& var, const std::string& start, const std::string& stop, const std::string& step,
          std::vector<Stmt> body, bool unroll = false) {
    Stmt s; s.kind = StmtKind::For; s.var = Var{var, true}; s.expr = start; s.stop = stop; s.step = step;
    s.unroll = unroll; s.body = std::move(body); return s;
}
Stmt group(int role, std::vector<Stmt> body) { Stmt s; s.kind = StmtKind::WarpGroup; s.role = role; s.body = std::move(body); return s; }
Stmt wait(const std::string& mbar, const std::string& phase, const std::string& status_bit) {
    return barrier(OpKind::MbarWaitParity, mbar, phase, 0, status_bit);
}

}  // namespace

int op_kind_from_name(const std::string& name) { return op_from_name(name); }

// ---------------------------------------------------------------- lowering
Program lower(const KernelConfig& c, const tesserae_kernel_spec& ks) {
    Program p;
    p.name = c.name;
    p.family = c.desc.family;
    p.smem_bytes = c.smem_bytes;
    p.pipeline_depth = c.stages;
    p.origin = ks;
    p.origin_name = c.name;
    p.origin_tuning = (ks.tuning ? ks.tuning : "");
    const bool fp8blk = c.scale_mode == TESSERAE_SCALE_FP8_BLOCK, nvfp4 = c.scale_mode == TESSERAE_SCALE_NVFP4;
    const bool pair = c.cta_group == 2;
    const int row_bytes = 16 << c.desc.swizzle.b;

    // Cluster and roles of the kernel as built (the reference's six-warp table is Kernel_desc's; the mainloops use
    // four epilogue warps, and the block-scaled ones add promotion / scale warps, all under the Epilogue role).
    std::vector<std::pair<int, int>> roles = {{0, spec::Producer}, {1, spec::Consumer}};
    const int warps = c.threads / 32;
    for (int w = 2; w < warps; ++w) {
        const bool second_issuer = fp8blk && c.fp8_split && c.block_n == 256 && w == 2;
        const bool idle = fp8blk && (w == 3 || (w == 2 && !second_issuer));
        const bool clc_sched = c.clc && w == warps - 1;
        roles.push_back({w, second_issuer ? spec::Consumer : (idle || clc_sched) ? spec::Scheduler : spec::Epilogue});
    }
    p.cluster = spec::cluster_make(c.cta_group, 1, 1, warps, roles);

    // Parameters in launch order.
    p.params = {{"A_tmap", true}, {"B_tmap", true}, {c.scatter ? "C_tmaps" : "C_tmap", true}};
    if (c.grouped) p.params = {{"problem_table", false}, {"total_tiles", false}};   // the maps and sizes live in the table
    if (c.scatter) { p.params.push_back({"rows_per_owner", false}); p.params.push_back({"m_rotate", false}); }
    if (fp8blk) { p.params.push_back({"WS_tmap", true}); p.params.push_back({"scale_a", false}); p.params.push_back({"scale_b", false}); }
    if (nvfp4) { p.params.push_back({"SFA_tmap", true}); p.params.push_back({"SFB_tmap", true}); }
    if (c.grouped) p.params.push_back({"alpha", false});
    else for (const char* n : {"bias", "alpha", "M", "N", "K", "group_m"}) p.params.push_back({n, false});
    if (fp8blk) { p.params.push_back({"full_tiles", false}); p.params.push_back({"tail_splits", false}); }
    p.params.push_back({"status", false});

    // Tensors: global operands, the shared-memory ring (depth, rows, bytes of K : row-major inside a stage, the
    // layout the reference states column-major, lib/tirix/desc_to_tirix.ml:66-85), tensor memory, output staging.
    const int load_n = c.block_n / c.cta_group;
    p.tensors.push_back({"A", spec::Global, c.elem, {}, {}, 0});
    p.tensors.push_back({"B", spec::Global, c.elem, {}, {}, 0});
    p.tensors.push_back({"C", spec::Global, c.out_elem, {}, {}, 0});
    p.tensors.push_back({"smem_A", spec::Shared, c.elem, {c.stages, 128, row_bytes}, {128 * row_bytes, row_bytes, 1}, c.desc.swizzle.b});
    p.tensors.push_back({"smem_B", spec::Shared, c.elem, {c.stages, load_n, row_bytes}, {load_n * row_bytes, row_bytes, 1}, c.desc.swizzle.b});
    p.tensors.push_back({"smem_C", spec::Shared, c.out_elem, {32, 128}, {128, 1}, 3});
    const int acc_bufs = fp8blk ? (c.fp8_split ? 512 / 128 : 512 / c.block_n) : (nvfp4 && c.block_n == 256) ? 1 : 2;
    const int acc_cols = fp8blk ? (c.fp8_split ? 128 : c.block_n) : c.block_n;
    p.tensors.push_back({"tmem_acc", spec::TensorSpace, TESSERAE_F32, {acc_bufs, 128, acc_cols}, {acc_cols, 1 << 16, 1}, 0});
    if (nvfp4) {
        p.tensors.push_back({"SFA", spec::Global, TESSERAE_S8, {}, {}, 0});
        p.tensors.push_back({"SFB", spec::Global, TESSERAE_S8, {}, {}, 0});
        p.tensors.push_back({"smem_SFA", spec::Shared, TESSERAE_S8, {c.stages, 4, 512}, {2048, 512, 1}, 0});
        p.tensors.push_back({"smem_SFB", spec::Shared, TESSERAE_S8, {c.stages, 4 * (c.block_n / 128), 512}, {2048 * (c.block_n / 128), 512, 1}, 0});
        p.tensors.push_back({"tmem_SF", spec::TensorSpace, TESSERAE_S8, {c.stages, 32, 16 + 16 * (c.block_n / 128)}, {16 + 16 * (c.block_n / 128), 1 << 16, 1}, 0});
    }

    const std::string tile_m = std::to_string(128 * c.cta_group), bn = std::to_string(c.block_n);
    const std::string stages = std::to_string(c.stages);
    const std::string kblock = std::to_string(c.block_k);
    const std::string mma_kind = std::string("Sm100Tcgen05.") + (nvfp4 ? "mxf4nvf4.block_scale" : c.elem == TESSERAE_S8 ? "i8" :
                                 c.elem == TESSERAE_F8E4M3 ? "f8f6f4" : "f16");
    const long long stage_bytes = (128LL + load_n) * row_bytes * c.cta_group;

    std::vector<Stmt>& b = p.body;
    if (c.grouped) {
        // a grouped kernel reads its maps and sizes from the table row of the tile it is on
        for (const char* n : {"A_tmap", "B_tmap", "C_tmap", "bias", "M", "N", "K", "group_m"}) b.push_back(let(n, "problem_table"));
    }
    b.push_back(let("warp_id", "threadIdx.x / 32"));
    b.push_back(let("lane", "threadIdx.x % 32"));
    b.push_back(let("cta_rank", pair ? "cluster_ctarank" : "0"));
    b.push_back(let("num_m", "(M + " + tile_m + " - 1) / " + tile_m));
    b.push_back(let("num_n", "(N + " + bn + " - 1) / " + bn));
    b.push_back(let("num_tiles", "num_m * num_n"));
    b.push_back(let("num_k_blocks", "(K + " + kblock + " - 1) / " + kblock));
    b.push_back(let("first_tile", pair ? "clusterid.x" : "blockIdx.x"));
    b.push_back(let("tile_step", c.clc ? "0" : pair ? "nclusterid.x" : "gridDim.x"));   // (launch control: the ring gives the next tile)
    for (const char* bar : {"full_bar", "empty_bar", "tmem_full_bar", "tmem_empty_bar"}) b.push_back(let(bar, "smem_barriers"));
    if (nvfp4) { b.push_back(let("sf_full_bar", "smem_barriers")); b.push_back(let("sf_ready_bar", "smem_barriers")); }
    b.push_back(let("tmem_base", "0", true));
    if (c.clc) {
        // the scheduler's ring: the roles walk `sched_ring` instead of stepping by a fixed stride
        for (const char* bar : {"sched_full_bar", "sched_empty_bar", "clc_bar"}) b.push_back(let(bar, "smem_barriers"));
        b.push_back(let("clc_response", "smem_barriers"));
        b.push_back(let("sched_ring", "smem_barriers"));
    }

    // barrier set-up by one thread, then the TMEM allocation by the MMA warp
    int epi_warps_per_buffer = nvfp4 ? 8 : 4;
    if (fp8blk) {
        const int warp_cols = c.block_n / (c.promo_warps / 4), buf_cols = c.fp8_split ? 128 : c.block_n;
        epi_warps_per_buffer = 4 * buf_cols / warp_cols;
    }
    const int epi_arrivals = epi_warps_per_buffer * c.cta_group;
    std::vector<Stmt> init = {
        forr("s", "0", stages, "1", {barrier(OpKind::MbarInit, "full_bar", "", 1),
                                     barrier(OpKind::MbarInit, "empty_bar", "", fp8blk && c.fp8_split && c.block_n == 256 ? 2 : 1)}),
        forr("a", "0", std::to_string(acc_bufs), "1", {barrier(OpKind::MbarInit, "tmem_full_bar", "", 1),
                                                       barrier(OpKind::MbarInit, "tmem_empty_bar", "", epi_arrivals)})};
    if (nvfp4)
        init.push_back(forr("s", "0", stages, "1", {barrier(OpKind::MbarInit, "sf_full_bar", "", 1),
                                                    barrier(OpKind::MbarInit, "sf_ready_bar", "", 4 * c.cta_group)}));
    if (c.clc)
        init.push_back(forr("j", "0", "4", "1", {barrier(OpKind::MbarInit, "sched_full_bar", "", 1),
                                                 barrier(OpKind::MbarInit, "sched_empty_bar", "", c.cta_group + 1 + 4 * c.cta_group)}));
    if (c.clc) init.push_back(barrier(OpKind::MbarInit, "clc_bar", "", 1));
    b.push_back(iff("warp_id == 0 && lane == 0", init));
    if (pair) { b.push_back(barrier(OpKind::ClusterArrive)); b.push_back(barrier(OpKind::ClusterWait)); }
    Op alloc = mk(OpKind::TmemAlloc); alloc.var = "tmem_base"; alloc.imm = 512; alloc.sub = "cta_group::" + std::to_string(c.cta_group);
    if (fp8blk || nvfp4 || c.block_n * 2 > 256) alloc.imm = 512; else alloc.imm = c.block_n * 2 <= 32 ? 32 : c.block_n * 2 <= 64 ? 64 : c.block_n * 2 <= 128 ? 128 : 256;
    b.push_back(iff("warp_id == 1", {opstmt(alloc)}));
    b.push_back(barrier(OpKind::Tcgen05FenceBefore));
    if (pair) { b.push_back(barrier(OpKind::ClusterArrive)); b.push_back(barrier(OpKind::ClusterWait)); } else b.push_back(barrier(OpKind::CtaSync));
    b.push_back(barrier(OpKind::Tcgen05FenceAfter));

    // With the launch-control scheduler a role ends every tile by taking the next ring entry: bounded wait for the
    // entry, then its hand-back on the leader CTA's barrier.
    auto take_next = [&](std::vector<Stmt>& tile) {
        if (!c.clc) return;
        tile.push_back(wait("sched_full_bar", "(taken / 4) % 2", "TIMEOUT_SCHED"));
        tile.push_back(barrier(OpKind::MbarArrive, "sched_empty_bar", "", 0, "", true));
        tile.push_back(assign("taken", "taken + 1"));
    };
    // ---- producer: one lane walks tiles x K blocks, waits for a free stage, arms the byte count, issues the loads
    {
        std::vector<Stmt> kloop = {
            let("stage", "it % " + stages), let("phase", "(it / " + stages + ") % 2"),
            wait("empty_bar", "phase ^ 1", "TIMEOUT_EMPTY")};
        if (nvfp4) {
            kloop.push_back(barrier(OpKind::MbarArriveExpect, "sf_full_bar", std::to_string(2048 + 2048 * (c.block_n / 128))));
            kloop.push_back(copy("TmaLoad", "SFA", "smem_SFA", "sf_full_bar"));
            kloop.push_back(copy("TmaLoad", "SFB", "smem_SFB", "sf_full_bar"));
        }
        kloop.push_back(iff(pair ? "cta_rank == 0" : "1", {barrier(OpKind::MbarArriveExpect, "full_bar", std::to_string(stage_bytes))}));
        kloop.push_back(copy(pair ? "TmaPair" : "TmaLoad", "A", "smem_A", "full_bar"));
        kloop.push_back(copy(pair ? "TmaPair" : "TmaLoad", "B", "smem_B", "full_bar"));
        kloop.push_back(assign("it", "it + 1"));
        std::vector<Stmt> ptile = {forr("kb", "0", "num_k_blocks", "1", kloop)};
        take_next(ptile);
        std::vector<Stmt> body = {let("it", "0", true), let("taken", "0", true),
                                  forr("t", "first_tile", "num_tiles", "tile_step", ptile)};
        b.push_back(group(spec::Producer, {iff("lane == 0", body)}));
    }
    // ---- consumer: the MMA issuer (leader CTA of a pair); the whole warp waits, one elected lane issues
    {
        Op mma = mk(OpKind::Mma); mma.sub = mma_kind; mma.tensors = {"smem_A", "smem_B", "tmem_acc"}; mma.flag = !fp8blk; mma.imm = c.cta_group;
        Op da = mk(OpKind::SmemDescInit); da.var = "a_desc"; da.expr = "smem_A + stage"; da.imm = c.desc.swizzle.b;
        Op db = mk(OpKind::SmemDescInit); db.var = "b_desc"; db.expr = "smem_B + stage"; db.imm = c.desc.swizzle.b;
        Op free_stage = mk(OpKind::TmemCommit); free_stage.var = "empty_bar"; free_stage.imm = pair ? 3 : 0;
        Op acc_done = mk(OpKind::TmemCommit); acc_done.var = "tmem_full_bar"; acc_done.imm = pair ? 3 : 0;
        std::vector<Stmt> kloop = {let("stage", "it % " + stages), let("phase", "(it / " + stages + ") % 2")};
        if (fp8blk) kloop.push_back(wait("tmem_empty_bar", "acc_phase ^ 1", "TIMEOUT_TMEM_EMPTY"));
        kloop.push_back(wait("full_bar", "phase", "TIMEOUT_FULL"));
        if (nvfp4) kloop.push_back(wait("sf_ready_bar", "phase", "TIMEOUT_SCALE"));
        kloop.push_back(barrier(OpKind::Tcgen05FenceAfter));
        kloop.push_back(let("a_desc", "0")); kloop.push_back(let("b_desc", "0"));
        kloop.push_back(opstmt(da)); kloop.push_back(opstmt(db));
        kloop.push_back(forr("k", "0", std::to_string(row_bytes / 32), "1", {opstmt(mma)}, true));
        if (fp8blk) kloop.push_back(opstmt(acc_done));
        kloop.push_back(opstmt(free_stage));
        kloop.push_back(assign("it", "it + 1"));
        std::vector<Stmt> tile = {let("acc_phase", "(tile_iter / " + std::to_string(acc_bufs) + ") % 2")};
        if (!fp8blk) tile.push_back(wait("tmem_empty_bar", "acc_phase ^ 1", "TIMEOUT_TMEM_EMPTY"));
        tile.push_back(forr("kb", "0", "num_k_blocks", "1", kloop));
        if (!fp8blk) tile.push_back(opstmt(acc_done));
        tile.push_back(assign("tile_iter", "tile_iter + 1"));
        take_next(tile);
        b.push_back(group(spec::Consumer, {iff(pair ? "cta_rank == 0" : "1",
                                               {let("it", "0", true), let("tile_iter", "0", true), let("taken", "0", true),
                                                forr("t", "first_tile", "num_tiles", "tile_step", tile)})}));
    }
    // ---- scale warps (NVFP4): shared memory -> registers -> tensor memory, one warp per 32-lane quarter
    if (nvfp4) {
        Op st = mk(OpKind::TmemStore); st.vars = {"sf_regs"}; st.expr = "tmem_base + stage"; st.imm = 256;
        std::vector<Stmt> loop = {let("stage", "it % " + stages), let("phase", "(it / " + stages + ") % 2"),
                                  wait("sf_full_bar", "phase", "TIMEOUT_SCALE"), let("sf_regs", "0"),
                                  copy("SmemToReg", "smem_SFA", "tmem_SF"), copy("SmemToReg", "smem_SFB", "tmem_SF"), opstmt(st),
                                  barrier(OpKind::Tcgen05WaitSt), barrier(OpKind::Tcgen05FenceBefore), barrier(OpKind::WarpSync),
                                  barrier(OpKind::MbarArrive, "sf_ready_bar", "", 0, "", pair)};
        b.push_back(group(spec::Epilogue, {iff("warp_id >= 10", {forr("it", "0", "num_tiles * num_k_blocks", "1", loop)})}));
    }
    // ---- epilogue (and, for block-scaled FP8, the promotion in front of it)
    {
        Op ld = mk(OpKind::TmemLoad); ld.vars = {"frag"}; ld.expr = "tmem_base + acc"; ld.imm = 0;
        Op sts = mk(OpKind::StoreShared); sts.vars = {"frag"}; sts.expr = "smem_C + lane * 128";
        std::vector<Stmt> tile = {let("acc", "tile_iter % " + std::to_string(acc_bufs)),
                                  let("acc_phase", "(tile_iter / " + std::to_string(acc_bufs) + ") % 2"), let("frag", "0", true)};
        const Stmt release = barrier(OpKind::MbarArrive, "tmem_empty_bar", "", 0, "", pair);
        if (fp8blk) {
            Op fma = mk(OpKind::ScaleFma); fma.vars = {"accum", "frag", "scale"};
            tile.push_back(let("accum", "0", true));
            tile.push_back(forr("kb", "0", "num_k_blocks", "1",
                                {let("scale", "alpha * scale_a * scale_b"), wait("tmem_full_bar", "acc_phase", "TIMEOUT_TMEM_FULL"),
                                 barrier(OpKind::Tcgen05FenceAfter), opstmt(ld), barrier(OpKind::Tcgen05WaitLd),
                                 barrier(OpKind::Tcgen05FenceBefore), barrier(OpKind::WarpSync), release, opstmt(fma)}));
            sts.vars = {"accum"};
        } else {
            tile.push_back(wait("tmem_full_bar", "acc_phase", "TIMEOUT_TMEM_FULL"));
            tile.push_back(barrier(OpKind::Tcgen05FenceAfter));
            tile.push_back(opstmt(ld));
            tile.push_back(barrier(OpKind::Tcgen05WaitLd));
        }
        Op wr = mk(OpKind::BulkWaitRead); wr.imm = 1;
        tile.push_back(opstmt(wr));
        tile.push_back(opstmt(sts));
        tile.push_back(barrier(OpKind::MemFence));
        tile.push_back(barrier(OpKind::WarpSync));
        tile.push_back(iff("lane == 0", {copy(c.scatter == 2 ? "TmaReduceAdd" : "TmaStore", "smem_C", "C"), barrier(OpKind::BulkCommit)}));
        if (!fp8blk) { tile.push_back(barrier(OpKind::Tcgen05FenceBefore)); tile.push_back(barrier(OpKind::WarpSync)); tile.push_back(release); }
        tile.push_back(assign("tile_iter", "tile_iter + 1"));
        take_next(tile);
        const std::string who = fp8blk ? "warp_id >= 4" : nvfp4 ? "warp_id >= 2 && warp_id < 10" : c.clc ? "warp_id >= 2 && warp_id < " + std::to_string(warps - 1) : "warp_id >= 2";
        b.push_back(group(spec::Epilogue, {iff(who, {let("tile_iter", "0", true), let("taken", "0", true),
                                                     forr("t", "first_tile", "num_tiles", "tile_step", tile)})}));
    }
    // ---- scheduler (cluster launch control): one lane of the leader CTA's last warp cancels clusters that have not
    // started and feeds their tile ids to both CTAs of the pair
    if (c.clc) {
        Op tc = mk(OpKind::ClcTryCancel); tc.var = "clc_bar"; tc.expr = "clc_response";
        Op q = mk(OpKind::ClcQuery); q.vars = {"cancelled", "next_tile"}; q.expr = "clc_response";
        std::vector<Stmt> loop = {wait("sched_empty_bar", "((j / 4) % 2) ^ 1", "TIMEOUT_SCHED"),
                                  barrier(OpKind::MbarArriveExpect, "clc_bar", "16"), opstmt(tc),
                                  wait("clc_bar", "j % 2", "TIMEOUT_SCHED"),
                                  let("cancelled", "0", true), let("next_tile", "0", true), opstmt(q)};
        for (int r = 0; r < c.cta_group; ++r) {
            Op st = mk(OpKind::StoreCluster); st.var = "next_tile"; st.expr = "sched_ring + j % 4"; st.imm = r;
            loop.push_back(opstmt(st));
            loop.push_back(barrier(OpKind::MbarArrive, "sched_full_bar", "", 0, "", true));
        }
        b.push_back(group(spec::Scheduler, {iff("cta_rank == 0 && lane == 0", {forr("j", "0", "num_tiles", "1", loop)})}));
    }
    // ---- teardown
    b.push_back(barrier(OpKind::Tcgen05FenceBefore));
    if (pair) { b.push_back(barrier(OpKind::ClusterArrive)); b.push_back(barrier(OpKind::ClusterWait)); } else b.push_back(barrier(OpKind::CtaSync));
    Op dealloc = mk(OpKind::TmemDealloc); dealloc.var = "tmem_base"; dealloc.imm = alloc.imm; dealloc.sub = alloc.sub;
    b.push_back(iff("warp_id == 1", {barrier(OpKind::Tcgen05FenceAfter), opstmt(dealloc)}));
    return p;
}

// ---------------------------------------------------------------- verifier
namespace {

const std::set<std::string>& builtins() {
    static const std::set<std::string> b = {"threadIdx", "blockIdx", "gridDim", "blockDim", "x", "y", "z", "clusterid", "nclusterid",
                                            "cluster_ctarank", "smem_barriers", "true", "false"};
    return b;
}
std::vector<std::string> identifiers(const std::string& e) {
    std::vector<std::string> out;
    size_t i = 0;
    while (i < e.size()) {
        if (isalpha((unsigned char)e[i]) || e[i] == '_') {
            size_t j = i;
            while (j < e.size() && (isalnum((unsigned char)e[j]) || e[j] == '_')) ++j;
            out.push_back(e.substr(i, j - i));
            i = j;
        } else ++i;
    }
    return out;
}

struct Checker {
    const Program& p;
    std::vector<std::string> errors;
    std::set<std::string> tensor_names, globals;
    explicit Checker(const Program& prog) : p(prog) {
        for (auto& t : p.tensors) tensor_names.insert(t.name);
        for (auto& q : p.params) { tensor_names.insert(q.name); globals.insert(q.name); }
    }
    void err(const std::string& m) { errors.push_back(m); }
    void check_expr(const std::set<std::string>& scope, const std::string& e) {
        for (auto& id : identifiers(e))
            if (!scope.count(id) && !builtins().count(id) && !globals.count(id) && !tensor_names.count(id))
                err("undefined variable '" + id + "'");
    }
    void need_var(const std::set<std::string>& scope, const std::string& v, const std::string& what) {
        if (!scope.count(v)) err("undefined " + what);
    }
    void check_tensor(const std::string& name, const std::string& ctx) {
        if (!tensor_names.count(name)) err("unknown tensor '" + name + "' in " + ctx);
    }
    void check_op(const std::set<std::string>& scope, const Op& o) {
        switch (o.kind) {
            case OpKind::Copy:
                if (o.tensors.size() != 2) { err("copy needs a source and a destination tensor"); break; }
                check_tensor(o.tensors[0], "copy.src"); check_tensor(o.tensors[1], "copy.dst");
                if (!o.var.empty() && !scope.count(o.var)) err("undefined mbar '" + o.var + "' in copy");
                break;
            case OpKind::Mma:
                if (o.tensors.size() != 3) { err("mma needs three tensors"); break; }
                check_tensor(o.tensors[0], "mma.a"); check_tensor(o.tensors[1], "mma.b"); check_tensor(o.tensors[2], "mma.c");
                break;
            case OpKind::MbarInit: need_var(scope, o.var, "mbar '" + o.var + "' in MbarInit"); break;
            case OpKind::MbarArriveExpect: need_var(scope, o.var, "mbar '" + o.var + "' in MbarArriveExpect"); check_expr(scope, o.expr); break;
            case OpKind::MbarWaitParity:
                need_var(scope, o.var, "mbar '" + o.var + "' in MbarWaitParity"); check_expr(scope, o.expr);
                if (o.sub.empty()) err("MbarWaitParity on '" + o.var + "' names no status bit: every wait is bounded and reports its expiry");
                break;
            case OpKind::MbarArrive: need_var(scope, o.var, "mbar '" + o.var + "' in MbarArrive"); break;
            case OpKind::TmemAlloc: case OpKind::TmemDealloc: need_var(scope, o.var, "tmem addr '" + o.var + "'"); break;
            case OpKind::TmemLoad:
                for (auto& v : o.vars) need_var(scope, v, "dst var '" + v + "' in TmemLoad");
                check_expr(scope, o.expr); break;
            case OpKind::TmemStore:
                for (auto& v : o.vars) need_var(scope, v, "src var '" + v + "' in TmemStore");
                check_expr(scope, o.expr); break;
            case OpKind::TmemCommit: need_var(scope, o.var, "mbar '" + o.var + "' in TmemCommit"); break;
            case OpKind::SmemDescInit: need_var(scope, o.var, "desc var '" + o.var + "'"); check_expr(scope, o.expr); break;
            case OpKind::ClcTryCancel: need_var(scope, o.var, "mbar '" + o.var + "' in ClcTryCancel"); check_expr(scope, o.expr); break;
            case OpKind::ClcQuery:
                for (auto& v : o.vars) need_var(scope, v, "variable '" + v + "' in ClcQuery");
                check_expr(scope, o.expr); break;
            case OpKind::StoreCluster: need_var(scope, o.var, "variable '" + o.var + "' in StoreCluster"); check_expr(scope, o.expr); break;
            case OpKind::ScaleFma: case OpKind::StoreShared:
                for (auto& v : o.vars) need_var(scope, v, "variable '" + v + "'");
                check_expr(scope, o.expr); break;
            default: break;
        }
    }
    // returns the scope after the statement (a let extends the scope of what follows it, as in the reference)
    std::set<std::string> check_stmt(std::set<std::string> scope, const Stmt& s, std::set<std::string>* mut) {
        switch (s.kind) {
            case StmtKind::Let: case StmtKind::LetMut:
                check_expr(scope, s.expr); scope.insert(s.var.name);
                if (s.kind == StmtKind::LetMut) mut->insert(s.var.name); else mut->erase(s.var.name);
                return scope;
            case StmtKind::Assign:
                if (!scope.count(s.var.name)) err("undefined variable '" + s.var.name + "' in SAssign");
                else if (!mut->count(s.var.name)) err("assigning to immutable variable '" + s.var.name + "'");
                check_expr(scope, s.expr);
                return scope;
            case StmtKind::OpStmt: check_op(scope, s.op); return scope;
            case StmtKind::If:
                check_expr(scope, s.expr);
                check_block(scope, s.body, mut); check_block(scope, s.body2, mut);
                return scope;
            case StmtKind::For: {
                check_expr(scope, s.expr); check_expr(scope, s.stop);
                const std::string st = s.step;
                if (st == "0") err("SFor '" + s.var.name + "' has zero step");
                std::set<std::string> inner = scope; inner.insert(s.var.name);
                std::set<std::string> m2 = *mut; m2.insert(s.var.name);
                check_block(inner, s.body, &m2);
                return scope;
            }
            case StmtKind::Pipeline:
                if (s.stages <= 0) err("SPipeline has invalid stage count " + std::to_string(s.stages));
                check_block(scope, s.body, mut); check_block(scope, s.body2, mut); check_block(scope, s.body3, mut);
                return scope;
            case StmtKind::WarpGroup: {
                bool found = false;
                for (auto& r : p.cluster.roles) if (r.second == s.role) found = true;
                if (!found) err("SWarpGroup role not in cluster warp_roles");
                check_block(scope, s.body, mut);
                return scope;
            }
            case StmtKind::Pragma: check_block(scope, s.body, mut); return scope;
            case StmtKind::Seq: {
                std::set<std::string> sc = scope;
                for (auto& x : s.body) sc = check_stmt(sc, x, mut);
                return scope;
            }
            case StmtKind::Empty: return scope;
        }
        return scope;
    }
    void check_block(const std::set<std::string>& scope, const std::vector<Stmt>& body, std::set<std::string>* mut) {
        std::set<std::string> sc = scope;
        std::set<std::string> m = *mut;
        for (auto& s : body) sc = check_stmt(sc, s, &m);
    }
};

void count_in(const std::vector<Stmt>& body, OpKind k, int* n) {
    for (auto& s : body) {
        if (s.kind == StmtKind::OpStmt && s.op.kind == k) ++*n;
        count_in(s.body, k, n); count_in(s.body2, k, n); count_in(s.body3, k, n);
    }
}

}  // namespace

std::vector<std::string> verify(const Program& p) {
    Checker c(p);
    std::set<std::string> scope, mut;
    for (auto& s : p.body) scope = c.check_stmt(scope, s, &mut);
    // structure beyond scope: what a kernel that runs needs (no counterpart in the reference's verifier)
    if (p.family == 2) {
        int allocs = 0, deallocs = 0;
        count_in(p.body, OpKind::TmemAlloc, &allocs); count_in(p.body, OpKind::TmemDealloc, &deallocs);
        if (allocs != deallocs) c.err("tensor memory is allocated " + std::to_string(allocs) + " time(s) and freed " + std::to_string(deallocs));
    }
    if (p.pipeline_depth < 0) c.err("negative pipeline depth");
    return c.errors;
}

int count_ops(const Program& p, OpKind kind) { int n = 0; count_in(p.body, kind, &n); return n; }

// ---------------------------------------------------------------- text form
namespace {

std::string join(const spec::Ints& v) {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + std::to_string(v[i]);
    return s.empty() ? "-" : s;
}
std::string joins(const std::vector<std::string>& v) {
    std::string s;
    for (size_t i = 0; i < v.size(); ++i) s += (i ? "," : "") + v[i];
    return s;
}
void print_block(std::ostringstream& o, const std::vector<Stmt>& body, int depth);
void print_stmt(std::ostringstream& o, const Stmt& s, int depth) {
    const std::string ind(size_t(2 * depth), ' ');
    switch (s.kind) {
        case StmtKind::Let: o << ind << "let " << s.var.name << " = " << s.expr << "\n"; break;
        case StmtKind::LetMut: o << ind << "letmut " << s.var.name << " = " << s.expr << "\n"; break;
        case StmtKind::Assign: o << ind << "assign " << s.var.name << " = " << s.expr << "\n"; break;
        case StmtKind::OpStmt: {
            const Op& p = s.op;
            o << ind << "op " << kOpNames[int(p.kind)];
            if (!p.sub.empty()) o << " sub=" << p.sub;
            if (!p.tensors.empty()) o << " tensors=" << joins(p.tensors);
            if (!p.var.empty()) o << " var=" << p.var;
            if (!p.vars.empty()) o << " vars=" << joins(p.vars);
            if (p.imm != 0) o << " imm=" << p.imm;
            if (p.flag) o << " flag";
            if (!p.expr.empty()) o << " expr=" << p.expr;
            o << "\n";
            break;
        }
        case StmtKind::If:
            o << ind << "if " << s.expr << "\n"; print_block(o, s.body, depth + 1);
            if (!s.body2.empty()) { o << ind << "else\n"; print_block(o, s.body2, depth + 1); }
            o << ind << "end\n"; break;
        case StmtKind::For:
            o << ind << "for " << s.var.name << " = " << s.expr << " ; " << s.stop << " ; " << s.step << (s.unroll ? " unroll" : "") << "\n";
            print_block(o, s.body, depth + 1); o << ind << "end\n"; break;
        case StmtKind::Pipeline:
            o << ind << "pipeline stages=" << s.stages << "\n"; print_block(o, s.body, depth + 1);
            o << ind << "mainloop\n"; print_block(o, s.body2, depth + 1);
            o << ind << "epilogue\n"; print_block(o, s.body3, depth + 1); o << ind << "end\n"; break;
        case StmtKind::WarpGroup:
            o << ind << "warpgroup " << (s.role >= 0 && s.role < 4 ? kRoleNames[s.role] : "?") << "\n";
            print_block(o, s.body, depth + 1); o << ind << "end\n"; break;
        case StmtKind::Pragma: o << ind << "pragma " << s.text << "\n"; print_block(o, s.body, depth + 1); o << ind << "end\n"; break;
        case StmtKind::Seq: o << ind << "seq\n"; print_block(o, s.body, depth + 1); o << ind << "end\n"; break;
        case StmtKind::Empty: o << ind << "empty\n"; break;
    }
}
void print_block(std::ostringstream& o, const std::vector<Stmt>& body, int depth) { for (auto& s : body) print_stmt(o, s, depth); }

std::vector<std::string> split(const std::string& s, char sep) {
    std::vector<std::string> out; std::string cur;
    for (char ch : s) { if (ch == sep) { out.push_back(cur); cur.clear(); } else cur += ch; }
    out.push_back(cur);
    return out;
}
std::string trim(const std::string& s) {
    size_t a = 0, b = s.size();
    while (a < b && isspace((unsigned char)s[a])) ++a;
    while (b > a && isspace((unsigned char)s[b - 1])) --b;
    return s.substr(a, b - a);
}
spec::Ints ints_of(const std::string& s) {
    spec::Ints v;
    if (s == "-" || s.empty()) return v;
    for (auto& x : split(s, ',')) v.push_back(atoll(x.c_str()));
    return v;
}
// key=value tokens of a header line (values without spaces)
std::string kv(const std::vector<std::string>& toks, const std::string& key, const std::string& dflt = "") {
    for (auto& t : toks) if (t.compare(0, key.size() + 1, key + "=") == 0) return t.substr(key.size() + 1);
    return dflt;
}

struct Parser {
    std::vector<std::string> lines;
    size_t at = 0;
    std::string error;
    bool fail(const std::string& m) { if (error.empty()) error = "line " + std::to_string(at + 1) + ": " + m; return false; }
    // parses statements until a line that is one of `stops`; leaves `at` on that line
    bool block(std::vector<Stmt>* out, const std::set<std::string>& stops) {
        while (at < lines.size()) {
            const std::string ln = trim(lines[at]);
            if (ln.empty() || ln[0] == '#') { ++at; continue; }
            const std::string head = ln.substr(0, ln.find(' '));
            if (stops.count(head)) return true;
            Stmt s;
            if (head == "let" || head == "letmut" || head == "assign") {
                const size_t eq = ln.find(" = ");
                if (eq == std::string::npos) return fail("expected '<name> = <expr>'");
                s.kind = head == "let" ? StmtKind::Let : head == "letmut" ? StmtKind::LetMut : StmtKind::Assign;
                s.var = Var{trim(ln.substr(head.size(), eq - head.size())), head != "let"};
                s.expr = trim(ln.substr(eq + 3));
                ++at;
            } else if (head == "op") {
                std::string rest = trim(ln.substr(2));
                const size_t ex = rest.find(" expr=");
                std::string expr;
                if (ex != std::string::npos) { expr = rest.substr(ex + 6); rest = rest.substr(0, ex); }
                else if (rest.compare(0, 5, "expr=") == 0) { expr = rest.substr(5); rest.clear(); }
                std::vector<std::string> toks;
                for (auto& t : split(rest, ' ')) if (!t.empty()) toks.push_back(t);
                if (toks.empty()) return fail("op without a kind");
                const int k = op_from_name(toks[0]);
                if (k < 0) return fail("unknown op '" + toks[0] + "'");
                s.kind = StmtKind::OpStmt;
                s.op.kind = OpKind(k);
                s.op.sub = kv(toks, "sub");
                const std::string ts = kv(toks, "tensors"), vs = kv(toks, "vars");
                if (!ts.empty()) s.op.tensors = split(ts, ',');
                if (!vs.empty()) s.op.vars = split(vs, ',');
                s.op.var = kv(toks, "var");
                s.op.imm = atoi(kv(toks, "imm", "0").c_str());
                for (auto& t : toks) if (t == "flag") s.op.flag = true;
                s.op.expr = expr;
                ++at;
            } else if (head == "if") {
                s.kind = StmtKind::If; s.expr = trim(ln.substr(2)); ++at;
                if (!block(&s.body, {"else", "end"})) return false;
                if (at < lines.size() && trim(lines[at]) == "else") { ++at; if (!block(&s.body2, {"end"})) return false; }
                if (at >= lines.size()) return fail("if without end");
                ++at;
            } else if (head == "for") {
                s.kind = StmtKind::For;
                std::string rest = trim(ln.substr(3));
                if (rest.size() > 7 && rest.compare(rest.size() - 7, 7, " unroll") == 0) { s.unroll = true; rest = trim(rest.substr(0, rest.size() - 7)); }
                const size_t eq = rest.find(" = ");
                if (eq == std::string::npos) return fail("expected 'for <var> = <start> ; <stop> ; <step>'");
                s.var = Var{trim(rest.substr(0, eq)), true};
                const std::vector<std::string> parts = split(rest.substr(eq + 3), ';');
                if (parts.size() != 3) return fail("expected three ';'-separated loop expressions");
                s.expr = trim(parts[0]); s.stop = trim(parts[1]); s.step = trim(parts[2]);
                ++at;
                if (!block(&s.body, {"end"})) return false;
                if (at >= lines.size()) return fail("for without end");
                ++at;
            } else if (head == "pipeline") {
                s.kind = StmtKind::Pipeline;
                s.stages = atoi(kv(split(ln, ' '), "stages", "0").c_str());
                ++at;
                if (!block(&s.body, {"mainloop"})) return false;
                if (at >= lines.size()) return fail("pipeline without mainloop");
                ++at;
                if (!block(&s.body2, {"epilogue"})) return false;
                if (at >= lines.size()) return fail("pipeline without epilogue");
                ++at;
                if (!block(&s.body3, {"end"})) return false;
                if (at >= lines.size()) return fail("pipeline without end");
                ++at;
            } else if (head == "warpgroup" || head == "pragma" || head == "seq") {
                s.kind = head == "warpgroup" ? StmtKind::WarpGroup : head == "pragma" ? StmtKind::Pragma : StmtKind::Seq;
                const std::string arg = head.size() < ln.size() ? trim(ln.substr(head.size())) : "";
                if (head == "warpgroup") { s.role = role_from_name(arg); if (s.role < 0) return fail("unknown warp role '" + arg + "'"); }
                if (head == "pragma") s.text = arg;
                ++at;
                if (!block(&s.body, {"end"})) return false;
                if (at >= lines.size()) return fail(head + " without end");
                ++at;
            } else if (head == "empty") { s.kind = StmtKind::Empty; ++at; }
            else return fail("unknown statement '" + head + "'");
            out->push_back(std::move(s));
        }
        return true;
    }
};

}  // namespace

std::string print(const Program& p) {
    std::ostringstream o;
    o << "tirix " << p.name << " family=" << p.family << " smem_bytes=" << p.smem_bytes << " pipeline_depth=" << p.pipeline_depth
      << " cluster=" << p.cluster.x << "," << p.cluster.y << "," << p.cluster.z << " warps=" << p.cluster.num_warps << " roles=";
    for (size_t i = 0; i < p.cluster.roles.size(); ++i)
        o << (i ? "," : "") << p.cluster.roles[i].first << ":" << kRoleNames[p.cluster.roles[i].second];
    o << "\n";
    const tesserae_kernel_spec& k = p.origin;
    o << "origin arch=" << k.arch << " elem=" << k.elem << " tile=" << k.tile_m << "," << k.tile_n << "," << k.tile_k << " stages=" << k.stages
      << " cta_group=" << k.cta_group << " out_elem=" << k.out_elem << " has_bias=" << k.has_bias << " scale_mode=" << k.scale_mode
      << " scatter=" << k.scatter << " grouped=" << k.grouped << " tuning=" << (p.origin_tuning.empty() ? "-" : p.origin_tuning) << "\n";
    for (auto& q : p.params) o << "param " << q.name << " " << (q.is_tma ? "tma" : "ptr") << "\n";
    for (auto& t : p.tensors)
        o << "tensor " << t.name << " space=" << t.space << " elem=" << t.elem << " swizzle=" << t.swizzle_b << " shape=" << join(t.shape)
          << " stride=" << join(t.stride) << "\n";
    o << "body\n";
    print_block(o, p.body, 1);
    o << "end\n";
    return o.str();
}

bool parse(const std::string& text, Program* out, std::string* err) {
    Parser ps;
    ps.lines = split(text, '\n');
    Program p;
    bool have_header = false;
    while (ps.at < ps.lines.size()) {
        const std::string ln = trim(ps.lines[ps.at]);
        if (ln.empty() || ln[0] == '#') { ++ps.at; continue; }
        std::vector<std::string> toks;
        for (auto& t : split(ln, ' ')) if (!t.empty()) toks.push_back(t);
        if (toks[0] == "tirix") {
            if (toks.size() < 2) { ps.fail("tirix line needs a name"); break; }
            p.name = toks[1];
            p.family = atoi(kv(toks, "family", "2").c_str());
            p.smem_bytes = atoll(kv(toks, "smem_bytes", "0").c_str());
            p.pipeline_depth = atoi(kv(toks, "pipeline_depth", "0").c_str());
            const spec::Ints cl = ints_of(kv(toks, "cluster", "1,1,1"));
            if (cl.size() != 3) { ps.fail("cluster needs three dimensions"); break; }
            std::vector<std::pair<int, int>> roles;
            const std::string rs = kv(toks, "roles");
            if (!rs.empty())
                for (auto& r : split(rs, ',')) {
                    const size_t c = r.find(':');
                    const int role = c == std::string::npos ? -1 : role_from_name(r.substr(c + 1));
                    if (role < 0) { ps.fail("bad role entry '" + r + "'"); break; }
                    roles.push_back({atoi(r.substr(0, c).c_str()), role});
                }
            if (!ps.error.empty()) break;
            try { p.cluster = spec::cluster_make(int(cl[0]), int(cl[1]), int(cl[2]), atoi(kv(toks, "warps", "1").c_str()), roles); }
            catch (const std::exception& e) { ps.fail(e.what()); break; }
            have_header = true; ++ps.at;
        } else if (toks[0] == "origin") {
            tesserae_kernel_spec& k = p.origin;
            k.arch = atoi(kv(toks, "arch", "2").c_str()); k.elem = atoi(kv(toks, "elem", "1").c_str());
            const spec::Ints t = ints_of(kv(toks, "tile", "128,256,64"));
            if (t.size() != 3) { ps.fail("tile needs three numbers"); break; }
            k.tile_m = int(t[0]); k.tile_n = int(t[1]); k.tile_k = int(t[2]);
            k.stages = atoi(kv(toks, "stages", "0").c_str()); k.cta_group = atoi(kv(toks, "cta_group", "0").c_str());
            k.out_elem = atoi(kv(toks, "out_elem", "0").c_str()); k.has_bias = atoi(kv(toks, "has_bias", "0").c_str());
            k.scale_mode = atoi(kv(toks, "scale_mode", "0").c_str()); k.scatter = atoi(kv(toks, "scatter", "0").c_str());
            k.grouped = atoi(kv(toks, "grouped", "0").c_str());
            const std::string tun = kv(toks, "tuning", "-");
            p.origin_tuning = tun == "-" ? "" : tun;
            ++ps.at;
        } else if (toks[0] == "param") {
            if (toks.size() != 3) { ps.fail("expected 'param <name> tma|ptr'"); break; }
            p.params.push_back({toks[1], toks[2] == "tma"}); ++ps.at;
        } else if (toks[0] == "tensor") {
            if (toks.size() < 2) { ps.fail("tensor line needs a name"); break; }
            Tensor t; t.name = toks[1];
            t.space = atoi(kv(toks, "space", "0").c_str()); t.elem = atoi(kv(toks, "elem", "0").c_str());
            t.swizzle_b = atoi(kv(toks, "swizzle", "0").c_str());
            t.shape = ints_of(kv(toks, "shape", "-")); t.stride = ints_of(kv(toks, "stride", "-"));
            if (t.shape.size() != t.stride.size()) { ps.fail("incompatible shape and stride"); break; }
            p.tensors.push_back(t); ++ps.at;
        } else if (toks[0] == "body") {
            ++ps.at;
            if (!ps.block(&p.body, {"end"})) break;
            if (ps.at >= ps.lines.size()) { ps.fail("body without end"); break; }
            ++ps.at;
        } else { ps.fail("unknown line '" + toks[0] + "'"); break; }
    }
    if (ps.error.empty() && !have_header) ps.fail("no 'tirix' header line");
    if (!ps.error.empty()) { if (err) *err = ps.error; return false; }
    p.origin_name = p.name;
    *out = std::move(p);
    out->origin.name = out->origin_name.c_str();
    out->origin.tuning = out->origin_tuning.empty() ? nullptr : out->origin_tuning.c_str();
    return true;
}

// ---------------------------------------------------------------- emission
int emit(const Program& p, BackendOutput* out, std::string* msg) {
    const std::vector<std::string> errs = verify(p);
    if (!errs.empty()) {
        if (msg) { *msg = "InvalidPipeline: the program does not verify: " + errs[0]; if (errs.size() > 1) *msg += " (+" + std::to_string(errs.size() - 1) + " more)"; }
        return spec::InvalidPipeline;
    }
    tesserae_kernel_spec ks = p.origin;
    ks.name = p.name.c_str();
    ks.tuning = p.origin_tuning.empty() ? nullptr : p.origin_tuning.c_str();
    KernelConfig cfg;
    std::string why;
    const int rc = derive_config(ks, &cfg, &why);
    if (rc != 0) { if (msg) *msg = why; return rc; }
    // The hand-written mainloops are the only code this backend emits.  The IR decides which one and with which
    // parameters; a program whose statements differ from that mainloop's own structure describes a kernel this
    // backend has no code for, and is refused rather than silently replaced.
    const Program want = lower(cfg, ks);
    if (print(want) != print(p)) {
        if (msg) {
            std::istringstream a(print(want)), b(print(p));
            std::string la, lb; int n = 0;
            while (std::getline(a, la) && std::getline(b, lb)) { ++n; if (la != lb) break; }
            *msg = "IncompatibleTile: the program's structure is not that of the mainloop its origin selects (first difference at line " +
                   std::to_string(n) + ": expected '" + trim(la) + "', found '" + trim(lb) + "')";
        }
        return spec::IncompatibleTile;
    }
    *out = tesserae::emit(cfg);
    std::string listing = "// Tirix program this source was emitted from:\n";
    std::istringstream in(print(p));
    std::string ln;
    while (std::getline(in, ln)) listing += "//   " + ln + "\n";
    out->includes = listing + out->includes;
    out->full_source = listing + out->full_source;
    return 0;
}

}  // namespace tesserae::tirix
