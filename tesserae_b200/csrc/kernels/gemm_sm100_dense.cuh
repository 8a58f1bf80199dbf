// Dense GEMM mainloop for sm_100a:  C[M,N] = alpha * (A[M,K] . B[N,K]^T) (+ bias[n]),
// A and B K-contiguous ("A row-major MxK, B column-major KxN"), fp32 accumulation in
// tensor memory, output bf16 or fp32.  It is the working form of the Blackwell template
// of the reference (lib/backend/backend_cute.ml:146-157 producer, :178-214 consumer,
// :218-235 epilogue, :257-366 kernel function): same block of 192 threads and the same
// producer / consumer / epilogue warp split (lib/kernel/kernel_desc.ml:128-135), the same
// smem ring addressed by stage = iter % depth, phase = (iter / depth) % 2
// (lib/pipeline/pipeline.ml:17-21) and the same per-stage byte count
// (bm + bn/2) * bk * bytes for a CTA pair (lib/pipeline/tile_io.ml:119-127).
//
// Differences from that sketch, all needed for a kernel that runs: 4 epilogue warps
// (warps 2..5, one per 32-lane TMEM quarter; 8 for the 512-column tile), empty-slot barriers
// armed by tcgen05.commit, a persistent tile loop with two TMEM accumulator buffers
// (lib/pipeline/tmem.ml:106-110) so that the epilogue of tile i overlaps the mainloop of tile
// i+1 (one buffer, handed back in two column groups, for the 512-column tile), a real instruction
// descriptor and shared-memory descriptors, a TMA-store epilogue with fused alpha, bias
// and cast, and bounded waits.  The SM100 load strategy tag of the reference
// (lib/pipeline/tile_io.ml:28-32) is lowered to per-CTA TMA loads: in a CTA pair each CTA
// loads its own 128 rows of A and its own half of the B tile, and the pair MMA
// (cta_group::2) reads both halves, so no operand byte is fetched twice by the pair.
//
// Compile-time configuration (macros, set by the emitter in front of this text):
//   TS_KERNEL_NAME   extern "C" symbol
//   TS_CTA_GROUP     1 or 2 (CTAs per MMA; 2 needs cluster dims (2,1,1))
//   TS_BLOCK_N       tile width (multiple of 16*TS_CTA_GROUP, <= 256: one MMA per K step; or 512 for a CTA pair: two
//                    MMA groups of 256 columns per K step, 320 threads -- see kMmaN below)
//   TS_STAGES        depth of the smem ring
//   TS_ELEM_BYTES    2 (bf16/f16) or 1 (e4m3)
//   TS_SWIZZLE_B     B of the operand tiles' Swizzle<B,4,3> (1..3), as Swizzle.smem_selector derives it from the
//                    spec's tile.k: one stage holds 16 << B bytes of K per row
//   TS_MMA_KIND      TS_KIND_F16, TS_KIND_F8F6F4 or TS_KIND_I8 (signed 8-bit operands, 32-bit integer accumulation)
//   TS_AB_FMT        operand format code of the instruction descriptor
//   TS_OUT_F32       0: bf16 output, 1: fp32 output
//   TS_HAS_BIAS      0/1: add bias[n] (bf16) after alpha scaling
//   TS_SCATTER       0/1: row-scattered output.  Rows [g*rows_per_owner, (g+1)*rows_per_owner) of C are
//                    stored through tensor map g of an array of up to 8 (one per owner), at row
//                    (row - g*rows_per_owner).  With maps that point into the owners' memory this is the
//                    GEMM -> reduce-scatter fusion of the K-split: each GPU's fp32 partial tiles go straight
//                    to the GPU that owns the rows (plain TMA stores over NVLink), tile by tile, while the
//                    mainloop continues; the owner then sums its G slots.
//                    TS_SCATTER 2: the same routing, but each tile is ADDED into the owner's buffer (TMA reduce, fp32
//                    add at the destination) instead of stored to a per-source slot: all G GPUs add into one
//                    M/G x N fp32 array per owner, which must hold zeros beforehand; no sum pass follows, only the
//                    cast.  The order in which the G contributions meet is not fixed, so beyond two GPUs the fp32
//                    sum can differ in the last place from run to run.
//                    m_rotate (scattered kernels): the tile order is rotated by this many M-tiles.  GPUs that run
//                    the same schedule would all send to the same owner at the same time (the rows of the first
//                    raster group) and queue up on that owner's NVLink ingress; with a different rotation per
//                    source GPU the owners are visited round robin.
//   TS_GROUPED       0/1: grouped GEMM.  One launch walks the tiles of a list of independent problems (each with its
//                    own A, B, C, bias, M, N, K): the problems' tensor maps and sizes sit in a table in global
//                    memory (TsGroupedProblem, written by the host before the launch), global tile t belongs to the
//                    problem whose [tile_start, next tile_start) holds it, and every role looks its problem up as
//                    it moves from tile to tile.  Tiles of different problems fill one wave together, so a list of
//                    small problems is not quantised problem by problem.
//   TS_CLC           0/1: dynamic tile order by cluster launch control -- the role the reference reserves a warp for
//                    (lib/pipeline/cluster.mli:17-21: "Scheduler: issues CLC try_cancel, feeds tile ids").  The grid
//                    has one cluster per tile instead of one per SM (pair).  Every cluster that runs computes its own
//                    tile and then, through its scheduler warp (the last warp of the leader CTA), asks the hardware to
//                    cancel a cluster that has not started yet and takes that cluster's tile, until no cluster is
//                    left to cancel.  A cluster that finishes a short tile early takes the next tile at once, so
//                    tiles of unequal length (a grouped launch of problems with different K) do not wait for a
//                    fixed round-robin turn.  Tile ids go to the roles of both CTAs through a ring of kSchedRing
//                    entries in shared memory with a full and an empty barrier per entry.
#pragma once

#ifndef TS_CLC
#define TS_CLC 0
#endif
#ifndef TS_GROUPED
#define TS_GROUPED 0
#endif
#if TS_GROUPED
// One row of the problem table; the table has n + 1 rows, the last one holding only tile_start = total tiles.
struct __align__(64) TsGroupedProblem {
    TsTensorMap a, b, c;
    const ts_u16* bias;
    int M, N, K;
    int tile_start, num_m, num_n, group_m;
    int pad[7];
};
static_assert(sizeof(TsGroupedProblem) == 448, "host and device must agree on the problem table's row");
#endif

#ifndef TS_SCATTER
#define TS_SCATTER 0
#endif
#if TS_SCATTER
struct TsTensorMapArray8 { TsTensorMap m[8]; };
#endif

#ifndef TS_SWIZZLE_B
#define TS_SWIZZLE_B 3
#endif

namespace ts_dense {

constexpr ts_u32 kBlockM      = 128;                          // rows per CTA
constexpr ts_u32 kTileM       = kBlockM * TS_CTA_GROUP;       // rows per MMA tile
constexpr ts_u32 kBlockN      = TS_BLOCK_N;
// One MMA instruction is at most 256 columns wide.  A 512-wide tile (CTA pairs only) is two MMA groups per K step,
// each into its own 256 columns of tensor memory: it streams (128 + 256) rows of operands per 1024 tensor cycles and
// CTA, 48 bytes per clock from L2 where the 256-wide tile needs 64 -- and 64 is what an SM can take, so the narrower
// tile runs at the supply limit (measured: with a quarter of the operand loads left out it is 15 % faster).  The
// price is one accumulator instead of two: the epilogue hands the halves back one by one, and the next tile's MMAs
// wait for them.
constexpr ts_u32 kMmaN        = kBlockN > 256 ? 256 : kBlockN;
constexpr ts_u32 kHalves      = kBlockN / kMmaN;              // MMA groups per K step
constexpr ts_u32 kLoadN       = kBlockN / TS_CTA_GROUP;       // B rows this CTA loads
constexpr ts_u32 kHalfRows    = kMmaN / TS_CTA_GROUP;         // of which one MMA group reads this many
constexpr ts_u32 kBlockKBytes = 16u << TS_SWIZZLE_B;          // one swizzle row: 32, 64 or 128 bytes of K
constexpr ts_u32 kBlockK      = kBlockKBytes / TS_ELEM_BYTES; // K elements per stage
constexpr ts_u32 kUmmaKBytes  = 32;                           // K bytes per MMA instruction
constexpr ts_u32 kNumUmma     = kBlockKBytes / kUmmaKBytes;   // MMAs per stage (4 with 128-byte rows)
constexpr ts_u32 kStages      = TS_STAGES;
constexpr ts_u32 kSmemA       = kBlockM * kBlockKBytes;       // 16384
constexpr ts_u32 kSmemB       = kLoadN * kBlockKBytes;
constexpr ts_u32 kStageBytes  = kSmemA + kSmemB;
constexpr ts_u32 kNumAcc      = 2 * kBlockN <= 512 ? 2 : 1;   // TMEM accumulator buffers
constexpr ts_u32 kTmemCols    = (kNumAcc * kBlockN <= 32) ? 32 : (kNumAcc * kBlockN <= 64) ? 64 :
                                (kNumAcc * kBlockN <= 128) ? 128 : (kNumAcc * kBlockN <= 256) ? 256 : 512;
constexpr ts_u32 kOutBytes    = TS_OUT_F32 ? 4 : 2;
constexpr ts_u32 kChunkCols   = 128 / kOutBytes;              // output columns per 128-byte staging row
constexpr ts_u32 kNumChunks   = kBlockN / kChunkCols;
constexpr ts_u32 kStoreBuf    = 32 * 128;                     // one warp's staging buffer: 32 rows x 128 B
// Four epilogue warps (one per 32-lane quarter of tensor memory); eight for the 512-column tile, two per quarter that
// take alternate store chunks, because there the accumulator's hand-back is exposed and has to be quick.
constexpr ts_u32 kNumEpiWarps = kHalves == 2 ? 8 : 4;
constexpr ts_u32 kEpiSplit    = kNumEpiWarps / 4;             // warps that share a lane quarter
#ifndef TS_STORE_BUFS
#define TS_STORE_BUFS 2
#endif
constexpr ts_u32 kStoreBufs   = TS_STORE_BUFS;                // staging buffers per epilogue warp (stores in flight + 1)
constexpr ts_u32 kSmemC       = kNumEpiWarps * kStoreBufs * kStoreBuf;
constexpr ts_u32 kSchedRing   = 4;                            // tile ids in flight between the scheduler warp and the roles
constexpr ts_u32 kNumBars     = 2 * kStages + kNumAcc + kNumAcc * kHalves + (TS_CLC ? 2 * kSchedRing + 1 : 0);
constexpr ts_u32 kSmemTotal   = kStages * kStageBytes + kSmemC + kNumBars * 8 + 16 + (TS_CLC ? 48 : 0);
constexpr ts_u32 kThreads     = 64 + 32 * kNumEpiWarps + (TS_CLC ? 32 : 0);   // producer, MMA issuer, epilogue warps (+ scheduler)
constexpr ts_u32 kNoTile      = 0xffffffffu;
// Arrivals that hand a ring entry back: the producer lane of each CTA, the MMA warp (leader only), the epilogue warps.
constexpr ts_u32 kSchedReaders = TS_CTA_GROUP + 1 + kNumEpiWarps * TS_CTA_GROUP;

static_assert(kBlockN % (16 * TS_CTA_GROUP) == 0 && kBlockN >= 16 * TS_CTA_GROUP && (kBlockN <= 256 || (kBlockN == 512 && TS_CTA_GROUP == 2)),
              "bad TS_BLOCK_N");
static_assert(kNumChunks % kHalves == 0, "a store chunk must not straddle two MMA groups");
static_assert((kNumChunks / kHalves) % kEpiSplit == 0, "the warps that share a lane quarter take equal shares of each MMA group");
static_assert(kBlockN % kChunkCols == 0, "TS_BLOCK_N must be a multiple of the store chunk");
static_assert(kNumAcc * kBlockN <= 512, "accumulators exceed tensor memory");
static_assert(kSmemTotal + 1024 <= 232448, "shared memory over the 227 KB limit");

// What a role needs to know about the tile it is on.
struct TileInfo {
    ts_u32 local_tile, num_m, num_n, num_k_blocks, group_m;
    int M, N;
    const TsTensorMap *a, *b, *c;
    const ts_u16* bias;
};
#if TS_GROUPED
// `cursor` is the problem the previous tile of this role belonged to: with the static order tiles only move forward;
// a dynamic order may hand out an earlier tile, and the search starts over.
TS_DEV TileInfo tile_info(const TsGroupedProblem* probs, ts_u32 t, ts_u32& cursor) {
    if (TS_CLC && t < (ts_u32)__ldg(&probs[cursor].tile_start)) cursor = 0;
    while (t >= (ts_u32)__ldg(&probs[cursor + 1].tile_start)) ++cursor;
    const TsGroupedProblem* pr = probs + cursor;
    TileInfo ti;
    ti.local_tile = t - (ts_u32)__ldg(&pr->tile_start);
    ti.num_m = (ts_u32)__ldg(&pr->num_m); ti.num_n = (ts_u32)__ldg(&pr->num_n); ti.group_m = (ts_u32)__ldg(&pr->group_m);
    ti.M = __ldg(&pr->M); ti.N = __ldg(&pr->N);
    ti.num_k_blocks = ((ts_u32)__ldg(&pr->K) + kBlockK - 1) / kBlockK;
    ti.a = &pr->a; ti.b = &pr->b; ti.c = &pr->c;
    ti.bias = reinterpret_cast<const ts_u16*>(__ldg(reinterpret_cast<const ts_u64*>(&pr->bias)));
    return ti;
}
#endif

}  // namespace ts_dense

extern "C" __global__ void __launch_bounds__(64 + 32 * (TS_BLOCK_N > 256 ? 8 : 4) + (TS_CLC ? 32 : 0), 1)
#if TS_GROUPED
TS_KERNEL_NAME(const TsGroupedProblem* __restrict__ probs, int total_tiles, float alpha, ts_u32* __restrict__ status)
#else
TS_KERNEL_NAME(const __grid_constant__ TsTensorMap tmap_a,
               const __grid_constant__ TsTensorMap tmap_b,
#if TS_SCATTER
               const __grid_constant__ TsTensorMapArray8 tmap_cs, int rows_per_owner, int m_rotate,
#else
               const __grid_constant__ TsTensorMap tmap_c,
#endif
               const ts_u16* __restrict__ bias,
               float alpha, int M, int N, int K, int group_m,
               ts_u32* __restrict__ status)
#endif
{
    using namespace ts_dense;
    extern __shared__ ts_u8 ts_smem_raw[];
    // 128-byte-swizzled tiles need 1024-byte alignment.
    const ts_u32 smem_base = (ts_smem_u32(ts_smem_raw) + 1023u) & ~1023u;
    const ts_u32 smem_a    = smem_base;
    const ts_u32 smem_b    = smem_a + kStages * kSmemA;
    const ts_u32 smem_c    = smem_b + kStages * kSmemB;
    const ts_u32 bar_base  = smem_c + kSmemC;
    const ts_u32 full_bar       = bar_base;                       // [kStages]
    const ts_u32 empty_bar      = full_bar + 8 * kStages;         // [kStages]
    const ts_u32 tmem_full_bar  = empty_bar + 8 * kStages;        // [kNumAcc]
    const ts_u32 tmem_empty_bar = tmem_full_bar + 8 * kNumAcc;    // [kNumAcc][kHalves]
#if TS_CLC
    const ts_u32 sched_full     = tmem_empty_bar + 8 * kNumAcc * kHalves;   // [kSchedRing] entry j holds a tile id
    const ts_u32 sched_empty    = sched_full + 8 * kSchedRing;    // [kSchedRing] every role of the pair has read it (leader CTA's)
    const ts_u32 clc_bar        = sched_empty + 8 * kSchedRing;   // the launch control's answer has landed
    const ts_u32 tmem_ptr_smem  = clc_bar + 8;                    // u32
    const ts_u32 clc_response   = (tmem_ptr_smem + 4 + 15u) & ~15u;   // 16 bytes
    const ts_u32 sched_ring     = clc_response + 16;              // [kSchedRing] u32
#else
    const ts_u32 tmem_ptr_smem  = tmem_empty_bar + 8 * kNumAcc * kHalves;   // u32
#endif

    const ts_u32 warp_id  = threadIdx.x >> 5;
    const ts_u32 lane     = threadIdx.x & 31u;
    const ts_u32 cta_rank = (TS_CTA_GROUP == 2) ? ts_cluster_ctarank() : 0u;
    const bool   is_leader = (cta_rank == 0);

#if TS_GROUPED
    const ts_u32 num_tiles = (ts_u32)total_tiles;
#else
    const ts_u32 num_m = ((ts_u32)M + kTileM - 1) / kTileM;
    const ts_u32 num_n = ((ts_u32)N + kBlockN - 1) / kBlockN;
    const ts_u32 num_tiles = num_m * num_n;
    const ts_u32 num_k_blocks = ((ts_u32)K + kBlockK - 1) / kBlockK;
    // the one problem of an ordinary launch, in the form the tile loops read
    TileInfo ti;
    ti.num_m = num_m; ti.num_n = num_n; ti.num_k_blocks = num_k_blocks; ti.group_m = (ts_u32)group_m;
    ti.M = M; ti.N = N; ti.a = &tmap_a; ti.b = &tmap_b; ti.bias = bias;
#if TS_SCATTER
    ti.c = &tmap_cs.m[0];
#else
    ti.c = &tmap_c;
#endif
#endif
    const ts_u32 first_tile = (TS_CTA_GROUP == 2) ? ts_cluster_id_x() : blockIdx.x;
    const ts_u32 tile_step  = (TS_CTA_GROUP == 2) ? ts_nclusters_x() : gridDim.x;

    if (warp_id == 0 && lane == 0) {
#if !TS_GROUPED
        ts_prefetch_tmap(&tmap_a);
        ts_prefetch_tmap(&tmap_b);
#if TS_SCATTER
        for (int g = 0; g * rows_per_owner < M && g < 8; ++g) ts_prefetch_tmap(&tmap_cs.m[g]);
#else
        ts_prefetch_tmap(&tmap_c);
#endif
#endif
        for (ts_u32 s = 0; s < kStages; ++s) {
            ts_mbar_init(full_bar + 8 * s, 1);    // producer's arrive.expect_tx (leader CTA)
            ts_mbar_init(empty_bar + 8 * s, 1);   // one tcgen05.commit
        }
        for (ts_u32 b = 0; b < kNumAcc; ++b) ts_mbar_init(tmem_full_bar + 8 * b, 1);          // one tcgen05.commit
        for (ts_u32 b = 0; b < kNumAcc * kHalves; ++b)
            ts_mbar_init(tmem_empty_bar + 8 * b, kNumEpiWarps * TS_CTA_GROUP);               // one arrive per epilogue warp
#if TS_CLC
        for (ts_u32 j = 0; j < kSchedRing; ++j) {
            ts_mbar_init(sched_full + 8 * j, 1);                 // the scheduler's arrive (one per CTA, on that CTA's barrier)
            ts_mbar_init(sched_empty + 8 * j, kSchedReaders);    // every reader of the pair, on the leader's barrier
        }
        ts_mbar_init(clc_bar, 1);
#endif
        ts_fence_mbar_init();
    }
    if (TS_CTA_GROUP == 2) ts_cluster_sync();   // both CTAs of the pair are running before TMEM is split
    if (warp_id == 1) {
        ts_tmem_alloc<TS_CTA_GROUP>(tmem_ptr_smem, kTmemCols);
        ts_tmem_relinquish<TS_CTA_GROUP>();
    }
    ts_tc_fence_before();
    if (TS_CTA_GROUP == 2) ts_cluster_sync(); else __syncthreads();
    ts_tc_fence_after();
    ts_u32 tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_ptr_smem) : "memory");

#if TS_CLC
    // The next tile of this cluster for a role that has walked `taken` tiles (its own first tile, then ring entries
    // 0, 1, ...).  Every calling lane reads the entry; `releaser` (one lane per role instance) hands it back once the
    // lanes that called together have read it (`warp_wide`: the whole warp calls).
    const ts_u32 leader_sched_empty = ts_mapa(sched_empty, 0);
    auto clc_next = [&](ts_u32& taken, bool& ok, bool releaser, bool warp_wide) -> ts_u32 {
        const ts_u32 j = taken++, slot = j % kSchedRing;
        if (!ts_mbar_wait_cluster(sched_full + 8 * slot, (j / kSchedRing) & 1u)) {
            if (releaser) atomicOr(status, TS_ERR_TIMEOUT_SCHED);
            ok = false;
            return kNoTile;
        }
        ts_u32 t;
        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(t) : "r"(sched_ring + 4 * slot) : "memory");
        if (warp_wide) __syncwarp();
        if (releaser) ts_mbar_arrive_release_cluster(leader_sched_empty + 8 * slot);
        return t;
    };
#endif

    if (warp_id == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // In a pair, every byte count is signalled on the leader CTA's full barrier.
            ts_u32 it = 0;
            bool ok = true;
#if TS_GROUPED
            ts_u32 cursor = 0;
#endif
#if TS_CLC
            ts_u32 taken = 0;
            for (ts_u32 t = first_tile; t < num_tiles && ok; t = clc_next(taken, ok, true, false)) {
#else
            for (ts_u32 t = first_tile; t < num_tiles && ok; t += tile_step) {
#endif
#if TS_GROUPED
                const TileInfo ti = tile_info(probs, t, cursor);
                const ts_u32 lt = ti.local_tile;
#else
                const ts_u32 lt = t;
#endif
                ts_u32 m_blk, n_blk;
                ts_decode_tile(lt, ti.num_m, ti.num_n, ti.group_m, m_blk, n_blk);
#if TS_SCATTER
                m_blk = (m_blk + (ts_u32)m_rotate) % num_m;
#endif
                const int a_row = (int)(m_blk * kTileM + cta_rank * kBlockM);
                const int b_row = (int)(n_blk * kBlockN + cta_rank * kHalfRows);    // + h * kMmaN for MMA group h
                for (ts_u32 kb = 0; kb < ti.num_k_blocks; ++kb, ++it) {
                    const ts_u32 s = it % kStages;
                    const ts_u32 ph = (it / kStages) & 1u;
                    if (!ts_mbar_wait(empty_bar + 8 * s, ph ^ 1u)) {
                        atomicOr(status, TS_ERR_TIMEOUT_EMPTY); ok = false; break;
                    }
                    const int kc = (int)(kb * kBlockK);
                    if (TS_CTA_GROUP == 1) {
                        ts_mbar_arrive_expect_tx(full_bar + 8 * s, kStageBytes);
                        ts_tma_load_2d(smem_a + s * kSmemA, ti.a, full_bar + 8 * s, kc, a_row);
                        ts_tma_load_2d(smem_b + s * kSmemB, ti.b, full_bar + 8 * s, kc, b_row);     // (one MMA group: kHalves is 1)
                    } else {
                        const ts_u32 leader_full = ts_mapa(full_bar + 8 * s, 0);
                        if (is_leader) ts_mbar_arrive_expect_tx(full_bar + 8 * s, kStageBytes * 2);
                        ts_tma_load_2d_pair(smem_a + s * kSmemA, ti.a, leader_full, kc, a_row);
#pragma unroll
                        for (ts_u32 h = 0; h < kHalves; ++h)      // this CTA's rows of B for each MMA group, one after the other
                            ts_tma_load_2d_pair(smem_b + s * kSmemB + h * kHalfRows * kBlockKBytes, ti.b, leader_full, kc,
                                                b_row + (int)(h * kMmaN));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp_id == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp walks the loop (and waits on the barriers); one elected lane issues.
        if (is_leader) {
            constexpr ts_u32 idesc = ts_idesc_dense(TS_AB_FMT, TS_AB_FMT, kTileM, kMmaN, TS_MMA_KIND == TS_KIND_I8 ? 2u : 1u);
            const bool elected = ts_elect_one();
            ts_u32 it = 0, tile_iter = 0;
            bool ok = true;
#if TS_GROUPED
            ts_u32 cursor = 0;
#endif
#if TS_CLC
            ts_u32 taken = 0;
            for (ts_u32 t = first_tile; t < num_tiles && ok; t = clc_next(taken, ok, elected, true), ++tile_iter) {
#else
            for (ts_u32 t = first_tile; t < num_tiles && ok; t += tile_step, ++tile_iter) {
#endif
#if TS_GROUPED
                const TileInfo ti = tile_info(probs, t, cursor);
#endif
                const ts_u32 acc = tile_iter % kNumAcc;
                const ts_u32 acc_ph = (tile_iter / kNumAcc) & 1u;
                const ts_u32 d_tmem = tmem_base + acc * kBlockN;
                // The MMAs of column group h for the K block in stage s (one elected lane issues).
                auto issue_group = [&](ts_u32 h, ts_u32 s, ts_u32 kb) {
                    const ts_u64 a_desc = ts_smem_desc_kmajor<TS_SWIZZLE_B>(smem_a + s * kSmemA);
                    const ts_u64 b_desc = ts_smem_desc_kmajor<TS_SWIZZLE_B>(smem_b + s * kSmemB + h * kHalfRows * kBlockKBytes);
                    if (elected) {
#pragma unroll
                        for (ts_u32 k = 0; k < kNumUmma; ++k) {
                            // +32 bytes along K inside the swizzle row = +2 in the address field
                            ts_umma<TS_CTA_GROUP, TS_MMA_KIND>(d_tmem + h * kMmaN, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0u);
                        }
                    }
                };
                // frees the smem stage (in both CTAs of a pair) once the MMAs issued so far have read it
                auto free_stage = [&](ts_u32 s) {
                    if (elected) {
                        if (TS_CTA_GROUP == 1) ts_umma_commit<1>(empty_bar + 8 * s);
                        else                   ts_umma_commit_pair(empty_bar + 8 * s, 3);
                    }
                };
                // The epilogue hands the accumulator back one column group at a time; each group is waited for in
                // front of its first MMA.
                auto wait_group = [&](ts_u32 h) -> bool {
                    if (!ts_mbar_wait(tmem_empty_bar + 8 * (acc * kHalves + h), acc_ph ^ 1u)) {
                        if (elected) atomicOr(status, TS_ERR_TIMEOUT_TMEM_EMPTY);
                        return false;
                    }
                    ts_tc_fence_after();
                    return true;
                };
                auto wait_stage = [&](ts_u32 i) -> bool {
                    if (!ts_mbar_wait(full_bar + 8 * (i % kStages), (i / kStages) & 1u)) {
                        if (elected) atomicOr(status, TS_ERR_TIMEOUT_FULL);
                        return false;
                    }
                    ts_tc_fence_after();
                    return true;
                };
                // With two column groups and one accumulator, the tile starts with group 0 alone for as many K blocks as
                // the ring holds (their stages stay held), then group 1 for the same blocks: the epilogue of the tile
                // before has that long to hand group 1 back after group 0.
                ts_u32 head = 0;
                if (kHalves == 2) {
                    head = ti.num_k_blocks < kStages ? ti.num_k_blocks : kStages;
                    ok = wait_group(0);
                    for (ts_u32 kb = 0; kb < head && ok; ++kb) {
                        ok = wait_stage(it + kb);
                        if (ok) issue_group(0, (it + kb) % kStages, kb);
                        __syncwarp();
                    }
                    if (ok) ok = wait_group(1);
                    for (ts_u32 kb = 0; kb < head && ok; ++kb) {
                        issue_group(1, (it + kb) % kStages, kb);
                        free_stage((it + kb) % kStages);
                        __syncwarp();
                    }
                    if (!ok) break;
                    it += head;
                }
                for (ts_u32 kb = head; kb < ti.num_k_blocks; ++kb, ++it) {
                    const ts_u32 s = it % kStages;
                    if (!wait_stage(it)) { ok = false; break; }
                    if (kb == 0u && !wait_group(0)) { ok = false; break; }       // (only reached with one column group)
#pragma unroll
                    for (ts_u32 h = 0; h < kHalves; ++h) issue_group(h, s, kb);
                    free_stage(s);
                    __syncwarp();
                }
                if (!ok) break;
                if (elected) {
                    if (TS_CTA_GROUP == 1) ts_umma_commit<1>(tmem_full_bar + 8 * acc);
                    else                   ts_umma_commit_pair(tmem_full_bar + 8 * acc, 3);
                }
                __syncwarp();
            }
        }
        __syncwarp();
    } else if (warp_id < 2 + kNumEpiWarps) {
        // ------------------------------------------------------------ epilogue (warps 2..5)
        const ts_u32 quarter = warp_id & 3u;             // TMEM lanes this warp may read
        const ts_u32 store_smem = smem_c + (warp_id - 2) * kStoreBufs * kStoreBuf;
        const ts_u32 row_sw = (lane & 7u) << 4;          // 128-byte swizzle: 16-byte chunk ^= row % 8
        const ts_u32 leader_tmem_empty = (TS_CTA_GROUP == 2) ? ts_mapa(tmem_empty_bar, 0) : tmem_empty_bar;
        ts_u32 tile_iter = 0, chunk_iter = 0;
        bool ok = true;
#if TS_GROUPED
        ts_u32 cursor = 0;
#endif
#if TS_CLC
        ts_u32 taken = 0;
        for (ts_u32 t = first_tile; t < num_tiles && ok; t = clc_next(taken, ok, lane == 0, true), ++tile_iter) {
#else
        for (ts_u32 t = first_tile; t < num_tiles && ok; t += tile_step, ++tile_iter) {
#endif
#if TS_GROUPED
            const TileInfo ti = tile_info(probs, t, cursor);
            const ts_u32 lt = ti.local_tile;
#else
            const ts_u32 lt = t;
#endif
            const int M = ti.M, N = ti.N;                      // (shadow the launch arguments: per problem when grouped)
            const ts_u16* const bias = ti.bias;
            ts_u32 m_blk, n_blk;
            ts_decode_tile(lt, ti.num_m, ti.num_n, ti.group_m, m_blk, n_blk);
#if TS_SCATTER
            m_blk = (m_blk + (ts_u32)m_rotate) % num_m;
#endif
            const ts_u32 acc = tile_iter % kNumAcc;
            const ts_u32 acc_ph = (tile_iter / kNumAcc) & 1u;
            if (!ts_mbar_wait(tmem_full_bar + 8 * acc, acc_ph)) {
                if (lane == 0) atomicOr(status, TS_ERR_TIMEOUT_TMEM_FULL);
                ok = false; break;
            }
            ts_tc_fence_after();
            const int row0 = (int)(m_blk * kTileM + cta_rank * kBlockM + quarter * 32);
            const ts_u32 t_row = tmem_base + ((quarter * 32u) << 16) + acc * kBlockN;
            // (with two warps per lane quarter, warp `sub` takes chunks sub, sub + 2, ...: the first MMA group's chunks
            // come first for every warp, so that group goes back to the MMA issuer after half the drain)
            const ts_u32 sub = (warp_id - 2) / 4;
#pragma unroll 1
            for (ts_u32 j = sub; j < kNumChunks; j += kEpiSplit, ++chunk_iter) {
                const ts_u32 col0 = n_blk * kBlockN + j * kChunkCols;
                const ts_u32 buf = store_smem + (chunk_iter % kStoreBufs) * kStoreBuf;
                // the store that last read this staging buffer was issued kStoreBufs chunks ago
                if (lane == 0) ts_bulk_wait_read<kStoreBufs - 1>();
                __syncwarp();
                const ts_u32 row_addr = buf + lane * 128;
#if TS_OUT_F32
                ts_u32 v[32];
                ts_tmem_ld_32x32b_x32(t_row + j * kChunkCols, v);
                ts_tmem_wait_ld();
#pragma unroll
                for (ts_u32 c = 0; c < 8; ++c) {
                    float f[4];
#pragma unroll
                    for (ts_u32 i = 0; i < 4; ++i) f[i] = alpha * ts_acc_to_f32<TS_MMA_KIND>(v[4 * c + i]);
#if TS_HAS_BIAS
                    if (col0 + 4 * c < (ts_u32)N) {
                        const uint2 bb = __ldg(reinterpret_cast<const uint2*>(bias + col0 + 4 * c));
                        f[0] += ts_bf16_lo_to_f32(bb.x); f[1] += ts_bf16_hi_to_f32(bb.x);
                        f[2] += ts_bf16_lo_to_f32(bb.y); f[3] += ts_bf16_hi_to_f32(bb.y);
                    }
#endif
                    ts_st_shared_v4(row_addr + ((c << 4) ^ row_sw), __float_as_uint(f[0]), __float_as_uint(f[1]),
                                    __float_as_uint(f[2]), __float_as_uint(f[3]));
                }
#else
                ts_u32 v0[32], v1[32];
                ts_tmem_ld_32x32b_x32(t_row + j * kChunkCols, v0);
                ts_tmem_ld_32x32b_x32(t_row + j * kChunkCols + 32, v1);
                ts_tmem_wait_ld();
#pragma unroll
                for (ts_u32 c = 0; c < 8; ++c) {
                    float f[8];
#pragma unroll
                    for (ts_u32 i = 0; i < 8; ++i)
                        f[i] = alpha * ts_acc_to_f32<TS_MMA_KIND>(c < 4 ? v0[8 * c + i] : v1[8 * (c - 4) + i]);
#if TS_HAS_BIAS
                    if (col0 + 8 * c < (ts_u32)N) {
                        const uint4 bb = __ldg(reinterpret_cast<const uint4*>(bias + col0 + 8 * c));
                        f[0] += ts_bf16_lo_to_f32(bb.x); f[1] += ts_bf16_hi_to_f32(bb.x);
                        f[2] += ts_bf16_lo_to_f32(bb.y); f[3] += ts_bf16_hi_to_f32(bb.y);
                        f[4] += ts_bf16_lo_to_f32(bb.z); f[5] += ts_bf16_hi_to_f32(bb.z);
                        f[6] += ts_bf16_lo_to_f32(bb.w); f[7] += ts_bf16_hi_to_f32(bb.w);
                    }
#endif
                    ts_st_shared_v4(row_addr + ((c << 4) ^ row_sw),
                                    ts_pack_bf16x2(f[0], f[1]), ts_pack_bf16x2(f[2], f[3]),
                                    ts_pack_bf16x2(f[4], f[5]), ts_pack_bf16x2(f[6], f[7]));
                }
#endif
                ts_fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
#if TS_SCATTER
                    if (col0 < (ts_u32)N && row0 < M) {
                        const int owner = row0 / rows_per_owner;       // rows_per_owner is a multiple of 32
#if TS_SCATTER == 2
                        ts_tma_reduce_add_2d(&tmap_cs.m[owner], buf, (int)col0, row0 - owner * rows_per_owner);
#else
                        ts_tma_store_2d(&tmap_cs.m[owner], buf, (int)col0, row0 - owner * rows_per_owner);
#endif
                    }
#else
                    if (col0 < (ts_u32)N && row0 < M) ts_tma_store_2d(ti.c, buf, (int)col0, row0);
#endif
                    ts_bulk_commit();   // committed even when empty so that "one group pending" always means the previous chunk
                }
                if ((j + kEpiSplit) % (kNumChunks / kHalves) < kEpiSplit) {      // this warp's last chunk of an MMA group
                    // every column of one MMA group of this accumulator has been read: hand the group back to the MMA issuer
                    const ts_u32 grp = acc * kHalves + j / (kNumChunks / kHalves);
                    ts_tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (TS_CTA_GROUP == 2) ts_mbar_arrive_cluster(leader_tmem_empty + 8 * grp);
                        else                   ts_mbar_arrive(tmem_empty_bar + 8 * grp);
                    }
                }
            }
        }
        if (lane == 0) ts_bulk_wait_all();
        __syncwarp();
    }
#if TS_CLC
    else {
        // ------------------------------------------------------------ scheduler (the last warp, leader CTA, one lane)
        // Entry j of the ring: wait until every role of the pair has read what the entry held kSchedRing tiles ago,
        // ask the launch control for one more cluster's tile, and publish the answer (a tile id, or kNoTile once
        // nothing is left to cancel) to both CTAs: the id with a store to the CTA's shared memory, then an arrive
        // with release at cluster scope on that CTA's full barrier.
        if (is_leader && lane == 0) {
            for (ts_u32 j = 0;; ++j) {
                const ts_u32 slot = j % kSchedRing;
                if (!ts_mbar_wait_cluster(sched_empty + 8 * slot, ((j / kSchedRing) & 1u) ^ 1u)) {
                    atomicOr(status, TS_ERR_TIMEOUT_SCHED); break;
                }
                ts_mbar_arrive_expect_tx(clc_bar, 16);
                ts_clc_try_cancel(clc_response, clc_bar);
                if (!ts_mbar_wait(clc_bar, j & 1u)) { atomicOr(status, TS_ERR_TIMEOUT_SCHED); break; }
                ts_u32 first_cta_x;
                const bool got = ts_clc_query(clc_response, first_cta_x);
                const ts_u32 t = got ? first_cta_x / TS_CTA_GROUP : kNoTile;
                for (ts_u32 r = 0; r < TS_CTA_GROUP; ++r) {
                    ts_st_shared_cluster_u32(ts_mapa(sched_ring + 4 * slot, r), t);
                    ts_mbar_arrive_release_cluster(ts_mapa(sched_full + 8 * slot, r));
                }
                if (!got) break;       // (after a refusal no further request may be made)
            }
        }
        __syncwarp();
    }
#endif

    // ---------------------------------------------------------------- teardown
    ts_tc_fence_before();
    if (TS_CTA_GROUP == 2) ts_cluster_sync(); else __syncthreads();
    if (warp_id == 1) {
        ts_tc_fence_after();
        ts_tmem_dealloc<TS_CTA_GROUP>(tmem_base, kTmemCols);
    }
}
