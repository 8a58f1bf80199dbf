// Block-scaled FP8 (E4M3) GEMM mainloop for sm_100a:
//   C[m,n] = alpha * sum_kb sA[m,kb] * sB[n/128,kb] * ( sum_{k in block kb} qA[m,k] * qB[n,k] )  (+ bias[n])
// qA: M x K and qB: N x K E4M3 bytes, K-contiguous; sA: fp32 [M][K/128] (one scale per row and
// 128-wide K block), sB: fp32 [ceil(N/128)][K/128] (one scale per 128x128 block); fp32
// accumulation; output bf16 or fp32.  The reference has no FP8 element or scale concept
// (lib/core/elemtype.ml:9-14); this kernel extends its Blackwell skeleton
// (lib/backend/backend_cute.ml:257-366) in the same idiom.
//
// fp32 block scales are not a format the tensor core applies itself (its block-scale kinds
// want one power-of-two scale per 32 elements), so each 128-wide K block is multiplied by the
// tensor core alone (tcgen05.mma kind::f8f6f4, fresh accumulator) into a TMEM buffer, and
// promotion warps read it back (tcgen05.ld), scale it by alpha*sA*sB and add it into fp32
// registers while the tensor core works on the following blocks.
//
// Structure (what bounds it: the 128 x BLOCK_N multiply-adds per K block are half of the tensor
// core's time for that block on the FP32 pipe, and every hand-off between the tensor core and
// the promotion warps sits on a dependent chain):
//  - TMEM is four buffers of 128 columns.  A 256-wide tile is two MMA chains per K block, one
//    per 128 columns, each with its own issuing warp (warps 1 and 2), its own buffers and its
//    own promotion warps, so a chain has two K-block times for multiply -> read back -> release.
//    (TS_FP8_SPLIT 0 keeps one chain of 256-wide MMAs and two buffers.)
//  - Warpgroup 0 = TMA producer, the issuing warps, idle warps; it hands its registers to the
//    promotion warps (setmaxnreg), which hold 128 accumulators and two 32-column load buffers:
//    the load of the next 32 columns is in flight while the current 32 are multiplied.
//  - The issuing warps run converged and elect one lane per instruction; scales come through a
//    register ring refilled two K blocks ahead (sA, one row per lane) and a per-lane copy of
//    32 K blocks handed out by shuffle (sB); a buffer is released as soon as its last load
//    has landed; the epilogue fills all staging buffers of the warp before one fence and commit.
//
//  - Stream-K tail.  The host may name the last `num_tiles - full_tiles` tiles of the raster order as tail tiles
//    and split each into `tail_splits` ranges of K blocks; every (tile, range) is then a unit of work of its own,
//    dealt to the CTAs like a whole tile.  A tail unit adds its fp32 partial into a workspace tile with TMA
//    reduce-adds (no bias, no cast); the small kernel at the end of this file adds the bias, casts into C and
//    clears the workspace.  With a tile count a little over a whole number of waves this replaces a last wave
//    of a few tiles, one whole K loop long, by a wave of K-range units a fraction as long.  The order of the
//    additions into the workspace is not fixed, so tail tiles are not bit-reproducible from run to run.
//    Compiled in only with TS_FP8_TAIL (the host's notes give the measurements: it breaks even at best).
//
// Compile-time configuration (macros): TS_KERNEL_NAME, TS_CTA_GROUP (1|2), TS_BLOCK_N (128|256),
// TS_STAGES, TS_PROMO_WARPS (8|16), TS_OUT_F32, TS_HAS_BIAS, TS_FP8_SPLIT, TS_FP8_TAIL (0|1: without it the unit logic
// of the stream-K tail folds away at compile time and every unit is a whole tile).
#pragma once

#ifndef TS_PROMO_WARPS
#define TS_PROMO_WARPS 8
#endif

namespace ts_fp8 {

constexpr ts_u32 kBlockM      = 128;
constexpr ts_u32 kTileM       = kBlockM * TS_CTA_GROUP;
constexpr ts_u32 kBlockN      = TS_BLOCK_N;
constexpr ts_u32 kLoadN       = kBlockN / TS_CTA_GROUP;
constexpr ts_u32 kBlockK      = 128;                          // one scale block = one 128-byte swizzle row
constexpr ts_u32 kNumUmma     = 4;                            // 4 MMAs of K=32 per stage
constexpr ts_u32 kStages      = TS_STAGES;
constexpr ts_u32 kSmemA       = kBlockM * 128;
constexpr ts_u32 kSmemB       = kLoadN * 128;
constexpr ts_u32 kStageBytes  = kSmemA + kSmemB;
#ifndef TS_FP8_SPLIT
#define TS_FP8_SPLIT 1
#endif
constexpr ts_u32 kBufCols     = TS_FP8_SPLIT ? 128 : kBlockN;  // columns of one TMEM partial-product buffer = N of one MMA
constexpr ts_u32 kHalves      = kBlockN / kBufCols;           // MMA groups per K block, each into its own buffer
constexpr ts_u32 kNumAcc      = 512 / kBufCols;               // TMEM partial-product buffers
constexpr ts_u32 kTmemCols    = 512;
constexpr ts_u32 kNumPromoWarps = TS_PROMO_WARPS;
constexpr ts_u32 kWarpCols    = kBlockN / (kNumPromoWarps / 4); // columns one promotion warp owns
constexpr ts_u32 kOutBytes    = TS_OUT_F32 ? 4 : 2;
constexpr ts_u32 kChunkCols   = 128 / kOutBytes;
constexpr ts_u32 kStoreBuf    = 32 * 128;
constexpr ts_u32 kWarpChunks  = kWarpCols / kChunkCols;       // store chunks per warp and tile
constexpr ts_u32 kStoreBufs   = kWarpChunks >= 2 ? 2 : 1;     // staging buffers per warp
constexpr ts_u32 kSmemC       = kNumPromoWarps * kStoreBufs * kStoreBuf;
constexpr ts_u32 kNumBars     = 2 * kStages + 2 * kNumAcc;
constexpr ts_u32 kSmemTotal   = kStages * kStageBytes + kSmemC + kNumBars * 8 + 16;
constexpr ts_u32 kFirstPromoWarp = 4;                          // warpgroup 0: producer, MMA issuer, two idle warps
constexpr ts_u32 kThreads     = 32 * (kFirstPromoWarp + kNumPromoWarps);
constexpr int    kRegsIssue   = kNumPromoWarps == 8 ? 40 : 32;  // register budgets after the split (per thread)
constexpr int    kRegsPromo   = kNumPromoWarps == 8 ? 232 : 112;
constexpr ts_u32 kLdCols      = kNumPromoWarps == 8 ? 32 : 16;  // TMEM columns per load of the promotion loop
#ifndef TS_SCALE_RING
#define TS_SCALE_RING 2
#endif
constexpr ts_u32 kScaleRing   = TS_SCALE_RING;                // K blocks of scale prefetch held in registers
constexpr ts_u32 kBufWarps    = 4 * kBufCols / kWarpCols;     // promotion warps that read one buffer
constexpr ts_u32 kBRows       = kLoadN / kHalves;             // B rows of one MMA group in this CTA's shared memory
static_assert(kNumPromoWarps == 8 || kNumPromoWarps == 16, "TS_PROMO_WARPS must be 8 or 16");

static_assert(kBlockN == 128 || kBlockN == 256, "TS_BLOCK_N must be 128 or 256 (whole 128x128 scale blocks)");
static_assert(kWarpCols % kChunkCols == 0 && kWarpCols % 32 == 0, "store chunk must divide a warp's column range");
static_assert(kSmemTotal + 1024 <= 232448, "shared memory over the 227 KB limit");

// One unit of work: a tile and a range of its K blocks.  `range` packs first block | blocks << 16 (K < 2^23);
// `ws_row` is the unit's first workspace row, or kNoTail for a whole tile.
#ifndef TS_FP8_TAIL
#define TS_FP8_TAIL 0
#endif
constexpr bool kTail = TS_FP8_TAIL != 0;
constexpr ts_u32 kNoTail = 0xffffffffu;
TS_DEV void unit_of(ts_u32 u, ts_u32 full_tiles, ts_u32 splits, ts_u32 num_k_blocks, ts_u32& tile, ts_u32& range, ts_u32& ws_row) {
    if (!kTail || u < full_tiles) { tile = u; range = num_k_blocks << 16; ws_row = kNoTail; return; }
    const ts_u32 v = u - full_tiles, ti = v / splits, part = v - ti * splits;
    const ts_u32 kb0 = part * num_k_blocks / splits;
    tile = full_tiles + ti;
    range = kb0 | (((part + 1) * num_k_blocks / splits - kb0) << 16);
    ws_row = ti * kTileM;
}
// The same for a role that only needs the unit's number of K blocks.
TS_DEV ts_u32 unit_blocks_of(ts_u32 u, ts_u32 full_tiles, ts_u32 splits, ts_u32 num_k_blocks) {
    if (!kTail || u < full_tiles) return num_k_blocks;
    const ts_u32 part = (u - full_tiles) % splits;
    return (part + 1) * num_k_blocks / splits - part * num_k_blocks / splits;
}

TS_DEV void ts_tmem_ld(ts_u32 taddr, ts_u32 (&r)[16]) { ts_tmem_ld_32x32b_x16(taddr, r); }
TS_DEV void ts_tmem_ld(ts_u32 taddr, ts_u32 (&r)[32]) { ts_tmem_ld_32x32b_x32(taddr, r); }

// A tail unit's epilogue: this warp's 32 rows x kWarpCols fp32 partial sums (one row per lane, handed over in local
// memory) go through the warp's staging buffers, 32 columns per 128-byte row, and are added into the workspace by TMA.
__device__ __noinline__ void tail_add(const float* part, ts_u32 store_smem, ts_u32 row_sw, ts_u32 lane,
                                      const TsTensorMap* tmap_ws, int col0, int ws_row0) {
    constexpr ts_u32 kTailChunks = kWarpCols / 32;
    static_assert(kTailChunks % kStoreBufs == 0, "the tail's chunks must fill whole rounds of staging buffers");
#pragma unroll 1
    for (ts_u32 g = 0; g < kTailChunks / kStoreBufs; ++g) {
        if (lane == 0) ts_bulk_wait_read<0>();       // the stores that last read the staging buffers
        __syncwarp();
#pragma unroll 1
        for (ts_u32 b = 0; b < kStoreBufs; ++b) {
            const float* src = part + (g * kStoreBufs + b) * 32;
            const ts_u32 row_addr = store_smem + b * kStoreBuf + lane * 128;
#pragma unroll
            for (ts_u32 c = 0; c < 8; ++c)
                ts_st_shared_v4(row_addr + ((c << 4) ^ row_sw), __float_as_uint(src[4 * c]), __float_as_uint(src[4 * c + 1]),
                                __float_as_uint(src[4 * c + 2]), __float_as_uint(src[4 * c + 3]));
        }
        ts_fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            for (ts_u32 b = 0; b < kStoreBufs; ++b)
                ts_tma_reduce_add_2d(tmap_ws, store_smem + b * kStoreBuf, col0 + (int)((g * kStoreBufs + b) * 32), ws_row0);
            ts_bulk_commit();
        }
        __syncwarp();
    }
}

}  // namespace ts_fp8

extern "C" __global__ void __launch_bounds__(128 + 32 * TS_PROMO_WARPS, 1)
TS_KERNEL_NAME(const __grid_constant__ TsTensorMap tmap_a,
               const __grid_constant__ TsTensorMap tmap_b,
               const __grid_constant__ TsTensorMap tmap_c,
               const __grid_constant__ TsTensorMap tmap_ws,   // fp32 [tail tiles * tile rows][BLOCK_N]: the tail units' sums
               const float* __restrict__ scale_a,      // [M][K/128]
               const float* __restrict__ scale_b,      // [ceil(N/128)][K/128]
               const ts_u16* __restrict__ bias,
               float alpha, int M, int N, int K, int group_m,
               int full_tiles_arg, int tail_splits_arg,  // tiles computed whole; K ranges per remaining (tail) tile
               ts_u32* __restrict__ status)
{
    using namespace ts_fp8;
    extern __shared__ ts_u8 ts_smem_raw[];
    const ts_u32 smem_base = (ts_smem_u32(ts_smem_raw) + 1023u) & ~1023u;
    const ts_u32 smem_a    = smem_base;
    const ts_u32 smem_b    = smem_a + kStages * kSmemA;
    const ts_u32 smem_c    = smem_b + kStages * kSmemB;
    const ts_u32 bar_base  = smem_c + kSmemC;
    const ts_u32 full_bar       = bar_base;
    const ts_u32 empty_bar      = full_bar + 8 * kStages;
    const ts_u32 tmem_full_bar  = empty_bar + 8 * kStages;
    const ts_u32 tmem_empty_bar = tmem_full_bar + 8 * kNumAcc;
    const ts_u32 tmem_ptr_smem  = tmem_empty_bar + 8 * kNumAcc;

    const ts_u32 warp_id  = threadIdx.x >> 5;
    const ts_u32 lane     = threadIdx.x & 31u;
    const ts_u32 cta_rank = (TS_CTA_GROUP == 2) ? ts_cluster_ctarank() : 0u;
    const bool   is_leader = (cta_rank == 0);

    const ts_u32 num_m = ((ts_u32)M + kTileM - 1) / kTileM;
    const ts_u32 num_n = ((ts_u32)N + kBlockN - 1) / kBlockN;
    const ts_u32 num_tiles = num_m * num_n;
    const ts_u32 num_k_blocks = ((ts_u32)K + kBlockK - 1) / kBlockK;
    // (the host passes full_tiles <= tiles and 1 <= tail_splits <= K blocks; used as they come, so that they can be
    // re-read from the parameter bank instead of being held in registers across the promotion loop)
    const ts_u32 full_tiles = kTail ? (ts_u32)full_tiles_arg : num_tiles;
    const ts_u32 splits = kTail ? (ts_u32)tail_splits_arg : 1u;
    const ts_u32 num_units = kTail ? full_tiles + (num_tiles - full_tiles) * splits : num_tiles;
    const ts_u32 first_tile = (TS_CTA_GROUP == 2) ? ts_cluster_id_x() : blockIdx.x;
    const ts_u32 tile_step  = (TS_CTA_GROUP == 2) ? ts_nclusters_x() : gridDim.x;

    if (warp_id == 0 && lane == 0) {
        ts_prefetch_tmap(&tmap_a);
        ts_prefetch_tmap(&tmap_b);
        ts_prefetch_tmap(&tmap_c);
        if (kTail && full_tiles < num_tiles) ts_prefetch_tmap(&tmap_ws);
        for (ts_u32 s = 0; s < kStages; ++s) {
            ts_mbar_init(full_bar + 8 * s, 1);
            ts_mbar_init(empty_bar + 8 * s, kHalves);          // one commit per issuing warp
        }
        for (ts_u32 b = 0; b < kNumAcc; ++b) {
            ts_mbar_init(tmem_full_bar + 8 * b, 1);
            ts_mbar_init(tmem_empty_bar + 8 * b, kBufWarps * TS_CTA_GROUP);
        }
        ts_fence_mbar_init();
    }
    if (TS_CTA_GROUP == 2) ts_cluster_sync();
    if (warp_id == 1) {
        ts_tmem_alloc<TS_CTA_GROUP>(tmem_ptr_smem, kTmemCols);
        ts_tmem_relinquish<TS_CTA_GROUP>();
    }
    ts_tc_fence_before();
    if (TS_CTA_GROUP == 2) ts_cluster_sync(); else __syncthreads();
    ts_tc_fence_after();
    ts_u32 tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_ptr_smem) : "memory");

    // The promotion warps keep a 128 x BLOCK_N fp32 tile in registers plus two load buffers; the other warpgroup
    // needs next to nothing.
    // (Each budget is set at the top of its own branch: the compiler follows it per path.)
    if (warp_id < kFirstPromoWarp) {
    ts_setmaxnreg_dec<kRegsIssue>();
    if (warp_id == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ts_u32 it = 0;
            bool ok = true;
            for (ts_u32 u = first_tile; u < num_units && ok; u += tile_step) {
                ts_u32 tile = u, kb_begin = 0, kb_end = num_k_blocks;
                if (kTail && u >= full_tiles) {
                    const ts_u32 v = u - full_tiles, ti = v / splits, part = v - ti * splits;
                    tile = full_tiles + ti;
                    kb_begin = part * num_k_blocks / splits;
                    kb_end = (part + 1) * num_k_blocks / splits;
                }
                ts_u32 m_blk, n_blk;
                ts_decode_tile(tile, num_m, num_n, (ts_u32)group_m, m_blk, n_blk);
                const int a_row = (int)(m_blk * kTileM + cta_rank * kBlockM);
                const int b_row = (int)(n_blk * kBlockN + cta_rank * kLoadN);
                for (ts_u32 kb = kb_begin; kb < kb_end; ++kb, ++it) {
                    const ts_u32 s = it % kStages;
                    const ts_u32 ph = (it / kStages) & 1u;
                    if (!ts_mbar_wait(empty_bar + 8 * s, ph ^ 1u)) {
                        atomicOr(status, TS_ERR_TIMEOUT_EMPTY); ok = false; break;
                    }
                    const int kc = (int)(kb * kBlockK);
                    if (TS_CTA_GROUP == 1) {
                        ts_mbar_arrive_expect_tx(full_bar + 8 * s, kStageBytes);
                        ts_tma_load_2d(smem_a + s * kSmemA, &tmap_a, full_bar + 8 * s, kc, a_row);
                        ts_tma_load_2d(smem_b + s * kSmemB, &tmap_b, full_bar + 8 * s, kc, b_row);
                    } else {
                        const ts_u32 leader_full = ts_mapa(full_bar + 8 * s, 0);
                        if (is_leader) ts_mbar_arrive_expect_tx(full_bar + 8 * s, kStageBytes * 2);
                        ts_tma_load_2d_pair(smem_a + s * kSmemA, &tmap_a, leader_full, kc, a_row);
                        // MMA group h multiplies columns 128h..128h+127 of the tile: this CTA holds its 64 rows
                        // of B for each group, one after the other
#pragma unroll
                        for (ts_u32 h = 0; h < kHalves; ++h)
                            ts_tma_load_2d_pair(smem_b + s * kSmemB + h * kBRows * 128, &tmap_b, leader_full, kc,
                                                (int)(n_blk * kBlockN + h * kBufCols + cta_rank * kBRows));
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp_id <= kHalves) {
        // ------------------------------------------------------------ MMA issuer
        // One issuing warp per 128-column group of the tile (warp 1, and warp 2 for a 256-wide tile): each group is
        // its own chain of MMAs into its own TMEM buffers, so its promotion warps start while the tensor core is on
        // the other group, and each issuer has a whole K-block time for its waits and commits.  The whole warp walks
        // the loop (and waits on the barriers); one elected lane issues.
        if (is_leader) {
            constexpr ts_u32 idesc = ts_idesc_dense(TS_FMT_E4M3, TS_FMT_E4M3, kTileM, kBufCols);
            const ts_u32 h = warp_id - 1u;
            const bool elected = ts_elect_one();
            ts_u32 it = 0;     // k-block counter across tiles: selects the smem stage and, with h, the TMEM buffer
            bool ok = true;
            for (ts_u32 u = first_tile; u < num_units && ok; u += tile_step) {
                const ts_u32 unit_blocks = unit_blocks_of(u, full_tiles, splits, num_k_blocks);
                for (ts_u32 kb = 0; kb < unit_blocks; ++kb, ++it) {
                    const ts_u32 s = it % kStages;
                    const ts_u32 ph = (it / kStages) & 1u;
                    const ts_u32 unit = it * kHalves + h;
                    const ts_u32 acc = unit % kNumAcc;
                    const ts_u32 acc_ph = (unit / kNumAcc) & 1u;
                    if (!ts_mbar_wait(tmem_empty_bar + 8 * acc, acc_ph ^ 1u)) {
                        if (elected) atomicOr(status, TS_ERR_TIMEOUT_TMEM_EMPTY);
                        ok = false; break;
                    }
                    if (!ts_mbar_wait(full_bar + 8 * s, ph)) {
                        if (elected) atomicOr(status, TS_ERR_TIMEOUT_FULL);
                        ok = false; break;
                    }
                    ts_tc_fence_after();
                    const ts_u32 d_tmem = tmem_base + acc * kBufCols;
                    const ts_u64 a_desc = ts_smem_desc_sw128(smem_a + s * kSmemA);
                    const ts_u64 b_desc = ts_smem_desc_sw128(smem_b + s * kSmemB + h * kBRows * 128);
                    if (elected) {
#pragma unroll
                        for (ts_u32 k = 0; k < kNumUmma; ++k)
                            ts_umma<TS_CTA_GROUP, TS_KIND_F8F6F4>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, k != 0u);
                        // the partial product is complete; the smem stage is free once every issuer's MMAs have read it
                        if (TS_CTA_GROUP == 1) {
                            ts_umma_commit<1>(tmem_full_bar + 8 * acc);
                            ts_umma_commit<1>(empty_bar + 8 * s);
                        } else {
                            ts_umma_commit_pair(tmem_full_bar + 8 * acc, 3);
                            ts_umma_commit_pair(empty_bar + 8 * s, 3);
                        }
                    }
                    __syncwarp();
                }
            }
        }
        __syncwarp();
    }
    } else {
        // ------------------------------------------------------------ promotion + epilogue (warps 4..)
        ts_setmaxnreg_inc<kRegsPromo>();
        const ts_u32 quarter = warp_id & 3u;
        const ts_u32 half = (warp_id - kFirstPromoWarp) >> 2;                 // which kWarpCols-wide column group
        const ts_u32 store_smem = smem_c + (warp_id - kFirstPromoWarp) * kStoreBufs * kStoreBuf;
        const ts_u32 row_sw = (lane & 7u) << 4;
        const ts_u32 leader_tmem_empty = (TS_CTA_GROUP == 2) ? ts_mapa(tmem_empty_bar, 0) : tmem_empty_bar;
        const ts_u32 nkb_all = num_k_blocks;
        const ts_u32 n_scale_rows = ((ts_u32)N + 127u) / 128u;
        ts_u32 it = 0;
        bool ok = true;
        // Scales of the next kScaleRing K blocks sit in a register ring that is refilled that far ahead and is only
        // multiplied when its block comes up: a load whose result is used at once stalls this warp for a trip to
        // L2, which is longer than a promotion.  sB is the same for the whole warp: lane l keeps the scale of K
        // block 32*g + l, handed out by shuffle.  The ring of a tile is loaded before the epilogue of the tile
        // before it, so that the first promotion of a tile does not wait for it either.
        const float* sa_ptr;
        const float* sb_ptr;
        float sa_r[kScaleRing];
        float sb_l;
        // (kb0, nkb: the unit's range of K blocks; the pointers are moved to its first block)
        auto scales_of_tile = [&](ts_u32 mb, ts_u32 nb, ts_u32 kb0, ts_u32 nkb) __attribute__((always_inline)) {
            const ts_u32 r = mb * kTileM + cta_rank * kBlockM + quarter * 32 + lane;
            ts_u32 sb_row = (nb * kBlockN + half * kWarpCols) / 128u;
            if (sb_row >= n_scale_rows) sb_row = n_scale_rows - 1;
            sa_ptr = scale_a + (size_t)(r < (ts_u32)M ? r : 0u) * nkb_all + kb0;
            sb_ptr = scale_b + (size_t)sb_row * nkb_all + kb0;
            // (predicated loads, not selects: a select on the loaded value would wait for it here)
#pragma unroll
            for (ts_u32 j = 0; j < kScaleRing; ++j) { sa_r[j] = 0.f; if (j < nkb) sa_r[j] = __ldg(sa_ptr + j); }
            sb_l = 0.f;
            if (lane < nkb) sb_l = __ldg(sb_ptr + lane);
        };
        // Tile coordinates are decoded once per tile, one tile ahead (three integer divisions each: at the top of a
        // tile they run behind the first wait, at its end they would sit in front of the next tile's first load).
        ts_u32 m_blk = 0, n_blk = 0;
        const bool fast_decode = num_tiles < (1u << 22);
        const float inv_group = 1.0f / (float)((ts_u32)group_m * num_n), inv_gm = 1.0f / (float)group_m;
        ts_u32 un_range = 0;
        if (first_tile < num_units) {
            ts_u32 tile, ws_unused;
            unit_of(first_tile, full_tiles, splits, num_k_blocks, tile, un_range, ws_unused);
            ts_decode_tile(tile, num_m, num_n, (ts_u32)group_m, m_blk, n_blk);
            scales_of_tile(m_blk, n_blk, un_range & 0xffffu, un_range >> 16);
        }
        for (ts_u32 u = first_tile; u < num_units && ok; u += tile_step) {
            const bool has_next = u + tile_step < num_units;
            ts_u32 m_next = 0, n_next = 0;
            if (has_next) {
                // (the tile index of the next unit is one compare for a whole tile and a division for a tail unit; its
                // range of K blocks is worked out after this unit's K loop, so that nothing more stays live across it)
                const ts_u32 un = u + tile_step;
                const ts_u32 tile = (!kTail || un < full_tiles) ? un : full_tiles + (un - full_tiles) / splits;
                if (fast_decode) ts_decode_tile_fast(tile, num_m, num_n, (ts_u32)group_m, inv_group, inv_gm, m_next, n_next);
                else             ts_decode_tile(tile, num_m, num_n, (ts_u32)group_m, m_next, n_next);
            }
            const ts_u32 nkb = kTail ? un_range >> 16 : nkb_all;
            const ts_u32 col_base = n_blk * kBlockN + half * kWarpCols;
            // 128 x BLOCK_N fp32 accumulators of the tile, one row per lane, held as packed pairs: the multiply-adds
            // are issued two at a time (fma.rn.f32x2: the same two roundings as two scalar fmas, half the issue slots).
            ts_u64 acc2[kWarpCols / 2];
#pragma unroll
            for (ts_u32 i = 0; i < kWarpCols / 2; ++i) acc2[i] = 0ull;
            constexpr ts_u32 kRounds = kWarpCols / kLdCols;
            static_assert(kRounds % 2 == 0, "the two load buffers alternate per round and must line up across K blocks");
            const ts_u32 grp = (half * kWarpCols) / kBufCols;                      // the MMA group this warp reads
            const ts_u32 col_in_buf = (half * kWarpCols) % kBufCols;
            ts_u32 p0[kLdCols], p1[kLdCols];      // two TMEM load buffers, used in turn
            // First load of the tile: columns 0..kLdCols-1 of the first K block's partial product.
            {
                const ts_u32 unit = it * kHalves + grp;
                const ts_u32 buf = unit % kNumAcc;
                if (!ts_mbar_wait(tmem_full_bar + 8 * buf, (unit / kNumAcc) & 1u)) {
                    if (lane == 0) atomicOr(status, TS_ERR_TIMEOUT_TMEM_FULL);
                    ok = false;
                }
                if (ok) {
                    ts_tc_fence_after();
                    ts_tmem_ld(tmem_base + ((quarter * 32u) << 16) + buf * kBufCols + col_in_buf, p0);
                }
            }
#pragma unroll 1
            for (ts_u32 kb0 = 0; kb0 < nkb && ok; kb0 += kScaleRing) {
#pragma unroll
            for (ts_u32 j = 0; j < kScaleRing; ++j) {
                const ts_u32 kb = kb0 + j;
                if (kb >= nkb || !ok) continue;
                if ((kb & 31u) == 0u && kb != 0u && kb + lane < nkb) sb_l = __ldg(sb_ptr + kb + lane);
                const float s = alpha * sa_r[j] * __shfl_sync(0xffffffffu, sb_l, (int)(kb & 31u));
                if (kb + kScaleRing < nkb) sa_r[j] = __ldg(sa_ptr + kb + kScaleRing);
                const ts_u64 s2 = ts_pack_f32x2(__float_as_uint(s), __float_as_uint(s));
                const ts_u32 unit = it * kHalves + grp;
                const ts_u32 buf = unit % kNumAcc;
                const ts_u32 t_row = tmem_base + ((quarter * 32u) << 16) + buf * kBufCols + col_in_buf;
                // kLdCols columns at a time, two register buffers: the load of the next group is in flight while the
                // multiply-adds of the current one issue.  The buffer goes back to the tensor core as soon as its last
                // load has landed; the first load of the NEXT K block is then issued in front of this block's last
                // multiply-adds, so that no K block starts with an exposed trip to tensor memory.
#pragma unroll
                for (ts_u32 c = 0; c < kRounds; ++c) {
                    ts_tmem_wait_ld();
                    if (c + 1 < kRounds) {
                        if (c & 1u) ts_tmem_ld(t_row + (c + 1) * kLdCols, p0); else ts_tmem_ld(t_row + (c + 1) * kLdCols, p1);
                    } else {
                        ts_tc_fence_before();
                        __syncwarp();
                        if (lane == 0) {
                            if (TS_CTA_GROUP == 2) ts_mbar_arrive_cluster(leader_tmem_empty + 8 * buf);
                            else                   ts_mbar_arrive(tmem_empty_bar + 8 * buf);
                        }
                        if (kb + 1 < nkb) {
                            const ts_u32 unit_n = (it + 1) * kHalves + grp;
                            const ts_u32 buf_n = unit_n % kNumAcc;
                            if (!ts_mbar_wait(tmem_full_bar + 8 * buf_n, (unit_n / kNumAcc) & 1u)) {
                                if (lane == 0) atomicOr(status, TS_ERR_TIMEOUT_TMEM_FULL);
                                ok = false;
                            }
                            if (ok) {
                                ts_tc_fence_after();
                                ts_tmem_ld(tmem_base + ((quarter * 32u) << 16) + buf_n * kBufCols + col_in_buf, p0);
                            }
                        }
                    }
#pragma unroll
                    for (ts_u32 i = 0; i < kLdCols / 2; ++i) {
                        const ts_u64 pp = (c & 1u) ? ts_pack_f32x2(p1[2 * i], p1[2 * i + 1]) : ts_pack_f32x2(p0[2 * i], p0[2 * i + 1]);
                        acc2[(c * kLdCols) / 2 + i] = ts_fma_f32x2(pp, s2, acc2[(c * kLdCols) / 2 + i]);
                    }
                }
                ++it;
            }
            }
            ts_tmem_wait_ld();      // (nothing is outstanding on the healthy path; after a timed-out wait there may be)
            float acc[kWarpCols];
#pragma unroll
            for (ts_u32 i = 0; i < kWarpCols / 2; ++i) ts_unpack_f32x2(acc2[i], acc[2 * i], acc[2 * i + 1]);
            if (!ok) break;
            // The next tile's first scales: ask for the lines now (no register is tied up while the accumulators
            // are still live), load them after the epilogue.
            ts_u32 next_range = 0, next_ws = kNoTail;
            if (has_next) {
                ts_u32 tile;
                unit_of(u + tile_step, full_tiles, splits, num_k_blocks, tile, next_range, next_ws);
                scales_of_tile(m_next, n_next, next_range & 0xffffu, next_range >> 16);
            }
            // ---- epilogue from registers (alpha is already in the scales): bias, cast, swizzled staging, TMA
            // store.  The warp fills all its staging buffers, then one fence and one commit cover their stores.
            // (a tail unit's workspace row is worked out here, from the unit index, rather than carried across the K loop)
            const ts_u32 un_ws = (kTail && u >= full_tiles) ? ((u - full_tiles) / splits) * kTileM : kNoTail;
            if (kTail && un_ws != kNoTail) {
                // ---- tail unit: the fp32 partial of this range of K blocks is added into the tile's workspace rows;
                // bias and cast wait for the kernel that closes the tail.  The accumulators are handed over through
                // local memory to a function that is not inlined: with this second epilogue inline the compiler
                // allocates the promotion loop's registers differently and every tile is a tenth slower (measured).
                float part[kWarpCols];
#pragma unroll
                for (ts_u32 i = 0; i < kWarpCols; ++i) part[i] = acc[i];
                tail_add(part, store_smem, row_sw, lane, &tmap_ws, (int)(half * kWarpCols),
                         (int)(un_ws + cta_rank * kBlockM + quarter * 32));
                m_blk = m_next; n_blk = n_next; un_range = next_range;
                continue;
            }
            const int row0 = (int)(m_blk * kTileM + cta_rank * kBlockM + quarter * 32);
#pragma unroll
            for (ts_u32 g = 0; g < kWarpChunks / kStoreBufs; ++g) {
                if (lane == 0) ts_bulk_wait_read<0>();       // the stores that last read the staging buffers
                __syncwarp();
#pragma unroll
                for (ts_u32 b = 0; b < kStoreBufs; ++b) {
                    const ts_u32 j = g * kStoreBufs + b;
                    const ts_u32 col0 = col_base + j * kChunkCols;
                    const ts_u32 row_addr = store_smem + b * kStoreBuf + lane * 128;
#pragma unroll
                    for (ts_u32 c = 0; c < 8; ++c) {
#if TS_OUT_F32
                        float f[4];
#pragma unroll
                        for (ts_u32 i = 0; i < 4; ++i) f[i] = acc[j * kChunkCols + 4 * c + i];
#if TS_HAS_BIAS
                        if (col0 + 4 * c < (ts_u32)N) {
                            const uint2 bb = __ldg(reinterpret_cast<const uint2*>(bias + col0 + 4 * c));
                            f[0] += ts_bf16_lo_to_f32(bb.x); f[1] += ts_bf16_hi_to_f32(bb.x);
                            f[2] += ts_bf16_lo_to_f32(bb.y); f[3] += ts_bf16_hi_to_f32(bb.y);
                        }
#endif
                        ts_st_shared_v4(row_addr + ((c << 4) ^ row_sw), __float_as_uint(f[0]), __float_as_uint(f[1]),
                                        __float_as_uint(f[2]), __float_as_uint(f[3]));
#else
                        float f[8];
#pragma unroll
                        for (ts_u32 i = 0; i < 8; ++i) f[i] = acc[j * kChunkCols + 8 * c + i];
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
#endif
                    }
                }
                ts_fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
#pragma unroll
                    for (ts_u32 b = 0; b < kStoreBufs; ++b) {
                        const ts_u32 col0 = col_base + (g * kStoreBufs + b) * kChunkCols;
                        if (col0 < (ts_u32)N && row0 < M) ts_tma_store_2d(&tmap_c, store_smem + b * kStoreBuf, (int)col0, row0);
                    }
                    ts_bulk_commit();
                }
            }
            m_blk = m_next; n_blk = n_next; un_range = next_range;
        }
        if (lane == 0) ts_bulk_wait_all();
        __syncwarp();
    }

    // ---------------------------------------------------------------- teardown
    ts_tc_fence_before();
    if (TS_CTA_GROUP == 2) ts_cluster_sync(); else __syncthreads();
    if (warp_id == 1) {
        ts_tc_fence_after();
        ts_tmem_dealloc<TS_CTA_GROUP>(tmem_base, kTmemCols);
    }
}

// Closes the stream-K tail: C = cast(workspace + bias) for the tail tiles, and the workspace is cleared for the next
// call.  Grid (tail tiles, kTailBlocksY): a block takes tile rows / kTailBlocksY rows of one tail tile, 256 threads,
// four columns per thread and step -- one or two steps per thread, so that the pass is a single round trip to L2
// and not a chain of them.
#define TS_CAT2(a, b) a##b
#define TS_CAT(a, b) TS_CAT2(a, b)
extern "C" __global__ void __launch_bounds__(256)
TS_CAT(TS_KERNEL_NAME, _tail)(float* __restrict__ ws, void* __restrict__ c_out, const ts_u16* __restrict__ bias,
                              int M, int N, long long ldc, int group_m, int full_tiles)
{
    using namespace ts_fp8;
    const ts_u32 num_m = ((ts_u32)M + kTileM - 1) / kTileM;
    const ts_u32 num_n = ((ts_u32)N + kBlockN - 1) / kBlockN;
    ts_u32 m_blk, n_blk;
    ts_decode_tile((ts_u32)full_tiles + blockIdx.x, num_m, num_n, (ts_u32)group_m, m_blk, n_blk);
    constexpr ts_u32 kVecPerRow = kBlockN / 4;
    const ts_u32 rows_per_block = kTileM / gridDim.y;
    float4* wt = reinterpret_cast<float4*>(ws + (size_t)blockIdx.x * kTileM * kBlockN);
    for (ts_u32 i = threadIdx.x; i < rows_per_block * kVecPerRow; i += blockDim.x) {
        const ts_u32 r = blockIdx.y * rows_per_block + i / kVecPerRow, cv = i % kVecPerRow;
        const size_t wi = (size_t)r * kVecPerRow + cv;
        float4 v = wt[wi];
        wt[wi] = make_float4(0.f, 0.f, 0.f, 0.f);
        const ts_u32 row = m_blk * kTileM + r, col = n_blk * kBlockN + 4 * cv;
        if (row >= (ts_u32)M || col >= (ts_u32)N) continue;
#if TS_HAS_BIAS
        const uint2 bb = __ldg(reinterpret_cast<const uint2*>(bias + col));
        v.x += ts_bf16_lo_to_f32(bb.x); v.y += ts_bf16_hi_to_f32(bb.x);
        v.z += ts_bf16_lo_to_f32(bb.y); v.w += ts_bf16_hi_to_f32(bb.y);
#endif
#if TS_OUT_F32
        *reinterpret_cast<float4*>(static_cast<float*>(c_out) + (size_t)row * ldc + col) = v;
#else
        *reinterpret_cast<uint2*>(static_cast<ts_u16*>(c_out) + (size_t)row * ldc + col) =
            make_uint2(ts_pack_bf16x2(v.x, v.y), ts_pack_bf16x2(v.z, v.w));
#endif
    }
}
