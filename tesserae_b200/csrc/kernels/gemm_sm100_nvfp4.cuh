// NVFP4 GEMM mainloop for sm_100a:
//   C[m,n] = alpha * sum_k (qA[m,k] * sfA[m,k/16]) * (qB[n,k] * sfB[n,k/16])  (+ bias[n])
// qA: M x K and qB: N x K E2M1 values, two per byte along K (even k in the low nibble),
// K-contiguous; sfA / sfB: one UE4M3 scale per row and 16 consecutive K elements; the two
// per-tensor fp32 scales are folded into alpha by the host.  fp32 accumulation in tensor
// memory, output bf16 or fp32.  The reference has no 4-bit element or scale concept
// (lib/core/elemtype.ml:9-14); this kernel extends its Blackwell skeleton
// (lib/backend/backend_cute.ml:257-366) in the same idiom.
//
// The tensor core applies the scales itself (tcgen05.mma kind::mxf4nvf4.block_scale,
// scale_vec::4X: K = 64 per instruction, four scales per row).  It reads them from tensor
// memory, where row r of a 128-row block sits in lane r % 32 (replicated to the four 32-lane
// quarters), 32-bit column r / 32, byte j for the j-th scale of the instruction.  The scale
// arrays are therefore stored in global memory already in that order, as 512-byte chunks
//   chunk(rb, kg)[ (r % 32) * 16 + (r / 32) * 4 + j ] = scale(row 128*rb + r, K block 4*kg + j)
// laid out [row block rb][K group kg], so that one stage (K = 256 = 4 chunks) of one row block
// is 2 KB contiguous and TMA brings it to shared memory as it is.
//
// Shared memory -> tensor memory: four scale warps, one per 32-lane quarter, read their
// 16 bytes per chunk from shared memory and write them with tcgen05.st.  (tcgen05.cp from
// the MMA-issuing thread does the same copy, but it runs in the tensor pipe in front of the
// MMAs: twelve copies per stage cost about half the MMA time of the stage.)  The scales of
// stage s live in TMEM scale region s, so the region is free exactly when the smem stage is.
//
// Warp layout (448 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2..9 epilogue
// (warp w reads TMEM lanes 32*(w%4).. and the column half (w-2)/4), warps 10..13 scale warps.
// With a 256-wide tile the accumulator has a single TMEM buffer (256 columns + the scale
// regions fill tensor memory): the epilogue drains it in two passes of 64 columns per warp and
// hands it back to the MMA issuer as soon as the second pass is in registers.
//
// Compile-time configuration (macros): TS_KERNEL_NAME, TS_CTA_GROUP (1|2), TS_BLOCK_N (128|256),
// TS_STAGES, TS_OUT_F32, TS_HAS_BIAS.
#pragma once


namespace ts_nvfp4 {

constexpr ts_u32 kBlockM      = 128;
constexpr ts_u32 kTileM       = kBlockM * TS_CTA_GROUP;
constexpr ts_u32 kBlockN      = TS_BLOCK_N;
constexpr ts_u32 kLoadN       = kBlockN / TS_CTA_GROUP;
constexpr ts_u32 kBlockK      = 256;                          // K elements per stage = 128 bytes
constexpr ts_u32 kNumUmma     = 4;                            // 4 MMAs of K=64 per stage
constexpr ts_u32 kStages      = TS_STAGES;
constexpr ts_u32 kSmemA       = kBlockM * 128;
constexpr ts_u32 kSmemB       = kLoadN * 128;
constexpr ts_u32 kSfChunk     = 512;                          // one 128-row x 4-scale block
constexpr ts_u32 kSmemSfa     = kNumUmma * kSfChunk;          // 2 KB: this CTA's 128 rows of A
constexpr ts_u32 kNBlocks     = kBlockN / 128;                // 128-row blocks of B in the tile
constexpr ts_u32 kSmemSfb     = kNBlocks * kNumUmma * kSfChunk;
constexpr ts_u32 kOperandBytes = kSmemA + kSmemB;             // per CTA and stage, counted on the leader's full barrier
constexpr ts_u32 kScaleBytes  = kSmemSfa + kSmemSfb;          // per CTA and stage, counted on this CTA's scale barrier
constexpr ts_u32 kNumAcc      = (kBlockN == 256) ? 1 : 2;
constexpr ts_u32 kSfaCols     = kNumUmma * 4;                 // 4 TMEM columns per MMA and 128 rows
constexpr ts_u32 kSfbCols     = kNumUmma * 4 * kNBlocks;
constexpr ts_u32 kSfCols      = kSfaCols + kSfbCols;          // TMEM columns of one stage's scales
constexpr ts_u32 kSfBase      = kNumAcc * kBlockN;            // first scale column
constexpr ts_u32 kTmemCols    = 512;
constexpr ts_u32 kNumEpiWarps = 8;
constexpr ts_u32 kNumSfWarps  = 4;
constexpr ts_u32 kWarpCols    = kBlockN / 2;                  // columns one epilogue warp owns
constexpr ts_u32 kPassCols    = 64;                           // columns drained per pass
constexpr ts_u32 kPasses      = kWarpCols / kPassCols;
constexpr ts_u32 kOutBytes    = TS_OUT_F32 ? 4 : 2;
constexpr ts_u32 kChunkCols   = 128 / kOutBytes;
constexpr ts_u32 kPassChunks  = kPassCols / kChunkCols;
constexpr ts_u32 kStoreBuf    = 32 * 128;
constexpr ts_u32 kSmemC       = kNumEpiWarps * kStoreBuf;     // one staging buffer per epilogue warp
constexpr ts_u32 kNumBars     = 4 * kStages + 2 * kNumAcc;
constexpr ts_u32 kSmemTotal   = kStages * (kOperandBytes + kScaleBytes) + kSmemC + kNumBars * 8 + 16;
constexpr ts_u32 kThreads     = 448;

static_assert(kBlockN == 128 || kBlockN == 256, "TS_BLOCK_N must be 128 or 256 (whole 128-row scale blocks)");
static_assert(kSfBase + kStages * kSfCols <= kTmemCols, "accumulators and scale regions exceed tensor memory");
static_assert(kWarpCols % kPassCols == 0 && kPassCols % kChunkCols == 0, "bad epilogue split");
static_assert(kSfaCols == 16 && (kSfbCols == 16 || kSfbCols == 32), "scale stores are written for 16-column groups");
static_assert(kSmemTotal + 1024 <= 232448, "shared memory over the 227 KB limit");

}  // namespace ts_nvfp4

extern "C" __global__ void __launch_bounds__(448, 1)
TS_KERNEL_NAME(const __grid_constant__ TsTensorMap tmap_a,
               const __grid_constant__ TsTensorMap tmap_b,
               const __grid_constant__ TsTensorMap tmap_c,
               const __grid_constant__ TsTensorMap tmap_sfa,   // u32 [row blocks * K groups][128], box {128, 4}
               const __grid_constant__ TsTensorMap tmap_sfb,
               const ts_u16* __restrict__ bias,
               float alpha, int M, int N, int K, int group_m,
               ts_u32* __restrict__ status)
{
    using namespace ts_nvfp4;
    extern __shared__ ts_u8 ts_smem_raw[];
    const ts_u32 smem_base = (ts_smem_u32(ts_smem_raw) + 1023u) & ~1023u;
    const ts_u32 smem_a    = smem_base;
    const ts_u32 smem_b    = smem_a + kStages * kSmemA;
    const ts_u32 smem_sfa  = smem_b + kStages * kSmemB;
    const ts_u32 smem_sfb  = smem_sfa + kStages * kSmemSfa;
    const ts_u32 smem_c    = smem_sfb + kStages * kSmemSfb;
    const ts_u32 bar_base  = smem_c + kSmemC;
    const ts_u32 full_bar       = bar_base;                      // [kStages] operands landed (leader CTA)
    const ts_u32 empty_bar      = full_bar + 8 * kStages;        // [kStages] MMAs of the stage retired (both CTAs)
    const ts_u32 sf_full_bar    = empty_bar + 8 * kStages;       // [kStages] this CTA's scale chunks landed
    const ts_u32 sf_ready_bar   = sf_full_bar + 8 * kStages;     // [kStages] scales are in TMEM (leader CTA)
    const ts_u32 tmem_full_bar  = sf_ready_bar + 8 * kStages;    // [kNumAcc]
    const ts_u32 tmem_empty_bar = tmem_full_bar + 8 * kNumAcc;   // [kNumAcc]
    const ts_u32 tmem_ptr_smem  = tmem_empty_bar + 8 * kNumAcc;

    const ts_u32 warp_id  = threadIdx.x >> 5;
    const ts_u32 lane     = threadIdx.x & 31u;
    const ts_u32 cta_rank = (TS_CTA_GROUP == 2) ? ts_cluster_ctarank() : 0u;
    const bool   is_leader = (cta_rank == 0);

    const ts_u32 num_m = ((ts_u32)M + kTileM - 1) / kTileM;
    const ts_u32 num_n = ((ts_u32)N + kBlockN - 1) / kBlockN;
    const ts_u32 num_tiles = num_m * num_n;
    const ts_u32 num_k_blocks = ((ts_u32)K + kBlockK - 1) / kBlockK;
    const ts_u32 k_groups = (ts_u32)K / 64u;                 // 512-byte scale chunks per row block
    const ts_u32 first_tile = (TS_CTA_GROUP == 2) ? ts_cluster_id_x() : blockIdx.x;
    const ts_u32 tile_step  = (TS_CTA_GROUP == 2) ? ts_nclusters_x() : gridDim.x;
    const ts_u32 my_tiles = (first_tile < num_tiles) ? (num_tiles - first_tile + tile_step - 1) / tile_step : 0u;
    const ts_u32 total = my_tiles * num_k_blocks;            // stages this CTA runs, across its tiles

    if (warp_id == 0 && lane == 0) {
        ts_prefetch_tmap(&tmap_a);
        ts_prefetch_tmap(&tmap_b);
        ts_prefetch_tmap(&tmap_c);
        ts_prefetch_tmap(&tmap_sfa);
        ts_prefetch_tmap(&tmap_sfb);
        for (ts_u32 s = 0; s < kStages; ++s) {
            ts_mbar_init(full_bar + 8 * s, 1);
            ts_mbar_init(empty_bar + 8 * s, 1);
            ts_mbar_init(sf_full_bar + 8 * s, 1);
            ts_mbar_init(sf_ready_bar + 8 * s, kNumSfWarps * TS_CTA_GROUP);
        }
        for (ts_u32 b = 0; b < kNumAcc; ++b) {
            ts_mbar_init(tmem_full_bar + 8 * b, 1);
            ts_mbar_init(tmem_empty_bar + 8 * b, kNumEpiWarps * TS_CTA_GROUP);
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

    if (warp_id == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ts_u32 it = 0;
            bool ok = true;
            for (ts_u32 t = first_tile; t < num_tiles && ok; t += tile_step) {
                ts_u32 m_blk, n_blk;
                ts_decode_tile(t, num_m, num_n, (ts_u32)group_m, m_blk, n_blk);
                const int a_row = (int)(m_blk * kTileM + cta_rank * kBlockM);
                const int b_row = (int)(n_blk * kBlockN + cta_rank * kLoadN);
                const ts_u32 sfa_rb = m_blk * TS_CTA_GROUP + cta_rank;      // this CTA's 128-row block of A
                const ts_u32 sfb_rb = n_blk * kNBlocks;                      // first 128-row block of the B tile
                for (ts_u32 kb = 0; kb < num_k_blocks; ++kb, ++it) {
                    const ts_u32 s = it % kStages;
                    const ts_u32 ph = (it / kStages) & 1u;
                    if (!ts_mbar_wait(empty_bar + 8 * s, ph ^ 1u)) {
                        atomicOr(status, TS_ERR_TIMEOUT_EMPTY); ok = false; break;
                    }
                    // Scales first: they have one more hop to make than the operands (shared memory -> registers ->
                    // tensor memory, by the scale warps) before the MMAs of the stage can start.
                    // scales: 4 chunks (rows of the chunk table) per 128-row block and stage, into this CTA's
                    // own shared memory and onto its own barrier; each CTA of a pair fetches all of the B tile's
                    const ts_u32 sbar = sf_full_bar + 8 * s;
                    ts_mbar_arrive_expect_tx(sbar, kScaleBytes);
                    ts_tma_load_2d(smem_sfa + s * kSmemSfa, &tmap_sfa, sbar, 0, (int)(sfa_rb * k_groups + kb * 4));
#pragma unroll
                    for (ts_u32 nb = 0; nb < kNBlocks; ++nb)
                        ts_tma_load_2d(smem_sfb + s * kSmemSfb + nb * kNumUmma * kSfChunk, &tmap_sfb, sbar, 0,
                                       (int)((sfb_rb + nb) * k_groups + kb * 4));
                    const int kc = (int)(kb * 128u);                         // byte column of this stage in A and B
                    if (TS_CTA_GROUP == 1) {
                        ts_mbar_arrive_expect_tx(full_bar + 8 * s, kOperandBytes);
                        ts_tma_load_2d(smem_a + s * kSmemA, &tmap_a, full_bar + 8 * s, kc, a_row);
                        ts_tma_load_2d(smem_b + s * kSmemB, &tmap_b, full_bar + 8 * s, kc, b_row);
                    } else {
                        const ts_u32 leader_full = ts_mapa(full_bar + 8 * s, 0);
                        if (is_leader) ts_mbar_arrive_expect_tx(full_bar + 8 * s, kOperandBytes * 2);
                        ts_tma_load_2d_pair(smem_a + s * kSmemA, &tmap_a, leader_full, kc, a_row);
                        ts_tma_load_2d_pair(smem_b + s * kSmemB, &tmap_b, leader_full, kc, b_row);
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp_id == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The whole warp walks the loop (and waits on the barriers); one elected lane issues.
        if (is_leader) {
            // E2M1 x E2M1, UE4M3 scales, fp32 accumulate, both operands K-major
            constexpr ts_u32 idesc = ts_idesc_block_scaled(TS_FMT_E2M1_MXF4, TS_FMT_E2M1_MXF4, kTileM, kBlockN, 0u, 0u, 0u);
            const bool elected = ts_elect_one();
            bool ok = true;
            for (ts_u32 it = 0; it < total && ok; ++it) {
                const ts_u32 kb = it % num_k_blocks;
                const ts_u32 tile_iter = it / num_k_blocks;
                const ts_u32 acc = tile_iter % kNumAcc;
                const ts_u32 s = it % kStages;
                const ts_u32 ph = (it / kStages) & 1u;
                if (kb == 0) {
                    if (!ts_mbar_wait(tmem_empty_bar + 8 * acc, ((tile_iter / kNumAcc) & 1u) ^ 1u)) {
                        if (elected) atomicOr(status, TS_ERR_TIMEOUT_TMEM_EMPTY);
                        ok = false; break;
                    }
                }
                if (!ts_mbar_wait(full_bar + 8 * s, ph)) { if (elected) atomicOr(status, TS_ERR_TIMEOUT_FULL); ok = false; break; }
                if (!ts_mbar_wait(sf_ready_bar + 8 * s, ph)) { if (elected) atomicOr(status, TS_ERR_TIMEOUT_SCALE); ok = false; break; }
                ts_tc_fence_after();
                const ts_u32 d_tmem = tmem_base + acc * kBlockN;
                const ts_u32 sfa_tmem = tmem_base + kSfBase + s * kSfCols;     // 4 columns per MMA
                const ts_u32 sfb_tmem = sfa_tmem + kSfaCols;                   // 4 * kNBlocks columns per MMA
                const ts_u64 a_desc = ts_smem_desc_sw128(smem_a + s * kSmemA);
                const ts_u64 b_desc = ts_smem_desc_sw128(smem_b + s * kSmemB);
                if (elected) {
#pragma unroll
                    for (ts_u32 k = 0; k < kNumUmma; ++k)
                        ts_umma_nvfp4<TS_CTA_GROUP>(d_tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb | k) != 0u,
                                                    sfa_tmem + k * 4, sfb_tmem + k * 4 * kNBlocks);
                    // frees the smem stage and its TMEM scale region (in both CTAs of a pair) once these MMAs retire
                    if (TS_CTA_GROUP == 1) ts_umma_commit<1>(empty_bar + 8 * s);
                    else                   ts_umma_commit_pair(empty_bar + 8 * s, 3);
                    if (kb + 1 == num_k_blocks) {
                        if (TS_CTA_GROUP == 1) ts_umma_commit<1>(tmem_full_bar + 8 * acc);
                        else                   ts_umma_commit_pair(tmem_full_bar + 8 * acc, 3);
                    }
                }
                __syncwarp();
            }
        }
        __syncwarp();
    } else if (warp_id >= 2 + kNumEpiWarps) {
        // ------------------------------------------------------------ scale warps (10..13)
        // Warp w serves TMEM lanes 32*(w%4)..: lane l holds row l of every chunk (16 bytes = 4 columns).
        const ts_u32 quarter = warp_id & 3u;
        const ts_u32 leader_ready = (TS_CTA_GROUP == 2) ? ts_mapa(sf_ready_bar, 0) : sf_ready_bar;
        bool ok = true;
        for (ts_u32 it = 0; it < total && ok; ++it) {
            const ts_u32 s = it % kStages;
            const ts_u32 ph = (it / kStages) & 1u;
            // The producer refills stage s only after the MMAs that read it (and its scale region) retired,
            // so "chunks landed" also means "region s may be overwritten".
            if (!ts_mbar_wait(sf_full_bar + 8 * s, ph)) {
                if (lane == 0) atomicOr(status, TS_ERR_TIMEOUT_SCALE);
                ok = false; break;
            }
            const ts_u32 t_sf = tmem_base + ((quarter * 32u) << 16) + kSfBase + s * kSfCols;
            ts_u32 r[16];
            // A: chunk k -> columns 4k..4k+3
#pragma unroll
            for (ts_u32 k = 0; k < kNumUmma; ++k)
                ts_ld_shared_v4(smem_sfa + s * kSmemSfa + k * kSfChunk + lane * 16, r[4 * k], r[4 * k + 1], r[4 * k + 2], r[4 * k + 3]);
            ts_tmem_st_32x32b_x16(t_sf, r);
            // B: chunk (nb, k) -> columns kSfaCols + 4*kNBlocks*k + 4*nb ..; 16 columns per store
#pragma unroll
            for (ts_u32 g = 0; g < kSfbCols / 16; ++g) {
#pragma unroll
                for (ts_u32 q = 0; q < 4; ++q) {
                    const ts_u32 col = g * 16 + q * 4;               // column offset inside the B scale block
                    const ts_u32 k = col / (4 * kNBlocks), nb = (col / 4) % kNBlocks;
                    ts_ld_shared_v4(smem_sfb + s * kSmemSfb + (nb * kNumUmma + k) * kSfChunk + lane * 16,
                                    r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                }
                ts_tmem_st_32x32b_x16(t_sf + kSfaCols + g * 16, r);
            }
            ts_tmem_wait_st();
            ts_tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (TS_CTA_GROUP == 2) ts_mbar_arrive_cluster(leader_ready + 8 * s);
                else                   ts_mbar_arrive(sf_ready_bar + 8 * s);
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        const ts_u32 quarter = warp_id & 3u;
        const ts_u32 half = (warp_id - 2) >> 2;
        const ts_u32 store_smem = smem_c + (warp_id - 2) * kStoreBuf;
        const ts_u32 row_sw = (lane & 7u) << 4;
        const ts_u32 row_addr = store_smem + lane * 128;
        const ts_u32 leader_tmem_empty = (TS_CTA_GROUP == 2) ? ts_mapa(tmem_empty_bar, 0) : tmem_empty_bar;
        ts_u32 tile_iter = 0;
        bool ok = true;
        for (ts_u32 t = first_tile; t < num_tiles && ok; t += tile_step, ++tile_iter) {
            ts_u32 m_blk, n_blk;
            ts_decode_tile(t, num_m, num_n, (ts_u32)group_m, m_blk, n_blk);
            const ts_u32 acc = tile_iter % kNumAcc;
            const ts_u32 acc_ph = (tile_iter / kNumAcc) & 1u;
            if (!ts_mbar_wait(tmem_full_bar + 8 * acc, acc_ph)) {
                if (lane == 0) atomicOr(status, TS_ERR_TIMEOUT_TMEM_FULL);
                ok = false; break;
            }
            ts_tc_fence_after();
            const ts_u32 t_row = tmem_base + ((quarter * 32u) << 16) + acc * kBlockN + half * kWarpCols;
            const int row0 = (int)(m_blk * kTileM + cta_rank * kBlockM + quarter * 32);
            const ts_u32 col_base = n_blk * kBlockN + half * kWarpCols;
#if !TS_OUT_F32
            if (kPasses == 2) {
                // bf16 output, 128 columns per warp: the first 64 columns are scaled, biased and packed to bf16 in
                // registers (32 words) at once, so that the second 64 can be loaded straight after them and the
                // accumulator handed back to the MMA issuer before anything is staged or stored.  The time from
                // "accumulator complete" to "accumulator free" is two TMEM loads and 64 conversions; it is the part
                // of a tile that no MMA can overlap, because tensor memory has room for one 256-column accumulator.
                ts_u32 v[kPassCols], w0[kPassCols / 2];
                ts_tmem_ld_32x32b_x32(t_row, reinterpret_cast<ts_u32(&)[32]>(v[0]));
                ts_tmem_ld_32x32b_x32(t_row + 32, reinterpret_cast<ts_u32(&)[32]>(v[32]));
                ts_tmem_wait_ld();
                auto pack8 = [&](ts_u32 col0, ts_u32 c, ts_u32 (&out)[4]) __attribute__((always_inline)) {
                    float f[8];
#pragma unroll
                    for (ts_u32 i = 0; i < 8; ++i) f[i] = alpha * __uint_as_float(v[8 * c + i]);
#if TS_HAS_BIAS
                    if (col0 + 8 * c < (ts_u32)N) {
                        const uint4 bb = __ldg(reinterpret_cast<const uint4*>(bias + col0 + 8 * c));
                        f[0] += ts_bf16_lo_to_f32(bb.x); f[1] += ts_bf16_hi_to_f32(bb.x);
                        f[2] += ts_bf16_lo_to_f32(bb.y); f[3] += ts_bf16_hi_to_f32(bb.y);
                        f[4] += ts_bf16_lo_to_f32(bb.z); f[5] += ts_bf16_hi_to_f32(bb.z);
                        f[6] += ts_bf16_lo_to_f32(bb.w); f[7] += ts_bf16_hi_to_f32(bb.w);
                    }
#endif
                    out[0] = ts_pack_bf16x2(f[0], f[1]); out[1] = ts_pack_bf16x2(f[2], f[3]);
                    out[2] = ts_pack_bf16x2(f[4], f[5]); out[3] = ts_pack_bf16x2(f[6], f[7]);
                };
#pragma unroll
                for (ts_u32 c = 0; c < 8; ++c) pack8(col_base, c, reinterpret_cast<ts_u32(&)[4]>(w0[4 * c]));
                ts_tmem_ld_32x32b_x32(t_row + kPassCols, reinterpret_cast<ts_u32(&)[32]>(v[0]));
                ts_tmem_ld_32x32b_x32(t_row + kPassCols + 32, reinterpret_cast<ts_u32(&)[32]>(v[32]));
                ts_tmem_wait_ld();
                ts_tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if (TS_CTA_GROUP == 2) ts_mbar_arrive_cluster(leader_tmem_empty + 8 * acc);
                    else                   ts_mbar_arrive(tmem_empty_bar + 8 * acc);
                }
#pragma unroll
                for (ts_u32 p = 0; p < 2; ++p) {
                    const ts_u32 col0 = col_base + p * kPassCols;
                    if (lane == 0) ts_bulk_wait_read<0>();         // the previous store has read the staging buffer
                    __syncwarp();
#pragma unroll
                    for (ts_u32 c = 0; c < 8; ++c) {
                        ts_u32 o[4];
                        if (p == 0) { o[0] = w0[4 * c]; o[1] = w0[4 * c + 1]; o[2] = w0[4 * c + 2]; o[3] = w0[4 * c + 3]; }
                        else pack8(col0, c, o);
                        ts_st_shared_v4(row_addr + ((c << 4) ^ row_sw), o[0], o[1], o[2], o[3]);
                    }
                    ts_fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (col0 < (ts_u32)N && row0 < M) ts_tma_store_2d(&tmap_c, store_smem, (int)col0, row0);
                        ts_bulk_commit();
                    }
                }
                continue;
            }
#endif
#pragma unroll
            for (ts_u32 p = 0; p < kPasses; ++p) {
                ts_u32 v[kPassCols];
                ts_tmem_ld_32x32b_x32(t_row + p * kPassCols, reinterpret_cast<ts_u32(&)[32]>(v[0]));
                ts_tmem_ld_32x32b_x32(t_row + p * kPassCols + 32, reinterpret_cast<ts_u32(&)[32]>(v[32]));
                ts_tmem_wait_ld();
                if (p + 1 == kPasses) {
                    // the whole accumulator is in registers (or already stored): hand it back
                    ts_tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (TS_CTA_GROUP == 2) ts_mbar_arrive_cluster(leader_tmem_empty + 8 * acc);
                        else                   ts_mbar_arrive(tmem_empty_bar + 8 * acc);
                    }
                }
#pragma unroll
                for (ts_u32 j = 0; j < kPassChunks; ++j) {
                    const ts_u32 col0 = col_base + p * kPassCols + j * kChunkCols;
                    if (lane == 0) ts_bulk_wait_read<0>();         // the previous store has read the staging buffer
                    __syncwarp();
#pragma unroll
                    for (ts_u32 c = 0; c < 8; ++c) {
#if TS_OUT_F32
                        float f[4];
#pragma unroll
                        for (ts_u32 i = 0; i < 4; ++i) f[i] = alpha * __uint_as_float(v[j * kChunkCols + 4 * c + i]);
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
                        for (ts_u32 i = 0; i < 8; ++i) f[i] = alpha * __uint_as_float(v[j * kChunkCols + 8 * c + i]);
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
                    ts_fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (col0 < (ts_u32)N && row0 < M) ts_tma_store_2d(&tmap_c, store_smem, (int)col0, row0);
                        ts_bulk_commit();
                    }
                }
            }
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
