// Thin device wrappers over the sm_100a PTX that the GEMM mainloops are built from:
// mbarrier, TMA (cp.async.bulk.tensor), tcgen05 (alloc / mma / commit / ld / cp / fence)
// and the cluster primitives.  The header is self-contained (no CUDA or libc includes) so
// the same text compiles under nvcc and under NVRTC with no include path.
//
// It covers the primitive vocabulary of the reference IR (lib/tirix/tirix.mli:103-161:
// MbarInit, MbarArriveExpect, MbarWaitParity, MbarArrive, ClusterArrive/Wait, TmaLoad,
// Mma(Sm100Tcgen05), TmemAlloc/Dealloc/Load/Commit, Tcgen05Fence/Wait, SmemDescInit) and
// replaces the text helpers of lib/backend/backend_cute.ml:55-85 and the PTX strings of
// lib/pipeline/tmem.ml:72-133 and lib/pipeline/cluster.ml:76-98 with working code.
//
// Every wait is bounded: a wait that runs out returns false, the caller records an
// error word in global memory and leaves its loop, and the kernel still tears down.
#pragma once

typedef unsigned char      ts_u8;
typedef unsigned short     ts_u16;
typedef unsigned int       ts_u32;
typedef unsigned long long ts_u64;
typedef long long          ts_i64;

#define TS_DEV __device__ __forceinline__

// Opaque 128-byte tensor map (same size and alignment as the driver's CUtensorMap).
struct __align__(64) TsTensorMap { ts_u64 opaque[16]; };

// Error bits written to the status word.
#define TS_ERR_TIMEOUT_EMPTY      0x01u  // producer ran out waiting for a free smem stage
#define TS_ERR_TIMEOUT_FULL       0x02u  // MMA issuer ran out waiting for TMA data
#define TS_ERR_TIMEOUT_TMEM_EMPTY 0x04u  // MMA issuer ran out waiting for the epilogue
#define TS_ERR_TIMEOUT_TMEM_FULL  0x08u  // epilogue ran out waiting for the accumulator
#define TS_ERR_TIMEOUT_SCALE      0x10u  // scale-factor pipeline ran out
#define TS_ERR_BAD_TMEM_BASE      0x20u  // the two CTAs of a pair got different TMEM bases
#define TS_ERR_TIMEOUT_TEST       0x40u  // the deliberately unsignalled barrier of the wait self-test
#define TS_ERR_TIMEOUT_SCHED      0x80u  // the tile scheduler's ring (cluster launch control) ran out

// tcgen05.mma kinds of the dense kernels.
#define TS_KIND_F16     0
#define TS_KIND_F8F6F4  1
#define TS_KIND_I8      2

#ifndef TS_WAIT_TIMEOUT_CYCLES
#define TS_WAIT_TIMEOUT_CYCLES 4000000000ll  // about two seconds of SM clocks
#endif

TS_DEV ts_u32 ts_smem_u32(const void* p) {
    return (ts_u32)__cvta_generic_to_shared(p);
}
TS_DEV ts_u32 ts_lane() { return threadIdx.x & 31u; }

// ---------------------------------------------------------------- cluster
TS_DEV ts_u32 ts_cluster_ctarank() {
    ts_u32 r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
TS_DEV ts_u32 ts_cluster_id_x() {
    ts_u32 r; asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r)); return r;
}
TS_DEV ts_u32 ts_nclusters_x() {
    ts_u32 r; asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r)); return r;
}
TS_DEV void ts_cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
TS_DEV void ts_cluster_wait()   { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
TS_DEV void ts_cluster_sync()   { ts_cluster_arrive(); ts_cluster_wait(); }
// Address of the same shared-memory location in CTA `rank` of this cluster.
TS_DEV ts_u32 ts_mapa(ts_u32 local_addr, ts_u32 rank) {
    ts_u32 r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank)); return r;
}

// ---------------------------------------------------------------- mbarrier
TS_DEV void ts_mbar_init(ts_u32 bar, ts_u32 count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
TS_DEV void ts_fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
TS_DEV void ts_fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
TS_DEV void ts_mbar_arrive_expect_tx(ts_u32 bar, ts_u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
TS_DEV void ts_mbar_arrive(ts_u32 bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
// Arrive on a barrier that lives in another CTA of the cluster (address from ts_mapa).
TS_DEV void ts_mbar_arrive_cluster(ts_u32 cluster_bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_bar) : "memory");
}
// The same with release semantics at cluster scope: what was written to the other CTA's shared memory before it
// (st.shared::cluster) is visible to a thread there that waits with ts_mbar_wait_cluster.
TS_DEV void ts_mbar_arrive_release_cluster(ts_u32 cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" :: "r"(cluster_bar) : "memory");
}
TS_DEV void ts_st_shared_cluster_u32(ts_u32 cluster_addr, ts_u32 v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(cluster_addr), "r"(v) : "memory");
}
TS_DEV bool ts_mbar_try_wait_cluster(ts_u32 bar, ts_u32 parity) {
    ts_u32 ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
TS_DEV bool ts_mbar_try_wait(ts_u32 bar, ts_u32 parity) {
    ts_u32 ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait for the phase with the given parity.  Returns false when the cycle budget
// ran out; the healthy path costs one try_wait.  The lanes that call it together get the
// same answer: once the first try has failed, the outcome of the polling loop is voted on
// by those lanes, so a barrier that completes just as the budget expires cannot send part
// of a warp down the error path in front of an aligned instruction.
TS_DEV bool ts_mbar_wait(ts_u32 bar, ts_u32 parity, ts_i64 budget = TS_WAIT_TIMEOUT_CYCLES) {
    if (ts_mbar_try_wait(bar, parity)) return true;
    const ts_u32 peers = __activemask();
    const ts_i64 t0 = clock64();
    bool ok = true;
    while (!ts_mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > budget) { ok = false; break; }
    }
    __syncwarp(peers);
    return __all_sync(peers, ok) != 0;
}

// Bounded wait with acquire at cluster scope (the barrier is signalled from another CTA of the cluster and guards
// data that CTA wrote here).
TS_DEV bool ts_mbar_wait_cluster(ts_u32 bar, ts_u32 parity, ts_i64 budget = TS_WAIT_TIMEOUT_CYCLES) {
    if (ts_mbar_try_wait_cluster(bar, parity)) return true;
    const ts_u32 peers = __activemask();
    const ts_i64 t0 = clock64();
    bool ok = true;
    while (!ts_mbar_try_wait_cluster(bar, parity)) {
        if (clock64() - t0 > budget) { ok = false; break; }
    }
    __syncwarp(peers);
    return __all_sync(peers, ok) != 0;
}

// ---------------------------------------------------------------- cluster launch control
// Asks the hardware to cancel the launch of one cluster of this grid that has not started yet.  The 16-byte answer
// lands in this CTA's shared memory at `response` and completes 16 bytes on `bar`.  After an answer that says
// "nothing was cancelled" no further request may be made by this cluster.
TS_DEV void ts_clc_try_cancel(ts_u32 response, ts_u32 bar) {
    asm volatile("clusterlaunchcontrol.try_cancel.async.shared::cta.mbarrier::complete_tx::bytes.b128 [%0], [%1];"
                 :: "r"(response), "r"(bar) : "memory");
}
// Reads an answer: true and the x index of the cancelled cluster's first CTA, or false.
TS_DEV bool ts_clc_query(ts_u32 response, ts_u32& first_cta_x) {
    ts_u32 got, x;
    asm volatile(
        "{\n\t.reg .b128 r;\n\t.reg .pred p;\n\t"
        "ld.shared.b128 r, [%2];\n\t"
        "clusterlaunchcontrol.query_cancel.is_canceled.pred.b128 p, r;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "mov.u32 %1, 0;\n\t"
        "@p clusterlaunchcontrol.query_cancel.get_first_ctaid::x.b32.b128 %1, r;\n\t}"
        : "=r"(got), "=r"(x) : "r"(response) : "memory");
    first_cta_x = x;
    return got != 0;
}

// ---------------------------------------------------------------- TMA
TS_DEV void ts_prefetch_tmap(const TsTensorMap* m) {
    asm volatile("prefetch.tensormap [%0];" :: "l"((ts_u64)m) : "memory");
}
// One 2-D tile, global -> this CTA's shared memory, completing `bar` (own CTA) by bytes.
TS_DEV void ts_tma_load_2d(ts_u32 dst, const TsTensorMap* m, ts_u32 bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :: "r"(dst), "l"((ts_u64)m), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
// Same, for a CTA pair: the data lands in this CTA's shared memory, the byte count is
// signalled on `cluster_bar`, which may live in the peer CTA (address from ts_mapa).
TS_DEV void ts_tma_load_2d_pair(ts_u32 dst, const TsTensorMap* m, ts_u32 cluster_bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        :: "r"(dst), "l"((ts_u64)m), "r"(cluster_bar), "r"(c0), "r"(c1) : "memory");
}
TS_DEV void ts_tma_load_3d(ts_u32 dst, const TsTensorMap* m, ts_u32 bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        :: "r"(dst), "l"((ts_u64)m), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
TS_DEV void ts_tma_store_2d(const TsTensorMap* m, ts_u32 src, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
        :: "l"((ts_u64)m), "r"(src), "r"(c0), "r"(c1) : "memory");
}
// Shared memory -> global with an fp32 add at the destination (the tensor map's element type is fp32): the tile
// is added into what the destination holds, element by element, in the memory system of the GPU that owns it.
// A store-type operation: nothing is read back.  Concurrent adds to one element arrive in no fixed order.
TS_DEV void ts_tma_reduce_add_2d(const TsTensorMap* m, ts_u32 src, int c0, int c1) {
    asm volatile(
        "cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
        :: "l"((ts_u64)m), "r"(src), "r"(c0), "r"(c1) : "memory");
}
TS_DEV void ts_bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> TS_DEV void ts_bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
TS_DEV void ts_bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// ---------------------------------------------------------------- tcgen05 / TMEM
template <int CTA_GROUP> TS_DEV void ts_tmem_alloc(ts_u32 dst_smem, ts_u32 ncols) {
    if (CTA_GROUP == 1)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(dst_smem), "r"(ncols) : "memory");
    else
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(dst_smem), "r"(ncols) : "memory");
}
template <int CTA_GROUP> TS_DEV void ts_tmem_relinquish() {
    if (CTA_GROUP == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    else                asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTA_GROUP> TS_DEV void ts_tmem_dealloc(ts_u32 taddr, ts_u32 ncols) {
    if (CTA_GROUP == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
    else                asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(ncols) : "memory");
}
TS_DEV void ts_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
TS_DEV void ts_tc_fence_after()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
TS_DEV void ts_tmem_wait_ld()    { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor for a K-major operand tile that TMA wrote with Swizzle<B,4,3>
// (lib/core/swizzle.ml:46-56 picks B from the bytes of K in one tile row: 32, 64 or 128 bytes for
// B = 1, 2, 3).  Rows are 16 << B bytes, 8-row groups are 8 rows apart (stride byte offset), the
// leading byte offset is unused for swizzled K-major tiles (encoded 1), descriptor version 1,
// layout type 6 / 4 / 2 for the 32 / 64 / 128-byte swizzle.  All byte fields drop their four low
// bits.  The host function of the same content is tesserae_umma_smem_desc.  The hardware form
// differs from the reference's sketch (lib/pipeline/smem_desc.ml:38-43), which is kept only as a
// bit-exact integer function on the host.
template <int SWZ_B> TS_DEV ts_u64 ts_smem_desc_kmajor(ts_u32 smem_addr) {
    static_assert(SWZ_B >= 1 && SWZ_B <= 3, "K-major operand tiles are swizzled with B in 1..3");
    constexpr ts_u32 row_bytes = 16u << SWZ_B;
    constexpr ts_u32 layout = SWZ_B == 3 ? 2u : (SWZ_B == 2 ? 4u : 6u);
    const ts_u32 lo = ((smem_addr & 0x3FFFFu) >> 4) | (1u << 16);
    const ts_u32 hi = ((8u * row_bytes) >> 4) | (1u << 14) | (layout << 29);
    return ((ts_u64)hi << 32) | lo;
}
TS_DEV ts_u64 ts_smem_desc_sw128(ts_u32 smem_addr) { return ts_smem_desc_kmajor<3>(smem_addr); }
// Descriptor for a tile without swizzle whose 8x16-byte core matrices are stored
// contiguously (128 bytes each): used for the scale-factor copies to TMEM.
TS_DEV ts_u64 ts_smem_desc_noswizzle(ts_u32 smem_addr, ts_u32 lbo_bytes, ts_u32 sbo_bytes) {
    const ts_u32 lo = ((smem_addr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
    const ts_u32 hi = (sbo_bytes >> 4) | (1u << 14);
    return ((ts_u64)hi << 32) | lo;
}

// Instruction descriptor of the dense kinds (kind::f16, kind::tf32, kind::f8f6f4):
// D format at [4,6) (1 = f32), A format at [7,10), B format at [10,13), transpose bits 15
// and 16 left 0 (both operands K-major), N>>3 at [17,23), M>>4 at [24,29).
#define TS_FMT_F16  0u
#define TS_FMT_BF16 1u
#define TS_FMT_E4M3 0u
#define TS_FMT_E2M1_MXF4 1u
#define TS_FMT_S8   1u
TS_DEV constexpr ts_u32 ts_idesc_dense(ts_u32 a_fmt, ts_u32 b_fmt, ts_u32 umma_m, ts_u32 umma_n, ts_u32 d_fmt = 1u) {
    return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}
// Accumulator word -> float: fp32 bits for the float kinds, a signed 32-bit integer for kind::i8.
template <int KIND> TS_DEV float ts_acc_to_f32(ts_u32 w) {
    return KIND == TS_KIND_I8 ? (float)(int)w : __uint_as_float(w);
}
// Block-scaled kinds (kind::mxf4nvf4 here): scale-factor ids at [4,6) (B) and [29,31) (A),
// scale format at bit 23 (0 = UE4M3, 1 = UE8M0).
TS_DEV constexpr ts_u32 ts_idesc_block_scaled(ts_u32 a_fmt, ts_u32 b_fmt, ts_u32 umma_m, ts_u32 umma_n,
                                              ts_u32 scale_fmt, ts_u32 a_sf_id, ts_u32 b_sf_id) {
    return (b_sf_id << 4) | (a_fmt << 7) | (b_fmt << 10) | ((umma_n >> 3) << 17) | (scale_fmt << 23) |
           ((umma_m >> 4) << 24) | (a_sf_id << 29);
}

// One lane of the (converged) warp, chosen by the hardware.  The MMA and TMA issue loops run with all 32 lanes
// and predicate only the issuing instructions on this lane: addresses and descriptors then stay warp-uniform
// values, which is what the tcgen05 instructions take, instead of per-thread values of a one-lane branch.
TS_DEV bool ts_elect_one() {
    ts_u32 pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0u;
}

// D[tmem] (+)= A[smem] * B[smem]; issued by one thread.
template <int CTA_GROUP, int KIND>
TS_DEV void ts_umma(ts_u32 d_tmem, ts_u64 a_desc, ts_u64 b_desc, ts_u32 idesc, ts_u32 accumulate) {
    if (CTA_GROUP == 1 && KIND == TS_KIND_F16)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else if (CTA_GROUP == 2 && KIND == TS_KIND_F16)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else if (CTA_GROUP == 1 && KIND == TS_KIND_I8)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else if (CTA_GROUP == 2 && KIND == TS_KIND_I8)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else if (CTA_GROUP == 1 && KIND == TS_KIND_F8F6F4)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// NVFP4: E2M1 operands, one UE4M3 scale per 16 K-elements, scales read from TMEM.
template <int CTA_GROUP>
TS_DEV void ts_umma_nvfp4(ts_u32 d_tmem, ts_u64 a_desc, ts_u64 b_desc, ts_u32 idesc, ts_u32 accumulate,
                          ts_u32 sfa_tmem, ts_u32 sfb_tmem) {
    if (CTA_GROUP == 1)
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
    else
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::2.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
                     :: "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// Shared memory -> TMEM copy of one 32-row x 16-byte block, replicated to the four
// 32-lane quarters (the form the scale-factor operands want).
template <int CTA_GROUP> TS_DEV void ts_tmem_cp_32x128b_warpx4(ts_u32 taddr, ts_u64 s_desc) {
    if (CTA_GROUP == 1) asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" :: "r"(taddr), "l"(s_desc) : "memory");
    else                asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" :: "r"(taddr), "l"(s_desc) : "memory");
}
// Make `bar` (own CTA) complete one arrival when all MMAs this thread issued so far retire.
template <int CTA_GROUP> TS_DEV void ts_umma_commit(ts_u32 bar) {
    if (CTA_GROUP == 1)
        asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
    else
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(bar) : "memory");
}
// Pair form: the arrival is delivered to the barrier at the same offset in every CTA of
// `cta_mask`.  This is an arrival signal, not a data load.
TS_DEV void ts_umma_commit_pair(ts_u32 bar, ts_u16 cta_mask) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(bar), "h"(cta_mask) : "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp reads lane
// (taddr.lane + t), columns taddr.col .. +31.  A warp may only name lanes of its own
// quarter, 32 * (warp_id % 4).
TS_DEV void ts_tmem_ld_32x32b_x32(ts_u32 taddr, ts_u32 (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
TS_DEV void ts_tmem_ld_32x32b_x16(ts_u32 taddr, ts_u32 (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
// Register budget of the calling warpgroup (4 consecutive warps, all of which execute this): the issuing warps
// give registers back, the warps that hold accumulators take them.  N is a multiple of 8 in [24, 256].
template <int N> TS_DEV void ts_setmaxnreg_inc() { asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" :: "n"(N)); }
template <int N> TS_DEV void ts_setmaxnreg_dec() { asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(N)); }
// Registers -> TMEM, the mirror of the loads above: thread t writes lane (taddr.lane + t),
// 16 consecutive 32-bit columns.  Completed by ts_tmem_wait_st().
TS_DEV void ts_tmem_st_32x32b_x16(ts_u32 taddr, const ts_u32 (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
           "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
TS_DEV void ts_tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
TS_DEV void ts_ld_shared_v4(ts_u32 addr, ts_u32& a, ts_u32& b, ts_u32& c, ts_u32& d) {
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr) : "memory");
}

// ---------------------------------------------------------------- tile order of the persistent kernels
// Tiles are walked in raster groups of `group_m` M-tiles: inside a group the M index runs fastest, so the tiles
// that are in flight together share a panel of A (group_m M-tiles) and a few N-tiles of B.  `group_m` is a launch
// argument: the host sizes it so that the A panel of a group stays in L2 while the group sweeps all of B.
TS_DEV void ts_decode_tile(ts_u32 t, ts_u32 num_m, ts_u32 num_n, ts_u32 group_m, ts_u32& m_blk, ts_u32& n_blk) {
    const ts_u32 group_size = group_m * num_n;
    const ts_u32 g = t / group_size;
    const ts_u32 first_m = g * group_m;
    const ts_u32 gm = (num_m - first_m < group_m) ? (num_m - first_m) : group_m;
    const ts_u32 r = t - g * group_size;
    m_blk = first_m + r % gm;
    n_blk = r / gm;
}
// x / d through a float reciprocal with an exact correction; x < 2^22, d >= 1.
TS_DEV ts_u32 ts_div_by_reciprocal(ts_u32 x, ts_u32 d, float inv_d) {
    ts_u32 q = (ts_u32)__float2uint_rz(__uint2float_rz(x) * inv_d);
    const int r = (int)x - (int)(q * d);
    if (r < 0) q -= 1u; else if (r >= (int)d) q += 1u;
    return q;
}
// The same map without an integer division on the common path (t < 2^22): for warps that decode between two tiles,
// where dependent divisions are a visible part of the gap.  inv_group = 1 / (group_m * num_n), inv_gm = 1 / group_m.
TS_DEV void ts_decode_tile_fast(ts_u32 t, ts_u32 num_m, ts_u32 num_n, ts_u32 group_m, float inv_group, float inv_gm,
                                ts_u32& m_blk, ts_u32& n_blk) {
    const ts_u32 group_size = group_m * num_n;
    const ts_u32 g = ts_div_by_reciprocal(t, group_size, inv_group);
    const ts_u32 r = t - g * group_size;
    const ts_u32 first_m = g * group_m;
    if (num_m - first_m >= group_m) {
        n_blk = ts_div_by_reciprocal(r, group_m, inv_gm);
        m_blk = first_m + r - n_blk * group_m;
    } else {
        const ts_u32 gm = num_m - first_m;
        m_blk = first_m + r % gm;
        n_blk = r / gm;
    }
}

// ---------------------------------------------------------------- small utilities
// Packed pairs of fp32 in one 64-bit register and the two-wide multiply-add over them: d = a * b + c per half,
// each half rounded once like a scalar fma.rn.
TS_DEV ts_u64 ts_pack_f32x2(ts_u32 lo, ts_u32 hi) {
    ts_u64 r; asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi)); return r;
}
TS_DEV void ts_unpack_f32x2(ts_u64 v, float& lo, float& hi) {
    ts_u32 a, b; asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
    lo = __uint_as_float(a); hi = __uint_as_float(b);
}
TS_DEV ts_u64 ts_fma_f32x2(ts_u64 a, ts_u64 b, ts_u64 c) {
    ts_u64 d; asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c)); return d;
}
// Two fp32 -> packed bf16x2 (round to nearest even); `lo` lands in the low half.
TS_DEV ts_u32 ts_pack_bf16x2(float lo, float hi) {
    ts_u32 r; asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo)); return r;
}
TS_DEV float ts_bf16_lo_to_f32(ts_u32 packed) { return __uint_as_float(packed << 16); }
TS_DEV float ts_bf16_hi_to_f32(ts_u32 packed) { return __uint_as_float(packed & 0xFFFF0000u); }
TS_DEV void ts_st_shared_v4(ts_u32 addr, ts_u32 a, ts_u32 b, ts_u32 c, ts_u32 d) {
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" :: "r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
