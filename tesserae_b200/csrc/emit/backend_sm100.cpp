// Backend: kernel spec -> specialised sm_100a CUDA source.
//
// Takes the place of Backend_cute.emit (lib/backend/backend_cute.ml:431-453) for the
// Blackwell family and returns the same record of sections
// (lib/backend/backend_cute.mli:10-21).  The reference builds its kernel from Printf
// templates; here the device code is hand-written once (csrc/kernels/*.cuh, embedded in the
// library) and the emitter specialises it by a block of #defines, so the text NVRTC
// compiles at run time is the text nvcc compiles at build time.
#include "backend_sm100.hpp"

#include <cctype>
#include <cstdio>
#include <cstdlib>

namespace tesserae {

namespace {

constexpr int kSmemLimit = 232448;   // 227 KB of dynamic shared memory per CTA on sm_100

// Dynamic shared memory of each kernel family; mirrors kSmemTotal in the .cuh plus the
// 1024-byte alignment slack.
int dense_smem_bytes(int cta_group, int block_n, int stages, int store_bufs, int row_bytes, int clc) {
    const int stage = (128 + block_n / cta_group) * row_bytes;
    const int sched = clc ? (2 * 4 + 1) * 8 + 48 : 0;     // the scheduler's ring: barriers, answer, tile ids
    const int epi_warps = block_n > 256 ? 8 : 4;
    return stages * stage + epi_warps * store_bufs * 4096 + (2 * stages + 4) * 8 + 16 + sched + 1024;
}
int fp8_smem_bytes(int cta_group, int block_n, int stages, int promo_warps, int out_bytes) {
    const int stage = 128 * 128 + (block_n / cta_group) * 128;
    const int warp_chunks = (block_n / (promo_warps / 4)) / (128 / out_bytes);
    const int store_bufs = warp_chunks >= 2 ? 2 : 1;
    return stages * stage + promo_warps * store_bufs * 4096 + (2 * stages + 2 * (512 / block_n)) * 8 + 16 + 1024;
}
int nvfp4_smem_bytes(int cta_group, int block_n, int stages) {
    const int stage = 128 * 128 + (block_n / cta_group) * 128 + 2048 + (block_n / 128) * 2048;
    const int num_acc = block_n == 256 ? 1 : 2;
    return stages * stage + 8 * 4096 + (4 * stages + 2 * num_acc) * 8 + 16 + 1024;
}
// Stage s of the NVFP4 kernel owns TMEM scale region s next to the accumulators: 512 columns bound the depth.
int nvfp4_max_stages(int block_n) {
    const int num_acc = block_n == 256 ? 1 : 2;
    return (512 - num_acc * block_n) / (16 + 16 * (block_n / 128));
}
int smem_bytes_for(const KernelConfig& c, int stages) {
    const int ob = c.out_elem == TESSERAE_F32 ? 4 : 2;
    if (c.scale_mode == TESSERAE_SCALE_FP8_BLOCK) return fp8_smem_bytes(c.cta_group, c.block_n, stages, c.promo_warps, ob);
    if (c.scale_mode == TESSERAE_SCALE_NVFP4) return nvfp4_smem_bytes(c.cta_group, c.block_n, stages);
    return dense_smem_bytes(c.cta_group, c.block_n, stages, c.store_bufs, 16 << c.desc.swizzle.b, c.clc);
}

std::string sanitize(const char* name) {
    std::string s = (name && *name) ? name : "tesserae_gemm";
    for (char& c : s) if (!isalnum((unsigned char)c) && c != '_') c = '_';
    if (isdigit((unsigned char)s[0])) s = "k_" + s;
    return s;
}

// "NAME=VALUE;NAME=VALUE" -> pairs; false on a malformed entry.
bool parse_tuning(const char* text, std::vector<std::pair<std::string, int>>* out, std::string* bad) {
    if (!text) return true;
    std::string s(text);
    size_t at = 0;
    while (at < s.size()) {
        size_t end = s.find(';', at);
        if (end == std::string::npos) end = s.size();
        std::string item = s.substr(at, end - at);
        at = end + 1;
        while (!item.empty() && isspace((unsigned char)item.back())) item.pop_back();
        while (!item.empty() && isspace((unsigned char)item.front())) item.erase(item.begin());
        if (item.empty()) continue;
        const size_t eq = item.find('=');
        if (eq == std::string::npos || eq == 0 || eq + 1 >= item.size()) { *bad = item; return false; }
        char* tail = nullptr;
        const long v = strtol(item.c_str() + eq + 1, &tail, 10);
        if (*tail != '\0') { *bad = item; return false; }
        out->emplace_back(item.substr(0, eq), int(v));
    }
    return true;
}

std::string strip_pragma_once(const char* text) {
    std::string s = text ? text : "";
    const std::string p = "#pragma once";
    size_t at = s.find(p);
    if (at != std::string::npos) s.replace(at, p.size(), "// (single translation unit)");
    return s;
}

// Text between the line containing `from` and the line containing `to` (exclusive).
std::string slice(const std::string& s, const char* from, const char* to) {
    size_t a = s.find(from);
    if (a == std::string::npos) return "";
    a = s.rfind('\n', a);
    a = (a == std::string::npos) ? 0 : a + 1;
    size_t b = to ? s.find(to, a + 1) : std::string::npos;
    if (b != std::string::npos) { b = s.rfind('\n', b); }
    return s.substr(a, b == std::string::npos ? std::string::npos : b - a);
}

}  // namespace

std::vector<std::string> nvrtc_options() {
    return {"--gpu-architecture=sm_100a", "--std=c++17", "-lineinfo", "-default-device"};
}

int derive_config(const tesserae_kernel_spec& ks, KernelConfig* cfg, std::string* msg) {
    spec::KernelDesc desc;
    int rc = spec::lower(sanitize(ks.name), ks.arch, ks.elem, ks.tile_m, ks.tile_n, ks.tile_k, &desc, msg);
    if (rc != spec::LowerOk) return rc;
    const std::string verr = spec::validate(desc);
    if (!verr.empty()) { if (msg) *msg = "IncompatibleTile: " + verr; return spec::IncompatibleTile; }

    KernelConfig c;
    c.name = desc.name;
    c.elem = ks.elem;
    c.desc = desc;
    c.cta_group = (ks.cta_group == 1) ? 1 : 2;
    c.out_elem = (ks.out_elem == TESSERAE_BF16) ? TESSERAE_BF16 : TESSERAE_F32;
    c.has_bias = ks.has_bias ? 1 : 0;
    c.scale_mode = ks.scale_mode;
    c.scatter = (ks.scatter == 1 || ks.scatter == 2) ? ks.scatter : 0;
    if (ks.scatter != 0 && c.scatter == 0) {
        if (msg) *msg = "IncompatibleTile: scatter must be 0, 1 (store to per-source slots) or 2 (add into the owner's buffer)";
        return spec::IncompatibleTile;
    }
    c.grouped = ks.grouped ? 1 : 0;
    if (c.grouped && (ks.scale_mode != TESSERAE_SCALE_NONE || c.scatter)) {
        if (msg) *msg = "IncompatibleTile: grouped launches are for the unscaled kernels without scattered output";
        return spec::IncompatibleTile;
    }
    if (c.scatter && (ks.scale_mode != TESSERAE_SCALE_NONE || ks.has_bias || c.out_elem != TESSERAE_F32)) {
        if (msg) *msg = "IncompatibleTile: scattered output is for unscaled kernels with fp32 output and no bias";
        return spec::IncompatibleTile;
    }
    // Staging depth of the dense epilogue: deeper when the stores may cross NVLink.
    c.store_bufs = c.scatter ? 4 : 2;
    // The spec's own tuning overrides (nothing is read from the environment).
    int want_promo_warps = 0;
    {
        std::vector<std::pair<std::string, int>> tv;
        std::string bad;
        if (!parse_tuning(ks.tuning, &tv, &bad)) {
            if (msg) *msg = "IncompatibleTile: malformed tuning entry '" + bad + "' (want NAME=VALUE)";
            return spec::IncompatibleTile;
        }
        for (const auto& kv : tv) {
            const std::string& key = kv.first;
            const int v = kv.second;
            bool ok = true;
            if (key == "GROUP_M") { ok = v >= 1 && v <= 64; c.group_m = v; }
            else if (key == "STORE_BUFS") { ok = v >= 2 && v <= 4; c.store_bufs = v; }
            else if (key == "FP8_PROMO_WARPS") { ok = v == 8 || v == 16; want_promo_warps = v; }
            else if (key == "FP8_SPLIT") { ok = v == 0 || v == 1; c.fp8_split = v; }
            else if (key == "TAIL_SPLITS") { ok = v >= 0 && v <= 64; c.tail_splits = v; }
            else if (key == "CLC") { ok = v == 0 || v == 1; c.clc = v; }
            else { if (msg) *msg = "IncompatibleTile: unknown tuning name '" + key + "'"; return spec::IncompatibleTile; }
            if (!ok) {
                if (msg) *msg = "IncompatibleTile: tuning value out of range: " + key + "=" + std::to_string(v);
                return spec::IncompatibleTile;
            }
        }
    }
    c.block_m = 128;
    c.block_n = ks.tile_n;
    c.block_k = ks.tile_k;
    c.threads = spec::thread_count(desc.cluster);
    if (c.clc && (ks.scale_mode != TESSERAE_SCALE_NONE || c.scatter)) {
        if (msg) *msg = "IncompatibleTile: the cluster-launch-control scheduler is for the unscaled kernels without scattered output";
        return spec::IncompatibleTile;
    }
    if (c.clc) c.threads += 32;        // the scheduler warp (Cluster's Scheduler role, lib/pipeline/cluster.mli:17-21)

    // What the hand-written mainloops cover: 128 rows per CTA, one swizzle row of K per stage, N a multiple
    // of the store chunk and of 16 per CTA.  The swizzle is the one Swizzle.smem_selector derives from the tile
    // (lib/core/swizzle.ml:46-56): the row a stage holds must be exactly the 16 << B bytes that Swizzle<B,4,3>
    // permutes, B in 1..3 for the dense kernels; the block-scaled kernels need the 128-byte row (their scale
    // blocks are one row wide).
    if (ks.tile_m != 128) { if (msg) *msg = "IncompatibleTile: tile.m must be 128 (rows per CTA)"; return spec::IncompatibleTile; }
    {
        const int64_t row_bytes = int64_t(ks.tile_k) * spec::elem_bits(ks.elem) / 8;
        const bool scaled = ks.scale_mode != TESSERAE_SCALE_NONE;
        if (desc.swizzle.b < 1 || desc.swizzle.b > 3 || row_bytes != (int64_t(16) << desc.swizzle.b) ||
            (scaled && desc.swizzle.b != 3)) {
            if (msg) *msg = scaled ? "IncompatibleTile: tile.k must span exactly 128 bytes (Swizzle<3,4,3>) for a block-scaled kernel"
                                   : "IncompatibleTile: tile.k must span 32, 64 or 128 bytes (Swizzle<1..3,4,3>)";
            return spec::IncompatibleTile;
        }
    }
    const int chunk = (c.out_elem == TESSERAE_F32) ? 32 : 64;
    // 512 columns: the unscaled CTA-pair kernels only (two MMA groups of 256 into one accumulator that fills tensor memory)
    const bool wide = c.block_n == 512 && c.cta_group == 2 && ks.scale_mode == TESSERAE_SCALE_NONE;
    if (!wide && (c.block_n < 16 * c.cta_group || c.block_n > 256 || c.block_n % (16 * c.cta_group) != 0 || c.block_n % chunk != 0)) {
        if (msg) *msg = "IncompatibleTile: tile.n must be a multiple of " + std::to_string(std::max(chunk, 16 * c.cta_group)) +
                        " and <= 256 (512 for an unscaled CTA-pair kernel)";
        return spec::IncompatibleTile;
    }
    if (wide) {
        c.threads += 128;              // eight epilogue warps: the one accumulator of the 512-column tile has to drain quickly
        c.store_bufs = 1;              // one staging buffer per epilogue warp keeps four stages in shared memory
    }
    if (ks.scale_mode == TESSERAE_SCALE_FP8_BLOCK && ks.elem != TESSERAE_F8E4M3) {
        if (msg) *msg = "UnsupportedElem: FP8 block scaling needs elem F8E4M3";
        return spec::UnsupportedElem;
    }
    if ((ks.scale_mode == TESSERAE_SCALE_NVFP4) != (ks.elem == TESSERAE_F4E2M1)) {
        if (msg) *msg = "UnsupportedElem: F4E2M1 and NVFP4 scaling go together";
        return spec::UnsupportedElem;
    }

    c.b_box_rows = (c.block_n > 256 ? 256 : c.block_n) / c.cta_group;      // one TMA load per MMA group of at most 256 columns
    if (c.scale_mode == TESSERAE_SCALE_FP8_BLOCK) {
        // Promotion warps on top of the producer and MMA warps.  8 (two per scheduler) measured
        // faster than 16 on the 256-wide tile: the TMEM reads contend with the running MMA, not with
        // each other.
        c.promo_warps = 8;
        if (want_promo_warps) {
            if ((c.block_n / (want_promo_warps / 4)) % ((c.out_elem == TESSERAE_F32) ? 32 : 64) != 0) {
                if (msg) *msg = "IncompatibleTile: FP8_PROMO_WARPS=" + std::to_string(want_promo_warps) + " leaves a warp less than one store chunk of columns";
                return spec::IncompatibleTile;
            }
            c.promo_warps = want_promo_warps;
        }
        c.threads = 128 + 32 * c.promo_warps;     // warpgroup 0 (producer, MMA issuer, two idle warps) + promotion warps
        if (c.cta_group == 2 && c.fp8_split) c.b_box_rows = 64;  // 64 rows per CTA and 128-column MMA group
        if (c.block_n != 128 && c.block_n != 256) {
            if (msg) *msg = "IncompatibleTile: FP8 block scaling needs tile.n of 128 or 256 (whole 128x128 scale blocks)";
            return spec::IncompatibleTile;
        }
    }
    if (c.scale_mode == TESSERAE_SCALE_NVFP4) {
        c.threads = 448;   // producer, MMA issuer, eight epilogue warps, four scale warps
        if (c.block_n != 128 && c.block_n != 256) {
            if (msg) *msg = "IncompatibleTile: NVFP4 needs tile.n of 128 or 256 (whole 128-row scale blocks)";
            return spec::IncompatibleTile;
        }
    }
    // Stage count: the reference fixes depth 4 (lib/kernel/kernel_desc.ml:136); here the ring is
    // as deep as shared memory allows unless the spec asks for fewer.
    int fit = 0;
    for (int s = 1; s <= 12; ++s) if (smem_bytes_for(c, s) <= kSmemLimit) fit = s;
    if (c.scale_mode == TESSERAE_SCALE_NVFP4 && fit > nvfp4_max_stages(c.block_n)) fit = nvfp4_max_stages(c.block_n);
    if (fit < 2) { if (msg) *msg = "InvalidPipeline: tile does not fit shared memory"; return spec::InvalidPipeline; }
    c.stages = (ks.stages > 0 && ks.stages < fit) ? ks.stages : fit;
    if (c.stages < 1) c.stages = 1;
    c.smem_bytes = smem_bytes_for(c, c.stages);
    *cfg = c;
    return spec::LowerOk;
}

BackendOutput emit(const KernelConfig& c) {
    BackendOutput o;
    o.filename = c.name + ".cuh";
    const bool fp8 = c.elem == TESSERAE_F8E4M3;
    const bool s8 = c.elem == TESSERAE_S8;
    char buf[2048];
    snprintf(buf, sizeof buf,
             "// %s — generated by the tesserae_b200 backend for sm_100a.\n"
             "// descriptor: family=Blackwell bm=%d bn=%d bk=%d elem=%s swizzle=Swizzle<%d,%d,%d>\n"
             "//   TileIO strategy=TmaPair (per-CTA TMA loads feeding a cta_group::%d MMA)\n"
             "//   pipeline depth=%d (reference default 4) tile_bytes=%lld cluster=__cluster_dims__(%d, 1, 1) via launch attribute\n"
             "//   block=%d threads, dynamic smem=%d bytes, sm_count=%d\n"
             "// #pragma once\n"
             "#define TS_KERNEL_NAME %s\n"
             "#define TS_CTA_GROUP %d\n"
             "#define TS_BLOCK_N %d\n"
             "#define TS_STAGES %d\n"
             "#define TS_ELEM_BYTES %d\n"
             "#define TS_MMA_KIND %s\n"
             "#define TS_AB_FMT %s\n"
             "#define TS_OUT_F32 %d\n"
             "#define TS_HAS_BIAS %d\n"
             "#define TS_PROMO_WARPS %d\n"
             "#define TS_SWIZZLE_B %d\n",
             o.filename.c_str(), c.block_m, c.block_n, c.block_k, spec::elem_name(c.elem), c.desc.swizzle.b,
             c.desc.swizzle.m, c.desc.swizzle.s, c.cta_group, c.stages, (long long)c.desc.pipeline.tile_bytes,
             c.cta_group, c.threads, c.smem_bytes, c.desc.sm_count, c.name.c_str(), c.cta_group, c.block_n, c.stages,
             (fp8 || s8) ? 1 : 2, fp8 ? "TS_KIND_F8F6F4" : s8 ? "TS_KIND_I8" : "TS_KIND_F16",
             fp8 ? "TS_FMT_E4M3" : s8 ? "TS_FMT_S8" : (c.elem == TESSERAE_F16 ? "TS_FMT_F16" : "TS_FMT_BF16"),
             c.out_elem == TESSERAE_F32 ? 1 : 0, c.has_bias, c.promo_warps ? c.promo_warps : 8, c.desc.swizzle.b);
    o.includes = buf;
    if (c.scatter) o.includes += "#define TS_SCATTER " + std::to_string(c.scatter) + "\n";
    if (c.grouped) o.includes += "#define TS_GROUPED 1\n";
    if (c.clc) o.includes += "#define TS_CLC 1\n";
    if (c.scale_mode == TESSERAE_SCALE_FP8_BLOCK && c.tail_splits >= 2) o.includes += "#define TS_FP8_TAIL 1\n";
    if (c.scale_mode == TESSERAE_SCALE_NONE) o.includes += "#define TS_STORE_BUFS " + std::to_string(c.store_bufs) + "\n";
    if (c.scale_mode == TESSERAE_SCALE_FP8_BLOCK) {
        o.includes += std::string("#define TS_FP8_SPLIT ") + (c.fp8_split ? "1\n" : "0\n");
    }
    o.includes += "// raster group height: " + (c.group_m > 0 ? std::to_string(c.group_m) + " M-tiles (from the spec)" : std::string("chosen per launch")) + "\n";
    o.helpers = strip_pragma_once(kSrcPtxSm100);
    const bool block_fp8 = c.scale_mode == TESSERAE_SCALE_FP8_BLOCK;
    const bool nvfp4 = c.scale_mode == TESSERAE_SCALE_NVFP4;
    const std::string body = strip_pragma_once(block_fp8 ? kSrcGemmFp8Block : nvfp4 ? kSrcGemmNvfp4 : kSrcGemmDense);
    o.shared_storage = slice(body, block_fp8 ? "namespace ts_fp8 {" : nvfp4 ? "namespace ts_nvfp4 {" : "namespace ts_dense {",
                             "extern \"C\" __global__");
    o.producer_body = slice(body, "------ TMA producer", "------ MMA issuer");
    o.consumer_body = slice(body, "------ MMA issuer", block_fp8 ? "------ promotion + epilogue" : "------ epilogue (warps");
    o.epilogue_body = slice(body, block_fp8 ? "------ promotion + epilogue" : "------ epilogue (warps", "------ teardown");
    o.kernel_func = slice(body, "extern \"C\" __global__", nullptr);
    snprintf(buf, sizeof buf,
             "// Host launch (what tesserae_gemm_run does; the reference's launcher text is\n"
             "// lib/backend/backend_cute.ml:368-429, cudaLaunchKernelEx with a cluster attribute):\n"
             "//   grid  = (%d * min(tiles, resident clusters), 1, 1)   tiles = ceil(M/%d) * ceil(N/%d)\n"
             "//   block = (%d, 1, 1)   cluster = (%d, 1, 1)   dynamic smem = %d\n"
             "//   args  = A_tmap, B_tmap, C_tmap (CUtensorMap by value), %sbias, alpha, M, N, K, group_m, %sstatus\n"
             "//   tesserae_launch_kernel_ex(fn, grid, block, cluster, %d, stream, args, %d);\n",
             c.cta_group, c.block_m * c.cta_group, c.block_n, c.threads, c.cta_group, c.smem_bytes,
             block_fp8 ? "WS_tmap, scale_a, scale_b, " : nvfp4 ? "SFA_tmap, SFB_tmap, " : "", block_fp8 ? "full_tiles, tail_splits, " : "",
             c.smem_bytes, block_fp8 ? 15 : nvfp4 ? 12 : 10);
    o.host_launcher = buf;
    o.full_source = o.includes + o.helpers + "\n" + body + "\n" + o.host_launcher;
    return o;
}

}  // namespace tesserae
