// Kernel configuration derived from a spec, and the source emitter.
#pragma once
#include "../../../include/tesserae_b200.h"
#include "../spec/tesserae_spec.hpp"

#include <string>
#include <vector>

namespace tesserae {

// Everything the device source is specialised on (the TS_* macros) and the launch needs.
struct KernelConfig {
    std::string name;        // extern "C" symbol
    int elem = TESSERAE_BF16;
    int out_elem = TESSERAE_F32;
    int cta_group = 2;
    int block_m = 128;       // rows per CTA
    int block_n = 256;       // tile width = MMA N
    int block_k = 64;        // K elements per stage (128 bytes)
    int stages = 4;
    int has_bias = 0;
    int scale_mode = TESSERAE_SCALE_NONE;
    int scatter = 0;         // row-scattered output (dense kernel only): 1 stored to per-source slots, 2 added into the owner's buffer
    int tail_splits = 0;     // FP8 block-scaled, stream-K tail: 0 = the host chooses per launch, 1 = never, n = at most n K ranges per tail tile
    int clc = 0;             // dense kernels: tile order by cluster launch control (scheduler warp) instead of the static walk
    int grouped = 0;         // the kernel walks a table of problems instead of one problem's tiles (dense kernel only)
    int promo_warps = 0;     // promotion warps of the FP8 block-scaled kernel (0 elsewhere)
    int store_bufs = 2;      // dense kernel: staging buffers per epilogue warp (4 when the stores cross NVLink)
    int group_m = 0;         // M-tiles per raster group of the persistent tile order; 0 = sized per launch from M and K
    int fp8_split = 1;       // FP8 block-scaled: 1 = one MMA chain and TMEM buffer per 128 columns, 0 = per tile width
    int b_box_rows = 128;    // rows of B one TMA load brings (the FP8 block-scaled pair kernel loads B per 128-column MMA group)
    int threads = 192;
    int smem_bytes = 0;      // dynamic shared memory to request
    spec::KernelDesc desc;   // the reference-shaped descriptor it was lowered from
};

// Lower.lower + the choices the reference hard-codes or leaves open (stage count by
// shared-memory fit, CTA pair or single CTA).  Returns a TESSERAE_LOWER_* code.
int derive_config(const tesserae_kernel_spec& spec, KernelConfig* cfg, std::string* msg);

struct BackendOutput {
    std::string filename, includes, helpers, shared_storage, producer_body, consumer_body, epilogue_body,
        kernel_func, host_launcher, full_source;
};
// Backend_cute.emit for the Blackwell family.
BackendOutput emit(const KernelConfig& cfg);

// NVRTC options every kernel of this backend is compiled with.
std::vector<std::string> nvrtc_options();

// Device source texts, embedded at build time from csrc/kernels/*.cuh.
extern const char* const kSrcPtxSm100;
extern const char* const kSrcGemmDense;
extern const char* const kSrcGemmFp8Block;
extern const char* const kSrcGemmNvfp4;

}  // namespace tesserae
