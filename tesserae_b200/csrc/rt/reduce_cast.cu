// Sum of fp32 partial products and cast to bf16: the step that follows the K-split GEMM (each
// K slice leaves an fp32 partial C; after the reduce-scatter between GPUs, or directly on one
// GPU, the partials are added and rounded to bf16 once).  HBM-bound: per output element it
// reads 4 bytes per partial and writes 2.  The reference has no counterpart (its C is always
// fp32, lib/kernel/kernel_desc.ml:218-220, and nothing is split).
#include "../../../include/tesserae_b200.h"
#include "errors.hpp"

#include <cuda_runtime.h>
#include <cstdint>
#include <string>

using tesserae::fail;

namespace {

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// Each thread handles 8 consecutive elements per step (two 16-byte loads per partial, one 16-byte store).
__global__ void __launch_bounds__(256) reduce_cast_kernel(const float* __restrict__ parts, int n_parts, size_t part_stride,
                                                          float alpha, uint16_t* __restrict__ out, size_t n) {
    const size_t n8 = n / 8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        float4 a = __ldcs(reinterpret_cast<const float4*>(parts) + 2 * i);
        float4 b = __ldcs(reinterpret_cast<const float4*>(parts) + 2 * i + 1);
        for (int p = 1; p < n_parts; ++p) {
            const float4* q = reinterpret_cast<const float4*>(parts + (size_t)p * part_stride) + 2 * i;
            const float4 c = __ldcs(q), d = __ldcs(q + 1);
            a.x += c.x; a.y += c.y; a.z += c.z; a.w += c.w;
            b.x += d.x; b.y += d.y; b.z += d.z; b.w += d.w;
        }
        uint4 o;
        o.x = pack_bf16x2(alpha * a.x, alpha * a.y); o.y = pack_bf16x2(alpha * a.z, alpha * a.w);
        o.z = pack_bf16x2(alpha * b.x, alpha * b.y); o.w = pack_bf16x2(alpha * b.z, alpha * b.w);
        reinterpret_cast<uint4*>(out)[i] = o;
    }
    // tail (n not a multiple of 8)
    const size_t t = n8 * 8 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) {
        float s = parts[t];
        for (int p = 1; p < n_parts; ++p) s += parts[(size_t)p * part_stride + t];
        out[t] = (uint16_t)(pack_bf16x2(alpha * s, 0.f) & 0xFFFFu);
    }
}

// out = bf16(alpha * acc) and acc = 0 in one pass: the step after the adding K-split epilogue, whose accumulation
// buffer must hold zeros again before its next use.  Reads 4 bytes, writes 2 + 4 per element.
// A warp's lanes take consecutive 16-byte pieces, so that every load and every store covers whole 32-byte sectors
// (a thread that takes 32 consecutive bytes as two 16-byte accesses half-fills the sectors of each instruction; for
// the stores of zeros that measured 1.7 TB/s against 5.8 for the same bytes laid out this way), and four loads are
// in flight per thread before the first store.
__global__ void __launch_bounds__(256) cast_clear_kernel(float* __restrict__ acc, float alpha, uint16_t* __restrict__ out, size_t n) {
    constexpr int kBatch = 4;
    const size_t n4 = n / 4;
    const size_t threads = (size_t)gridDim.x * blockDim.x;
    float4* acc4 = reinterpret_cast<float4*>(acc);
    uint2* out2 = reinterpret_cast<uint2*>(out);
    const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
    for (size_t base = (size_t)blockIdx.x * blockDim.x + threadIdx.x; base < n4; base += threads * kBatch) {
        float4 v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const size_t i = base + (size_t)u * threads;
            if (i < n4) v[u] = __ldcs(acc4 + i);
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
            const size_t i = base + (size_t)u * threads;
            if (i < n4) {
                acc4[i] = zero;
                out2[i] = make_uint2(pack_bf16x2(alpha * v[u].x, alpha * v[u].y), pack_bf16x2(alpha * v[u].z, alpha * v[u].w));
            }
        }
    }
    const size_t t = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (t < n) {
        out[t] = (uint16_t)(pack_bf16x2(alpha * acc[t], 0.f) & 0xFFFFu);
        acc[t] = 0.f;
    }
}

}  // namespace

extern "C" int tesserae_cast_clear_bf16(void* acc_f32, float alpha, void* out_bf16, size_t n_elems, void* stream) {
    if (!acc_f32 || !out_bf16) return fail("cast_clear: null argument");
    if (n_elems == 0) return 0;
    if ((reinterpret_cast<uintptr_t>(acc_f32) & 15u) || (reinterpret_cast<uintptr_t>(out_bf16) & 15u))
        return fail("cast_clear: buffers must be 16-byte aligned");
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t want = (n_elems / 16 + 255) / 256 + 1;
    const size_t cap = (size_t)sms * 8;
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    cast_clear_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<float*>(acc_f32), alpha,
                                                                           static_cast<uint16_t*>(out_bf16), n_elems);
    cudaError_t rc = cudaGetLastError();
    if (rc != cudaSuccess) return fail(std::string("cast_clear launch: ") + cudaGetErrorString(rc));
    return 0;
}

extern "C" int tesserae_reduce_cast_bf16(const void* parts, int n_parts, size_t part_stride_elems, float alpha,
                                         void* out_bf16, size_t n_elems, void* stream) {
    if (!parts || !out_bf16) return fail("reduce_cast: null argument");
    if (n_parts < 1) return fail("reduce_cast: n_parts must be >= 1");
    if (n_elems == 0) return 0;
    if ((reinterpret_cast<uintptr_t>(parts) & 15u) || (reinterpret_cast<uintptr_t>(out_bf16) & 15u) ||
        (n_parts > 1 && (part_stride_elems % 4) != 0))
        return fail("reduce_cast: buffers must be 16-byte aligned and the partial stride a multiple of 4 elements");
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t want = (n_elems / 8 + 255) / 256 + 1;
    const size_t cap = (size_t)sms * 8;                       // 8 resident blocks of 256 threads per SM
    const unsigned grid = (unsigned)(want < cap ? want : cap);
    reduce_cast_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const float*>(parts), n_parts, part_stride_elems, alpha, static_cast<uint16_t*>(out_bf16), n_elems);
    cudaError_t rc = cudaGetLastError();
    if (rc != cudaSuccess) return fail(std::string("reduce_cast launch: ") + cudaGetErrorString(rc));
    return 0;
}
