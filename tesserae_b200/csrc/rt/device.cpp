// Device buffers, module load, kernel launch, tensor maps.
//
// Plain-C counterparts of the reference's OCaml stubs:
//   lib/runtime/gpu_buffer_stubs.c:26-83   caml_gpu_alloc / free / copy_to_device / copy_to_host / ptr
//   lib/kernel/kernel_launch_stubs.c:21-107 caml_cuinit / module_load_ptx / module_unload / get_function /
//                                           launch_kernel / device_synchronize / device_info
// plus what a tcgen05/TMA kernel needs and the reference's launch stub cannot express:
// cuLaunchKernelEx with cluster dimensions, arguments larger than 8 bytes (a tensor map is
// 128 bytes, passed by value), an explicit stream, and tensor-map encoding.
#include "../../../include/tesserae_b200.h"
#include "driver_api.hpp"
#include "errors.hpp"

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <vector>

using tesserae::driver_api;
using tesserae::driver_error;
using tesserae::DriverApi;
using tesserae::fail;

namespace tesserae {

// Binds the runtime API's primary context of the current device to this thread so that
// driver calls (module load, launch) act on the same context as cudaMalloc and torch.
const DriverApi* driver_with_context(std::string* err) {
    const DriverApi* api = driver_api(err);
    if (!api) return nullptr;
    CUcontext ctx = nullptr;
    api->cuCtxGetCurrent(&ctx);
    if (!ctx) {
        cudaError_t rc = cudaFree(nullptr);   // creates / binds the primary context
        if (rc != cudaSuccess) { if (err) *err = std::string("CUDA context: ") + cudaGetErrorString(rc); return nullptr; }
    }
    return api;
}

int elem_tensor_map_type(int elem, CUtensorMapDataType* t) {
    switch (elem) {
        case TESSERAE_F16: *t = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; return 0;
        case TESSERAE_BF16: *t = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; return 0;
        case TESSERAE_F32: *t = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; return 0;
        case TESSERAE_S32: *t = CU_TENSOR_MAP_DATA_TYPE_INT32; return 0;
        case TESSERAE_S8:
        case TESSERAE_F8E4M3:
        case TESSERAE_F4E2M1:   // two E2M1 values per byte, addressed as bytes
            *t = CU_TENSOR_MAP_DATA_TYPE_UINT8; return 0;
        default: return -1;
    }
}

}  // namespace tesserae

extern "C" {

// ------------------------------------------------------------------ buffers
int tesserae_gpu_alloc(size_t n_bytes, void** dptr) {
    if (!dptr) return fail("gpu_alloc: null out pointer");
    *dptr = nullptr;
    void* p = nullptr;
    cudaError_t rc = cudaMalloc(&p, n_bytes ? n_bytes : 1);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    rc = cudaMemset(p, 0, n_bytes);
    if (rc != cudaSuccess) { cudaFree(p); return fail(cudaGetErrorString(rc)); }
    *dptr = p;
    return 0;
}

int tesserae_gpu_free(void* dptr) {
    if (!dptr) return 0;
    cudaError_t rc = cudaFree(dptr);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    return 0;
}

int tesserae_gpu_copy_to_device(void* dptr, const void* src, size_t n_bytes) {
    cudaError_t rc = cudaMemcpy(dptr, src, n_bytes, cudaMemcpyHostToDevice);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    return 0;
}

int tesserae_gpu_copy_to_host(void* dst, const void* dptr, size_t n_bytes) {
    cudaError_t rc = cudaMemcpy(dst, dptr, n_bytes, cudaMemcpyDeviceToHost);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    return 0;
}

// ------------------------------------------------------------------ modules
int tesserae_cuinit(void) {
    std::string err;
    if (!driver_api(&err)) return fail(err);
    return 0;
}

int tesserae_set_device(int device) {
    cudaError_t rc = cudaSetDevice(device);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    return 0;
}

int tesserae_module_load(const void* image, void** module) {
    if (!image || !module) return fail("module_load: null argument");
    std::string err;
    const DriverApi* api = tesserae::driver_with_context(&err);
    if (!api) return fail(err);
    CUmodule mod = nullptr;
    CUresult rc = api->cuModuleLoadData(&mod, image);
    if (rc != CUDA_SUCCESS) return fail(driver_error(api, "cuModuleLoadData", rc));
    *module = mod;
    return 0;
}

int tesserae_module_unload(void* module) {
    if (!module) return 0;
    std::string err;
    const DriverApi* api = driver_api(&err);
    if (!api) return fail(err);
    CUresult rc = api->cuModuleUnload(static_cast<CUmodule>(module));
    if (rc != CUDA_SUCCESS) return fail(driver_error(api, "cuModuleUnload", rc));
    return 0;
}

int tesserae_get_function(void* module, const char* name, void** function) {
    if (!module || !name || !function) return fail("get_function: null argument");
    std::string err;
    const DriverApi* api = driver_api(&err);
    if (!api) return fail(err);
    CUfunction fn = nullptr;
    CUresult rc = api->cuModuleGetFunction(&fn, static_cast<CUmodule>(module), name);
    if (rc != CUDA_SUCCESS) return fail(driver_error(api, "cuModuleGetFunction", rc));
    *function = fn;
    return 0;
}

int tesserae_launch_kernel(void* function, int gx, int gy, int gz, int bx, int by, int bz,
                           int smem_bytes, const int64_t* args, int n_args) {
    if (!function) return fail("launch_kernel: null function");
    std::string err;
    const DriverApi* api = tesserae::driver_with_context(&err);
    if (!api) return fail(err);
    std::vector<int64_t> vals(args, args + (n_args > 0 ? n_args : 0));
    std::vector<void*> params(vals.size());
    for (size_t i = 0; i < vals.size(); ++i) params[i] = &vals[i];
    CUresult rc = api->cuLaunchKernel(static_cast<CUfunction>(function), gx, gy, gz, bx, by, bz, smem_bytes,
                                      nullptr, params.empty() ? nullptr : params.data(), nullptr);
    if (rc != CUDA_SUCCESS) return fail(driver_error(api, "cuLaunchKernel", rc));
    return 0;
}

int tesserae_launch_kernel_ex(void* function, const int grid[3], const int block[3], const int cluster[3],
                              int smem_bytes, void* stream, const tesserae_launch_arg* args, int n_args) {
    if (!function || !grid || !block) return fail("launch_kernel_ex: null argument");
    std::string err;
    const DriverApi* api = tesserae::driver_with_context(&err);
    if (!api) return fail(err);
    std::vector<void*> params(n_args > 0 ? n_args : 0);
    for (int i = 0; i < n_args; ++i) params[i] = const_cast<void*>(args[i].data);
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = grid[0]; cfg.gridDimY = grid[1]; cfg.gridDimZ = grid[2];
    cfg.blockDimX = block[0]; cfg.blockDimY = block[1]; cfg.blockDimZ = block[2];
    cfg.sharedMemBytes = smem_bytes;
    cfg.hStream = static_cast<CUstream>(stream);
    CUlaunchAttribute attr[1];
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (cluster && cluster[0] * cluster[1] * cluster[2] > 1) {
        attr[0].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attr[0].value.clusterDim.x = cluster[0];
        attr[0].value.clusterDim.y = cluster[1];
        attr[0].value.clusterDim.z = cluster[2];
        cfg.numAttrs = 1;
    }
    // More than 48 KB of dynamic shared memory needs the function's opt-in; a caller that got the function from
    // tesserae_get_function has no other way to give it.  (Plans set it once at creation.)
    if (smem_bytes > 48 * 1024) {
        static thread_local void* opted_fn = nullptr;
        static thread_local int opted_bytes = 0;
        if (opted_fn != function || opted_bytes < smem_bytes) {
            CUresult arc = api->cuFuncSetAttribute(static_cast<CUfunction>(function),
                                                   CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem_bytes);
            if (arc != CUDA_SUCCESS) return fail(driver_error(api, "cuFuncSetAttribute(max dynamic smem)", arc));
            opted_fn = function; opted_bytes = smem_bytes;
        }
    }
    CUresult rc = api->cuLaunchKernelEx(&cfg, static_cast<CUfunction>(function),
                                        params.empty() ? nullptr : params.data(), nullptr);
    if (rc != CUDA_SUCCESS) return fail(driver_error(api, "cuLaunchKernelEx", rc));
    return 0;
}

int tesserae_device_synchronize(void) {
    cudaError_t rc = cudaDeviceSynchronize();
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    return 0;
}

int tesserae_device_info(char* buf, size_t buf_size) {
    if (!buf || buf_size == 0) return fail("device_info: null buffer");
    cudaDeviceProp prop;
    cudaError_t rc = cudaGetDeviceProperties(&prop, 0);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    snprintf(buf, buf_size, "%s (sm_%d%d)", prop.name, prop.major, prop.minor);
    return 0;
}

int tesserae_device_sm_count(int* sm_count) {
    int dev = 0, n = 0;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc == cudaSuccess) rc = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (rc != cudaSuccess) return fail(cudaGetErrorString(rc));
    if (sm_count) *sm_count = n;
    return 0;
}

int tesserae_runtime_is_available(void) {
    std::string err;
    if (!driver_api(&err)) return 0;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n > 0 ? 1 : 0;
}

// ------------------------------------------------------------------ tensor maps
int tesserae_tensor_map_2d(void* out_map128, int elem, const void* gptr, uint64_t inner, uint64_t outer,
                           uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer, int swizzle_b) {
    if (!out_map128 || !gptr) return fail("tensor_map_2d: null argument");
    std::string err;
    const DriverApi* api = driver_api(&err);
    if (!api) return fail(err);
    CUtensorMapDataType dt;
    if (tesserae::elem_tensor_map_type(elem, &dt) != 0) return fail("tensor_map_2d: unsupported element type");
    if ((reinterpret_cast<uintptr_t>(gptr) & 15u) != 0) return fail("tensor_map_2d: base address must be 16-byte aligned");
    if (row_stride_bytes % 16 != 0) return fail("tensor_map_2d: row stride must be a multiple of 16 bytes");
    if (box_inner == 0 || box_outer == 0 || box_inner > 256 || box_outer > 256) return fail("tensor_map_2d: box extents must be in 1..256");
    static const CUtensorMapSwizzle kSwizzle[4] = {CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_SWIZZLE_32B,
                                                   CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_SWIZZLE_128B};
    if (swizzle_b < 0 || swizzle_b > 3) return fail("tensor_map_2d: swizzle_b must be 0..3");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMap tm;
    CUresult rc = api->cuTensorMapEncodeTiled(&tm, dt, 2, const_cast<void*>(gptr), dims, strides, box, estr,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, kSwizzle[swizzle_b],
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) return fail(driver_error(api, "cuTensorMapEncodeTiled", rc));
    memcpy(out_map128, &tm, sizeof tm);
    return 0;
}

}  // extern "C"
