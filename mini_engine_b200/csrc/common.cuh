// Shared helpers of the CUDA sources: element conversion, warp reductions, launch checks.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ME_EXPORT extern "C" __attribute__((visibility("default")))

// Element type codes shared with the Python bindings.
enum : int { ME_F32 = 0, ME_BF16 = 1 };

// Error codes returned by launchers beside cudaError_t values (which are < 1000).
enum : int { ME_ERR_UNSUPPORTED = 1001, ME_ERR_ARGUMENT = 1002 };

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Butterfly reductions: every lane ends with the same value, formed in the same order
// whatever the data, so a row's statistics never depend on its neighbours in the batch.
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

static inline int launch_status() { return static_cast<int>(cudaGetLastError()); }

// Programmatic dependent launch.  Every kernel of this package is launched with the attribute
// that lets its CTAs become resident while the kernel before it in the stream is still running.
// Such a CTA may only set itself up and read weights (which no kernel writes); before it reads
// or writes anything that another kernel writes or reads it calls pdl_wait(), which returns once
// the preceding kernel has completed and its memory is visible.  pdl_trigger() tells the
// scheduler that the next kernel's CTAs may be made resident as far as this CTA is concerned.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// A kernel's opt-in to more than 48 KB of dynamic shared memory holds for one device only, so it
// is remembered per device ordinal (the device that is current when the kernel is launched).
struct SharedMemoryOptIn {
    bool done[64] = {};
    template <typename Kernel>
    int operator()(Kernel kernel, int bytes) {
        int device = 0;
        cudaError_t e = cudaGetDevice(&device);
        if (e != cudaSuccess) return static_cast<int>(e);
        const bool remembered = device >= 0 && device < 64;
        if (remembered && done[device]) return 0;
        e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return static_cast<int>(e);
        if (remembered) done[device] = true;
        return 0;
    }
};

template <typename... KernelArgs, typename... Args>
static inline int launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...));
}
