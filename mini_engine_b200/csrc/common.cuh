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
