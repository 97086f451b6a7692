// y[t][n] = sum_k x[t][k] * w[n][k] on CUDA cores, for any sizes.
//
// This is the true 32-bit matrix product of the float32 path (no tensor cores, no TF32) and
// the fallback of the bfloat16 path for shapes that TMA cannot address.  Every output element
// is one accumulator updated with fmaf for k = 0, 1, 2, ... in ascending order, so a row's
// result is bit-identical whatever other rows share the launch: splitting a prompt into
// portions or batching it with other requests cannot change a single bit.
//
// The weight keeps the checkpoint's [out, in] layout (torch Linear,
// src/mini_engine/model.py:97-100 of YuvGev00/mini-engine).
#include "common.cuh"

constexpr int TILE_T = 64;   // tokens per block
constexpr int TILE_N = 64;   // outputs per block
constexpr int TILE_K = 16;
constexpr int SIMT_THREADS = 256;  // 16 x 16 threads, each 4 x 4 outputs

template <typename T>
__global__ void __launch_bounds__(SIMT_THREADS)
gemm_simt_kernel(const T* __restrict__ x, const T* __restrict__ w, float* __restrict__ y, int tokens,
                 int outs, int inner) {
    __shared__ float xs[TILE_K][TILE_T + 4];
    __shared__ float ws[TILE_K][TILE_N + 4];
    const int t0 = blockIdx.y * TILE_T, n0 = blockIdx.x * TILE_N;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    pdl_trigger();
    pdl_wait();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = 0; k0 < inner; k0 += TILE_K) {
#pragma unroll
        for (int r = 0; r < (TILE_T * TILE_K) / SIMT_THREADS; ++r) {
            const int idx = threadIdx.x + r * SIMT_THREADS;
            const int row = idx / TILE_K, kk = idx % TILE_K;
            const int t = t0 + row, n = n0 + row, k = k0 + kk;
            xs[kk][row] = (t < tokens && k < inner) ? to_float(x[static_cast<size_t>(t) * inner + k]) : 0.0f;
            ws[kk][row] = (n < outs && k < inner) ? to_float(w[static_cast<size_t>(n) * inner + k]) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TILE_K; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = t0 + ty * 4 + i;
        if (t >= tokens) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < outs) y[static_cast<size_t>(t) * outs + n] = acc[i][j];
        }
    }
}

ME_EXPORT int me_gemm_simt(const void* x, const void* w, float* y, int type, int tokens, int outs, int inner,
                           cudaStream_t stream) {
    if (tokens <= 0 || outs <= 0) return 0;
    dim3 grid((outs + TILE_N - 1) / TILE_N, (tokens + TILE_T - 1) / TILE_T);
    if (grid.y > 65535) return ME_ERR_UNSUPPORTED;
    if (type == ME_BF16)
        return launch_kernel(gemm_simt_kernel<__nv_bfloat16>, grid, SIMT_THREADS, 0, stream,
                             static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w), y, tokens, outs,
                             inner);
    return launch_kernel(gemm_simt_kernel<float>, grid, SIMT_THREADS, 0, stream, static_cast<const float*>(x),
                         static_cast<const float*>(w), y, tokens, outs, inner);
}
