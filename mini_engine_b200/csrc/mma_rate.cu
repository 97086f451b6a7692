// The tensor pipe alone: cycles per tcgen05.mma of K = 16 when a CTA (or a CTA pair) does nothing but
// issue them on operands that lie in shared or tensor memory (zeros; nothing is loaded or stored
// meanwhile).  A measuring tool for `python -m mini_engine_b200.cli.kernel_bench mma-rate`, not part
// of any model step: it says what an MMA costs when nothing competes for shared memory, against which
// the product and attention kernels' own k blocks are read.
#include "tcgen05.cuh"

__device__ __forceinline__ void tcgen05_mma_bf16_ts_pair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8, %9, %10, %11, %12}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u), "r"(0u),
          "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// mode: 0 SS one CTA, 1 TS one CTA, 2 SS pair, 3 TS pair.  B K-major unless mn != 0.
template <int MODE, int N, int MN>
__global__ void __launch_bounds__(128) mma_rate_kernel(long long* out, int iters) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* a_tile = tiles;              // 128 rows x 64
    uint8_t* b_tile = tiles + 16384;      // up to 256 rows x 64
    uint64_t* bar = reinterpret_cast<uint64_t*>(tiles + 16384 + 32768);
    uint32_t* holder = reinterpret_cast<uint32_t*>(bar + 2);
    constexpr bool PAIR = MODE >= 2, TS = (MODE & 1) != 0;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0;
    for (int i = threadIdx.x; i < (16384 + 32768) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(tiles)[i] = 0;
    if (threadIdx.x == 0) { mbar_init(bar, 1); asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (threadIdx.x < 32) { if (PAIR) tcgen05_alloc_pair(holder, 512); else tcgen05_alloc(holder, 512); }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync();
    tcgen05_fence_after();
    const uint32_t tmem = *holder;
    if (threadIdx.x == 0 && rank == 0) {
        const uint32_t idesc = PAIR ? (make_idesc_pair(N) | (MN ? (1u << 16) : 0u)) : make_idesc(N, MN != 0);
        const uint64_t a_desc = smem_desc_sw128(smem_u32(a_tile));
        const uint64_t b_desc = MN ? smem_desc_sw128_mn(smem_u32(b_tile), 16384) : smem_desc_sw128(smem_u32(b_tile));
        const long long t0 = clock64();
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint64_t step = MN ? static_cast<uint64_t>((k * 16 * 128) >> 4) : static_cast<uint64_t>((k * 32) >> 4);
                if (PAIR) {
                    if (TS) tcgen05_mma_bf16_ts_pair(tmem, tmem + 256 + k * 8, b_desc + step, idesc, 1u);
                    else tcgen05_mma_bf16_pair(tmem, a_desc + (k * 32 >> 4), b_desc + step, idesc, 1u);
                } else {
                    if (TS) tcgen05_mma_bf16_ts(tmem, tmem + 256 + k * 8, b_desc + step, idesc, 1u);
                    else tcgen05_mma_bf16(tmem, a_desc + (k * 32 >> 4), b_desc + step, idesc, 1u);
                }
            }
        }
        if (PAIR) tcgen05_commit_pair(bar); else tcgen05_commit(bar);
        const bool ok = mbar_wait(bar, 0);
        const long long t1 = clock64();
        if (blockIdx.x == 0) out[0] = ok ? (t1 - t0) : -1;  // -1: the wait ran out
    } else if (threadIdx.x == 0 && PAIR) {
        mbar_wait(bar, 0);  // the commit arrives in both CTAs
    }
    tcgen05_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync();
    if (threadIdx.x < 32) { if (PAIR) tcgen05_dealloc_pair(tmem, 512); else tcgen05_dealloc(tmem, 512); }
}


template <int MODE, int N, int MN>
static int launch_rate(long long* cycles, int ctas, int iters, cudaStream_t stream) {
    constexpr int SMEM = 16384 + 32768 + 1024 + 256;
    auto kernel = mma_rate_kernel<MODE, N, MN>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, SMEM)) return e;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(ctas);
    config.blockDim = dim3(128);
    config.dynamicSmemBytes = SMEM;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = MODE >= 2 ? 2 : 1;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    return static_cast<int>(cudaLaunchKernelEx(&config, kernel, cycles, iters));
}

// `cycles` (device, one int64) receives the cycles that CTA 0 needed for 4 * iters MMAs of
// M = 128 (256 for a pair), N = n, K = 16, or -1 when its bounded wait ran out.
// pair: 0 one CTA, 1 a CTA pair (cta_group::2; ctas must be even); a_in_tensor_memory: 0 / 1;
// b_mn_major: the second operand's rows run along the reduction (as values do in attention).
ME_EXPORT int me_mma_rate(long long* cycles, int pair, int a_in_tensor_memory, int b_mn_major, int n, int ctas, int iters,
                          cudaStream_t stream) {
    if (ctas < 1 || iters < 1 || (pair && ctas % 2)) return ME_ERR_ARGUMENT;
    const int mode = (pair ? 2 : 0) + (a_in_tensor_memory ? 1 : 0);
#define ME_RATE_CASE(MODE, N, MN) \
    if (mode == MODE && n == N && (b_mn_major != 0) == (MN != 0)) return launch_rate<MODE, N, MN>(cycles, ctas, iters, stream);
    ME_RATE_CASE(0, 64, 0) ME_RATE_CASE(0, 128, 0) ME_RATE_CASE(0, 256, 0) ME_RATE_CASE(1, 128, 1) ME_RATE_CASE(1, 128, 0)
    ME_RATE_CASE(2, 64, 0) ME_RATE_CASE(2, 128, 0) ME_RATE_CASE(2, 256, 0) ME_RATE_CASE(3, 128, 1) ME_RATE_CASE(3, 128, 0)
#undef ME_RATE_CASE
    return ME_ERR_UNSUPPORTED;
}
