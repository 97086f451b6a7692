// y = x W^T in bfloat16 on the 5th-generation tensor cores of sm_100a: TMA loads into
// 128-byte-swizzled shared memory, tcgen05.mma with the accumulator in tensor memory,
// tcgen05.ld for the epilogue.
//
// Orientation.  The weight W [out, in] (the checkpoint's layout, src/mini_engine/model.py:97-100
// of YuvGev00/mini-engine) is the 128-row A operand; the tokens x [T, in] are the B operand
// with N = BLOCK_T in {16, ..., 256}.  The accumulator D[out row][token] therefore has one
// output feature per TMEM lane and one token per column, and the same kernel serves a
// 2,048-token prompt (BLOCK_T = 256) and a single decoded token (BLOCK_T = 16), where it
// streams the weight through shared memory at the rate of HBM.
//
// Work split.  grid = (token tiles, out tiles, k splits).  With few tokens there are too few
// output tiles to occupy 148 SMs, so the reduction axis is cut into `splits` ranges of 64-wide
// k blocks; split s writes its partial sum to out[s][T][out] and the consumer kernel adds the
// partials in ascending s.  Nothing is added atomically: results are reproducible.
//
// Roles (192 threads): warp 0 issues TMA loads, warp 1 allocates tensor memory and issues the
// MMAs, warps 2-5 read the accumulator (each warp its own 32 lanes) and store.  Stages are
// handed over with mbarriers: full[s] (TMA bytes arrived), empty[s] (tcgen05.commit: the MMAs
// that read stage s retired), accum (all MMAs retired).
//
// DUAL mode computes silu(x Wg^T) * (x Wu^T) (src/mini_engine/model.py:130): Wg and Wu tiles
// of the same 128 output features are loaded side by side, accumulate into two column ranges
// of tensor memory, and the epilogue applies the gate lane by lane, so the [T, 2 * inter]
// intermediate never exists.
//
// Launch overlap: the kernel is launched as a programmatic dependent of the kernel before it.
// Its CTAs become resident while that kernel still runs, set up their barriers and tensor memory
// and already request their first weight tiles (up to 128 KB per CTA); only the activation tiles
// and the stores wait for the predecessor (griddepcontrol.wait).  In a decode step this keeps
// the weight stream from HBM going across kernel boundaries.
//
// Every wait is bounded: after a limit of polls and of time a role records an error code in a device
// flag that the host reads, stops, and the CTA still frees its tensor memory and exits.
#include "tcgen05.cuh"

constexpr int BLOCK_N = 128;  // output features per CTA = UMMA M
constexpr int BLOCK_K = 64;   // one 128-byte swizzle row of bfloat16
constexpr int UMMA_K = 16;
constexpr int GEMM_THREADS = 192;
constexpr int SMEM_BUDGET = 200 * 1024;

__device__ int g_gemm_error = 0;  // 0 ok; else (role << 8) | detail of the first failure seen

// ------------------------------------------------------------------------------ kernel

template <int BLOCK_T, bool DUAL>
struct Config {
    static constexpr int A_BYTES = BLOCK_N * BLOCK_K * 2 * (DUAL ? 2 : 1);
    static constexpr int B_BYTES = BLOCK_T * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // Few tokens: the kernel only streams weights.  Four stages keep a CTA at 72-96 KB of shared
    // memory, so two or three CTAs share an SM and one's start-up and epilogue hide behind the
    // others' loads.  Many tokens: as many stages as fit, one CTA per SM.
    static constexpr int STAGES = BLOCK_T <= 64 ? 4 : ((SMEM_BUDGET / STAGE_BYTES) < 8 ? (SMEM_BUDGET / STAGE_BYTES) : 8);
    static constexpr int ACC_COLUMNS = BLOCK_T * (DUAL ? 2 : 1);
    static constexpr int TMEM_COLUMNS = ACC_COLUMNS < 32 ? 32 : ACC_COLUMNS;  // powers of two here
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

struct GemmParams {
    void* out;            // float [splits][tokens][outs], or bfloat16 [tokens][outs] in DUAL mode
    int tokens, outs, k_blocks, k_blocks_per_split;
    int dual_row_offset;  // row of W where the second (up) half starts
    int token_tiles, full_tiles, tail_parts;  // pair kernels: tiles along the tokens; whole ones; cuts of the rest
    int items;  // persistent pair kernel: whole tiles + parts of cut tiles
    int feature_tiles, group;  // persistent pair kernel: tiles along the features; token tiles of a group (see pair_item)
};

template <int BLOCK_T, bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    using C = Config<BLOCK_T, DUAL>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* accum = empty + C::STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Token tiles vary fastest in the grid: CTAs that run at the same time share a weight tile,
    // which then comes from DRAM once and from L2 for the others.
    const int n0 = blockIdx.y * BLOCK_N, t0 = blockIdx.x * BLOCK_T, split = blockIdx.z;
    const int kb_begin = split * p.k_blocks_per_split;
    const int kb_end = min(kb_begin + p.k_blocks_per_split, p.k_blocks);
    const int iterations = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(tmem_holder, C::TMEM_COLUMNS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        // ------------------------------------------------------------- TMA producer
        if (lane == 0) {
            pdl_trigger();
            // Weights are written by no kernel, so the first stages' weight tiles are requested
            // before the preceding kernel has finished; the activations wait for it.
            const int early = min(iterations, C::STAGES);
            for (int i = 0; i < early; ++i) {
                uint8_t* a_tile = tiles + i * C::STAGE_BYTES;
                mbar_expect_tx(&full[i], C::STAGE_BYTES);
                const int k = (kb_begin + i) * BLOCK_K;
                tma_load_2d(a_tile, &map_w, k, n0, &full[i]);
                if (DUAL) tma_load_2d(a_tile + BLOCK_N * BLOCK_K * 2, &map_w, k, p.dual_row_offset + n0, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(tiles + i * C::STAGE_BYTES + C::A_BYTES, &map_x, (kb_begin + i) * BLOCK_K, t0, &full[i]);
            int issued = early;
            for (int i = early; i < iterations; ++i, ++issued) {
                const int stage = i % C::STAGES;
                const uint32_t parity = (i / C::STAGES) & 1;
                if (!mbar_wait(&empty[stage], parity ^ 1)) { atomicCAS(&g_gemm_error, 0, (1 << 8) | stage); break; }
                uint8_t* a_tile = tiles + stage * C::STAGE_BYTES;
                uint8_t* b_tile = a_tile + C::A_BYTES;
                mbar_expect_tx(&full[stage], C::STAGE_BYTES);
                const int k = (kb_begin + i) * BLOCK_K;
                tma_load_2d(a_tile, &map_w, k, n0, &full[stage]);
                if (DUAL) tma_load_2d(a_tile + BLOCK_N * BLOCK_K * 2, &map_w, k, p.dual_row_offset + n0, &full[stage]);
                tma_load_2d(b_tile, &map_x, k, t0, &full[stage]);
            }
            // Copies still in flight must land before the CTA's shared memory is released.  On
            // the normal path the MMA warp has waited for every one of them already.
            if (issued < iterations || g_gemm_error != 0) {
                for (int i = max(issued - C::STAGES, 0); i < issued; ++i)
                    mbar_wait(&full[i % C::STAGES], (i / C::STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        // --------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BLOCK_T);
            bool ok = true;
            for (int i = 0; i < iterations && ok; ++i) {
                const int stage = i % C::STAGES;
                const uint32_t parity = (i / C::STAGES) & 1;
                if (!mbar_wait(&full[stage], parity)) { atomicCAS(&g_gemm_error, 0, (2 << 8) | stage); ok = false; break; }
                tcgen05_fence_after();
                const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
                const uint32_t b_addr = a_addr + C::A_BYTES;
                const uint64_t a_desc = smem_desc_sw128(a_addr);
                const uint64_t b_desc = smem_desc_sw128(b_addr);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t step = static_cast<uint64_t>((k * UMMA_K * 2) >> 4);  // 32 bytes per k step
                    const uint32_t accumulate = (i > 0 || k > 0) ? 1u : 0u;
                    tcgen05_mma_bf16(tmem_base, a_desc + step, b_desc + step, idesc, accumulate);
                    if (DUAL) {
                        const uint64_t a2_desc = smem_desc_sw128(a_addr + BLOCK_N * BLOCK_K * 2);
                        tcgen05_mma_bf16(tmem_base + BLOCK_T, a2_desc + step, b_desc + step, idesc, accumulate);
                    }
                }
                tcgen05_commit(&empty[stage]);  // arrives when the MMAs above no longer read the stage
            }
            tcgen05_commit(accum);
        }
    } else {
        // ------------------------------------------------------------------ epilogue
        const int quarter = warp & 3;  // a warp may read TMEM lanes [32 * (warp % 4), +32)
        const int n = n0 + quarter * 32 + lane;
        pdl_wait();  // the output buffer may still be read by the kernel before this one
        bool ok = mbar_wait(accum, 0);
        if (!ok && lane == 0) atomicCAS(&g_gemm_error, 0, (3 << 8));
        ok = __all_sync(0xffffffffu, ok) && g_gemm_error == 0;
        tcgen05_fence_after();
        if (ok && iterations > 0) {
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
            if (!DUAL) {
                float* out = static_cast<float*>(p.out) + static_cast<size_t>(split) * p.tokens * p.outs;
#pragma unroll 1
                for (int c0 = 0; c0 < BLOCK_T; c0 += 16) {
                    if (t0 + c0 >= p.tokens) break;  // uniform: the rest of the tile is padding
                    float v[16];
                    tcgen05_ld16(lane_base + c0, v);
                    if (n < p.outs) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int t = t0 + c0 + c;
                            if (t < p.tokens) out[static_cast<size_t>(t) * p.outs + n] = v[c];
                        }
                    }
                }
            } else {
                __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll 1
                for (int c0 = 0; c0 < BLOCK_T; c0 += 16) {
                    if (t0 + c0 >= p.tokens) break;
                    float gate[16], up[16];
                    tcgen05_ld16(lane_base + c0, gate);
                    tcgen05_ld16(lane_base + BLOCK_T + c0, up);
                    if (n < p.outs) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) {
                            const int t = t0 + c0 + c;
                            if (t < p.tokens) {
                                // The result is rounded to bfloat16, so the fast exponential and
                                // division (a few ulp of float32) cost no accuracy here.
                                const float activated = __fdividef(gate[c], 1.0f + __expf(-gate[c]));
                                out[static_cast<size_t>(t) * p.outs + n] = __float2bfloat16_rn(activated * up[c]);
                            }
                        }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem_base, C::TMEM_COLUMNS);
}

// ------------------------------------------- gated product for few tokens, gate on up stacked

// act[t][n] = silu(x . w[n]) * (x . w[dual_row_offset + n]) for up to 64 tokens without splitting
// the reduction: a CTA takes 64 gate rows and the 64 matching up rows as ONE 128-row operand (two
// TMA boxes of 64 rows, one under the other), so a single MMA per k step fills accumulator rows
// 0-63 with gate sums and 64-127 with up sums.  In the epilogue the two warps that hold the up
// rows pass them through shared memory to the two that hold the gate rows, which apply SwiGLU
// and write bfloat16: no partial sums in global memory and no separate activation kernel.
// `map_w` has boxes of 64 rows.  grid (token tiles, ceil(outs / 64)).
constexpr int STACK_ROWS = 64;

// All of a product's CTAs (192 for 12,288 features) are resident at once, two per SM where they
// do not go round, so the stages of each are what keeps loads in flight.
//
// KSPLIT == 2 (up to 16 tokens): the 192 CTAs above keep 20 MB on their way, and the weights come at
// 5.9 TB/s; twice as many CTAs of half the reduction each, three to an SM, stream them at 6.5 TB/s
// (measured with the plain split product; this kernel: 6.25 TB/s at 8 tokens, 32.2 us against
// 34.5 us for 12,288 gated features of 4,096).  With tiles of 32 and 64 tokens (three stages to fit
// three CTAs to an SM) the halves gain nothing (35.8 against 36.0 us, 39.9 against 39.4 us).  The two halves of a reduction are the two CTAs of a
// cluster: the second writes its sums into the first one's shared memory (st.shared::cluster),
// which adds them to its own before the activation, so there are still no partial sums in global
// memory and no second kernel.  grid (2 x token tiles, ceil(outs / 64)), clusters of 2 along x.
template <int BLOCK_T, int KSPLIT>
struct StackedConfig {
    static constexpr int A_BYTES = BLOCK_N * BLOCK_K * 2;  // 64 gate rows on 64 up rows
    static constexpr int B_BYTES = BLOCK_T * BLOCK_K * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    // one half of a split reduction: 72 KB, three CTAs to an SM; else 6, 5, 4 stages, two to an SM
    static constexpr int STAGES = KSPLIT == 2 ? 4 : (100 * 1024) / STAGE_BYTES + (BLOCK_T == 16 ? 1 : 0);
    static constexpr int TMEM_COLUMNS = BLOCK_T < 32 ? 32 : BLOCK_T;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ void st_cluster_f32(const float* local, uint32_t rank, float value) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(value) : "memory");
}

template <int BLOCK_T, int KSPLIT>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_stacked_swiglu_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    using C = StackedConfig<BLOCK_T, KSPLIT>;
    static_assert(BLOCK_T <= 64 && (STACK_ROWS + (KSPLIT == 2 ? BLOCK_N : 0)) * BLOCK_T * 4 <= C::STAGES * C::STAGE_BYTES,
                  "the exchange buffers reuse the stages");
    static_assert(KSPLIT == 1 || KSPLIT == 2, "one CTA or a cluster of two per reduction");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* accum = empty + C::STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = KSPLIT == 2 ? cluster_ctarank() : 0;  // which half of the reduction
    const int n0 = blockIdx.y * STACK_ROWS, t0 = (blockIdx.x / KSPLIT) * BLOCK_T;
    const int per_rank = (p.k_blocks + KSPLIT - 1) / KSPLIT;
    const int kb0 = static_cast<int>(rank) * per_rank;  // first k block of this CTA
    const int iterations = max(min(per_rank, p.k_blocks - kb0), 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(tmem_holder, C::TMEM_COLUMNS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;
    constexpr int HALF_A = STACK_ROWS * BLOCK_K * 2;  // bytes of 64 rows of a k block
    bool ok = true;  // of the epilogue warps: the sums are there

    if (warp == 0) {
        if (lane == 0) {
            pdl_trigger();
            const int early = min(iterations, C::STAGES);
            for (int i = 0; i < early; ++i) {
                uint8_t* a_tile = tiles + i * C::STAGE_BYTES;
                mbar_expect_tx(&full[i], C::STAGE_BYTES);
                tma_load_2d(a_tile, &map_w, (kb0 + i) * BLOCK_K, n0, &full[i]);
                tma_load_2d(a_tile + HALF_A, &map_w, (kb0 + i) * BLOCK_K, p.dual_row_offset + n0, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d(tiles + i * C::STAGE_BYTES + C::A_BYTES, &map_x, (kb0 + i) * BLOCK_K, t0, &full[i]);
            int issued = early;
            for (int i = early; i < iterations; ++i, ++issued) {
                const int stage = i % C::STAGES;
                if (!mbar_wait(&empty[stage], ((i / C::STAGES) & 1) ^ 1)) { atomicCAS(&g_gemm_error, 0, (30 << 8) | stage); break; }
                uint8_t* a_tile = tiles + stage * C::STAGE_BYTES;
                mbar_expect_tx(&full[stage], C::STAGE_BYTES);
                tma_load_2d(a_tile, &map_w, (kb0 + i) * BLOCK_K, n0, &full[stage]);
                tma_load_2d(a_tile + HALF_A, &map_w, (kb0 + i) * BLOCK_K, p.dual_row_offset + n0, &full[stage]);
                tma_load_2d(a_tile + C::A_BYTES, &map_x, (kb0 + i) * BLOCK_K, t0, &full[stage]);
            }
            if (issued < iterations || g_gemm_error != 0) {
                for (int i = max(issued - C::STAGES, 0); i < issued; ++i)
                    mbar_wait(&full[i % C::STAGES], (i / C::STAGES) & 1);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BLOCK_T);
            for (int i = 0; i < iterations; ++i) {
                const int stage = i % C::STAGES;
                if (!mbar_wait(&full[stage], (i / C::STAGES) & 1)) { atomicCAS(&g_gemm_error, 0, (31 << 8) | stage); break; }
                tcgen05_fence_after();
                const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
                const uint64_t a_desc = smem_desc_sw128(a_addr);
                const uint64_t b_desc = smem_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t step = static_cast<uint64_t>((k * UMMA_K * 2) >> 4);
                    tcgen05_mma_bf16(tmem_base, a_desc + step, b_desc + step, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tcgen05_commit(&empty[stage]);
            }
            tcgen05_commit(accum);
        }
    } else {
        pdl_wait();
        ok = iterations == 0 || mbar_wait(accum, 0);
        if (!ok && lane == 0) atomicCAS(&g_gemm_error, 0, (32 << 8));
        ok = __all_sync(0xffffffffu, ok) && g_gemm_error == 0;
        tcgen05_fence_after();
    }
    // All copies of this CTA have landed and all its MMAs have read them: the stages now carry the
    // sums on their way, first the other half's [token of the tile][row of the 128], then the up
    // sums [token of the tile][feature of the 64].
    float* other_half = reinterpret_cast<float*>(tiles);
    float* exchange = other_half + (KSPLIT == 2 ? BLOCK_N * BLOCK_T : 0);
    const int quarter = warp & 3;  // a warp may read TMEM lanes [32 * (warp % 4), +32): 0, 1 gate rows; 2, 3 up rows
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    if (KSPLIT == 2) {
        // Every thread of both CTAs takes part in the cluster's barriers, also after a wait that ran out.
        __syncthreads();
        cluster_sync();  // the first CTA's stages are free
        if (rank == 1 && warp >= 2 && ok && iterations > 0) {
#pragma unroll 1
            for (int c0 = 0; c0 < BLOCK_T; c0 += 16) {
                if (t0 + c0 >= p.tokens) break;
                float sums[16];
                tcgen05_ld16(lane_base + c0, sums);
#pragma unroll
                for (int c = 0; c < 16; ++c) st_cluster_f32(other_half + (c0 + c) * BLOCK_N + quarter * 32 + lane, 0, sums[c]);
            }
        }
        cluster_sync();  // the second CTA's sums are in the first one's shared memory
    }
    if (warp >= 2 && rank == 0) {
        const bool add = KSPLIT == 2 && p.k_blocks > per_rank;  // the other half had k blocks of its own
        const int feature = (quarter & 1) * 32 + lane;
        if (ok && quarter >= 2) {
#pragma unroll 1
            for (int c0 = 0; c0 < BLOCK_T; c0 += 16) {
                if (t0 + c0 >= p.tokens) break;
                float up[16];
                tcgen05_ld16(lane_base + c0, up);
#pragma unroll
                for (int c = 0; c < 16; ++c)
                    exchange[(c0 + c) * STACK_ROWS + feature] = up[c] + (add ? other_half[(c0 + c) * BLOCK_N + quarter * 32 + lane] : 0.0f);
            }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps
        if (ok && quarter < 2) {
            const int n = n0 + feature;
            __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll 1
            for (int c0 = 0; c0 < BLOCK_T; c0 += 16) {
                if (t0 + c0 >= p.tokens) break;
                float gate[16];
                tcgen05_ld16(lane_base + c0, gate);
                if (n < p.outs) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int t = t0 + c0 + c;
                        if (t < p.tokens) {
                            const float g = gate[c] + (add ? other_half[(c0 + c) * BLOCK_N + quarter * 32 + lane] : 0.0f);
                            const float activated = __fdividef(g, 1.0f + __expf(-g));
                            out[static_cast<size_t>(t) * p.outs + n] = __float2bfloat16_rn(activated * exchange[(c0 + c) * STACK_ROWS + feature]);
                        }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem_base, C::TMEM_COLUMNS);
}

// ----------------------------------------------------------- CTA-pair kernel (many tokens)

// For prompts, a pair of CTAs (a cluster of two, on the two SMs of a TPC) computes a tile of 256
// output features x 256 tokens with cta_group::2 MMAs (M = 256, N = 256).  Each CTA loads its own
// 128 weight rows and its own 128 of the 256 tokens, i.e. 32 KB per k block instead of the 48 KB
// that a lone CTA needs for its 128 x 256 tile, so a third less comes out of L2 per flop and six
// stages fit where four did.  No load is multicast: every CTA fetches its own tiles, and their
// bytes are counted on the barrier of the pair's rank-0 CTA, which issues the MMAs; its
// tcgen05.commit arrives on the stage and accumulator barriers of both CTAs.  Each CTA reads its
// own 128 accumulator rows from its own tensor memory in the epilogue.
//
// The grid is one-dimensional over tiles (token tiles fastest).  When the number of tiles is not a
// multiple of the number of SM pairs and the last wave is less than half full, its tiles are cut
// into 2 or 4 narrower ones (N = 128 or 64 in the instruction descriptor) that run side by side.
template <bool DUAL>
struct PairConfig {
    static constexpr int A_BYTES = BLOCK_N * BLOCK_K * 2 * (DUAL ? 2 : 1);
    static constexpr int B_BYTES = 128 * BLOCK_K * 2;  // this CTA's half of the 256 tokens
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int TMEM_COLUMNS = DUAL ? 512 : 256;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};
constexpr int PAIR_T = 256;

template <bool DUAL>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    using C = PairConfig<DUAL>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* accum = empty + C::STAGES;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(accum + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs
    // blockIdx.x = 2 * cluster + rank; clusters walk the tiles with the token tile fastest, so the
    // clusters that run together share a weight tile.
    const int cluster = blockIdx.x >> 1;
    int tile = cluster, token_offset = 0, width = PAIR_T;
    if (cluster >= p.full_tiles) {
        // Part i of a tile cut in `tail_parts`: the 16 units of 16 tokens are shared as evenly as
        // they divide (3 parts: 96, 80, 80 tokens).
        const int j = cluster - p.full_tiles;
        tile = p.full_tiles + j / p.tail_parts;
        const int part = j % p.tail_parts;
        const int base = (PAIR_T / 16) / p.tail_parts, extra = (PAIR_T / 16) % p.tail_parts;
        width = (base + (part < extra ? 1 : 0)) * 16;
        token_offset = (part * base + min(part, extra)) * 16;
    }
    const int t0 = (tile % p.token_tiles) * PAIR_T + token_offset;
    const int n0 = ((tile / p.token_tiles) * 2 + rank) * BLOCK_N;
    const int b_row = t0 + rank * (width / 2);  // this CTA's half of the tile's tokens
    // grid.y cuts the reduction (a plain product only): split s takes k blocks [kb_begin, +iterations)
    // and writes slice s of the output.
    const int split = blockIdx.y;
    const int kb_begin = split * p.k_blocks_per_split;
    const int iterations = min(p.k_blocks_per_split, p.k_blocks - kb_begin);

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc_pair(tmem_holder, C::TMEM_COLUMNS);
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before either signals the other's
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            pdl_trigger();
            const int early = min(iterations, C::STAGES);
            for (int i = 0; i < early; ++i) {
                uint8_t* a_tile = tiles + i * C::STAGE_BYTES;
                if (rank == 0) mbar_expect_tx(&full[i], 2 * C::STAGE_BYTES);  // the bytes of both CTAs
                tma_load_2d_pair(a_tile, &map_w, (kb_begin + i) * BLOCK_K, n0, &full[i]);
                if (DUAL) tma_load_2d_pair(a_tile + BLOCK_N * BLOCK_K * 2, &map_w, (kb_begin + i) * BLOCK_K, p.dual_row_offset + n0, &full[i]);
            }
            pdl_wait();
            for (int i = 0; i < early; ++i)
                tma_load_2d_pair(tiles + i * C::STAGE_BYTES + C::A_BYTES, &map_x, (kb_begin + i) * BLOCK_K, b_row, &full[i]);
            for (int i = early; i < iterations; ++i) {
                const int stage = i % C::STAGES;
                if (!mbar_wait(&empty[stage], ((i / C::STAGES) & 1) ^ 1)) { atomicCAS(&g_gemm_error, 0, (10 << 8) | stage); break; }
                uint8_t* a_tile = tiles + stage * C::STAGE_BYTES;
                if (rank == 0) mbar_expect_tx(&full[stage], 2 * C::STAGE_BYTES);
                tma_load_2d_pair(a_tile, &map_w, (kb_begin + i) * BLOCK_K, n0, &full[stage]);
                if (DUAL) tma_load_2d_pair(a_tile + BLOCK_N * BLOCK_K * 2, &map_w, (kb_begin + i) * BLOCK_K, p.dual_row_offset + n0, &full[stage]);
                tma_load_2d_pair(a_tile + C::A_BYTES, &map_x, (kb_begin + i) * BLOCK_K, b_row, &full[stage]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_idesc_pair(width);
            bool ok = true;
            for (int i = 0; i < iterations && ok; ++i) {
                const int stage = i % C::STAGES;
                if (!mbar_wait(&full[stage], (i / C::STAGES) & 1)) { atomicCAS(&g_gemm_error, 0, (11 << 8) | stage); ok = false; break; }
                tcgen05_fence_after();
                const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
                const uint64_t a_desc = smem_desc_sw128(a_addr);
                const uint64_t b_desc = smem_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
                for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                    const uint64_t step = static_cast<uint64_t>((k * UMMA_K * 2) >> 4);
                    const uint32_t accumulate = (i > 0 || k > 0) ? 1u : 0u;
                    tcgen05_mma_bf16_pair(tmem_base, a_desc + step, b_desc + step, idesc, accumulate);
                    if (DUAL) {
                        const uint64_t a2_desc = smem_desc_sw128(a_addr + BLOCK_N * BLOCK_K * 2);
                        tcgen05_mma_bf16_pair(tmem_base + PAIR_T, a2_desc + step, b_desc + step, idesc, accumulate);
                    }
                }
                tcgen05_commit_pair(&empty[stage]);
            }
            tcgen05_commit_pair(accum);
        }
    } else {
        const int quarter = warp & 3;
        const int n = n0 + quarter * 32 + lane;
        pdl_wait();
        bool ok = mbar_wait(accum, 0);
        if (!ok && lane == 0) atomicCAS(&g_gemm_error, 0, (12 << 8));
        ok = __all_sync(0xffffffffu, ok) && g_gemm_error == 0;
        tcgen05_fence_after();
        if (ok) {
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < width; c0 += 16) {
                if (t0 + c0 >= p.tokens) break;
                if (!DUAL) {
                    float v[16];
                    tcgen05_ld16(lane_base + c0, v);
                    if (n < p.outs) {
                        float* out = static_cast<float*>(p.out) + static_cast<size_t>(split) * p.tokens * p.outs;
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            if (t0 + c0 + c < p.tokens) out[static_cast<size_t>(t0 + c0 + c) * p.outs + n] = v[c];
                    }
                } else {
                    float gate[16], up[16];
                    tcgen05_ld16(lane_base + c0, gate);
                    tcgen05_ld16(lane_base + PAIR_T + c0, up);
                    if (n < p.outs) {
                        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            if (t0 + c0 + c < p.tokens) {
                                const float activated = __fdividef(gate[c], 1.0f + __expf(-gate[c]));
                                out[static_cast<size_t>(t0 + c0 + c) * p.outs + n] = __float2bfloat16_rn(activated * up[c]);
                            }
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // neither CTA leaves while the other may still read its shared or tensor memory
    if (warp == 1) tcgen05_dealloc_pair(tmem_base, C::TMEM_COLUMNS);
}

// ------------------------------------------- persistent CTA-pair kernel (many tokens)

// The pair kernel above with one pair per two SMs walking a list of tiles (pair c takes tiles c,
// c + pairs, ...: the pairs that run together still share a weight tile) and two accumulator
// buffers in tensor memory: while the epilogue warps of both CTAs drain the buffer of tile j, the
// MMAs of tile j + 1 fill the other one, and the TMA ring never drains between tiles.  Tiles are
// 256 features x 256 tokens.  A gated product's gate and up accumulators fill all 512 columns, so
// it has one buffer: its MMAs wait for the epilogue (eight warps per CTA there, to shorten it),
// but the next tile's operands are already in shared memory by then.
// Barrier `acc_empty[b]` lives in the rank-0 CTA and counts the epilogue warps of both CTAs.
template <bool DUAL>
struct PersistentConfig {
    static constexpr int TILE_T = 256;
    static constexpr int A_BYTES = BLOCK_N * BLOCK_K * 2 * (DUAL ? 2 : 1);
    static constexpr int B_BYTES = (TILE_T / 2) * BLOCK_K * 2;  // this CTA's half of the tile's tokens
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = SMEM_BUDGET / STAGE_BYTES;
    static constexpr int BUFFERS = DUAL ? 1 : 2;          // accumulator buffers in tensor memory
    static constexpr int BUFFER_COLUMNS = DUAL ? 512 : 256;
    static constexpr int TMEM_COLUMNS = 512;
    static constexpr int EPILOGUE_WARPS = DUAL ? 8 : 4;   // per CTA; a quarter of the rows each, the columns shared
    static constexpr int THREADS = 64 + 32 * EPILOGUE_WARPS;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

__device__ __forceinline__ void mbar_arrive_cluster(uint64_t* bar, uint32_t target_rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(bar)), "r"(target_rank));
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(remote) : "memory");
}

// Item `item` of the list: its first token, its feature tile (of 256 features) and its width in tokens.
template <int TILE_T>
__device__ __forceinline__ void pair_item(const GemmParams& p, int item, int& t0, int& feature_tile, int& width) {
    int tile = item, token_offset = 0;
    width = TILE_T;
    if (item >= p.full_tiles) {
        const int j = item - p.full_tiles;
        tile = p.full_tiles + j / p.tail_parts;
        const int part = j % p.tail_parts;
        const int base = (TILE_T / 16) / p.tail_parts, extra = (TILE_T / 16) % p.tail_parts;
        width = (base + (part < extra ? 1 : 0)) * 16;
        token_offset = (part * base + min(part, extra)) * 16;
    }
    // Tiles are numbered group by group: a group is `group` token tiles wide and all feature tiles
    // tall, and inside it the token tile runs fastest.  The pairs that work at the same time then
    // cover a block of about as many feature tiles as token tiles, so they ask for the fewest
    // different operand tiles, and the group's tokens are read once for all features.
    const int per_group = p.group * p.feature_tiles;
    const int g = tile / per_group, rest = tile % per_group;
    const int wide = min(p.group, p.token_tiles - g * p.group);
    t0 = (g * p.group + rest % wide) * TILE_T + token_offset;
    feature_tile = rest / wide;
}

template <bool DUAL>
__global__ void __launch_bounds__(PersistentConfig<DUAL>::THREADS)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, GemmParams p) {
    using C = PersistentConfig<DUAL>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + C::STAGES * C::STAGE_BYTES);
    uint64_t* empty = full + C::STAGES;
    uint64_t* acc_full = empty + C::STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0: issues the MMAs
    const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;
    const int iterations = p.k_blocks;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * C::EPILOGUE_WARPS); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc_pair(tmem_holder, C::TMEM_COLUMNS);
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // both CTAs' barriers exist before either signals the other's
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;

    if (warp == 0) {
        if (lane == 0) {
            pdl_trigger();
            int it = 0;  // k blocks loaded so far, over all items: stage = it % STAGES
            bool waited = false, ok = true;
            for (int item = pair; item < p.items && ok; item += pairs) {
                int t0, feature_tile, width;
                pair_item<C::TILE_T>(p, item, t0, feature_tile, width);
                const int n0 = (feature_tile * 2 + rank) * BLOCK_N;
                const int b_row = t0 + rank * (width / 2);  // this CTA's half of the tile's tokens
                int i = 0;
                if (!waited) {
                    // The weights do not come from the previous kernel: the first stages' weight
                    // tiles are on their way before the wait for it.
                    const int early = min(iterations, C::STAGES);
                    for (; i < early; ++i) {
                        uint8_t* a_tile = tiles + i * C::STAGE_BYTES;
                        if (rank == 0) mbar_expect_tx(&full[i], 2 * C::STAGE_BYTES);  // the bytes of both CTAs
                        tma_load_2d_pair(a_tile, &map_w, i * BLOCK_K, n0, &full[i]);
                        if (DUAL) tma_load_2d_pair(a_tile + BLOCK_N * BLOCK_K * 2, &map_w, i * BLOCK_K, p.dual_row_offset + n0, &full[i]);
                    }
                    pdl_wait();
                    waited = true;
                    for (int e = 0; e < early; ++e)
                        tma_load_2d_pair(tiles + e * C::STAGE_BYTES + C::A_BYTES, &map_x, e * BLOCK_K, b_row, &full[e]);
                    it = early;
                }
                for (; i < iterations; ++i, ++it) {
                    const int stage = it % C::STAGES;
                    if (!mbar_wait(&empty[stage], ((it / C::STAGES) & 1) ^ 1)) { atomicCAS(&g_gemm_error, 0, (20 << 8) | stage); ok = false; break; }
                    uint8_t* a_tile = tiles + stage * C::STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(&full[stage], 2 * C::STAGE_BYTES);
                    tma_load_2d_pair(a_tile, &map_w, i * BLOCK_K, n0, &full[stage]);
                    if (DUAL) tma_load_2d_pair(a_tile + BLOCK_N * BLOCK_K * 2, &map_w, i * BLOCK_K, p.dual_row_offset + n0, &full[stage]);
                    tma_load_2d_pair(a_tile + C::A_BYTES, &map_x, i * BLOCK_K, b_row, &full[stage]);
                }
            }
            if (!waited) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            int it = 0, j = 0;
            bool ok = true;
            for (int item = pair; item < p.items && ok; item += pairs, ++j) {
                int t0, feature_tile, width;
                pair_item<C::TILE_T>(p, item, t0, feature_tile, width);
                const int buffer = j % C::BUFFERS;
                if (!mbar_wait(&acc_empty[buffer], ((j / C::BUFFERS) & 1) ^ 1)) { atomicCAS(&g_gemm_error, 0, (21 << 8) | buffer); break; }
                tcgen05_fence_after();
                const uint32_t idesc = make_idesc_pair(width);
                const uint32_t d_tmem = tmem_base + buffer * C::BUFFER_COLUMNS;
                for (int i = 0; i < iterations; ++i, ++it) {
                    const int stage = it % C::STAGES;
                    if (!mbar_wait(&full[stage], (it / C::STAGES) & 1)) { atomicCAS(&g_gemm_error, 0, (22 << 8) | stage); ok = false; break; }
                    tcgen05_fence_after();
                    const uint32_t a_addr = smem_u32(tiles + stage * C::STAGE_BYTES);
                    const uint64_t a_desc = smem_desc_sw128(a_addr);
                    const uint64_t b_desc = smem_desc_sw128(a_addr + C::A_BYTES);
#pragma unroll
                    for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
                        const uint64_t step = static_cast<uint64_t>((k * UMMA_K * 2) >> 4);
                        const uint32_t accumulate = (i > 0 || k > 0) ? 1u : 0u;
                        tcgen05_mma_bf16_pair(d_tmem, a_desc + step, b_desc + step, idesc, accumulate);
                        if (DUAL) {
                            const uint64_t a2_desc = smem_desc_sw128(a_addr + BLOCK_N * BLOCK_K * 2);
                            tcgen05_mma_bf16_pair(d_tmem + C::TILE_T, a2_desc + step, b_desc + step, idesc, accumulate);
                        }
                    }
                    tcgen05_commit_pair(&empty[stage]);
                }
                if (ok) tcgen05_commit_pair(&acc_full[buffer]);
            }
        }
    } else {
        const int quarter = warp & 3;
        pdl_wait();
        int j = 0;
        for (int item = pair; item < p.items; item += pairs, ++j) {
            int t0, feature_tile, width;
            pair_item<C::TILE_T>(p, item, t0, feature_tile, width);
            const int buffer = j % C::BUFFERS;
            const int n = (feature_tile * 2 + rank) * BLOCK_N + quarter * 32 + lane;
            bool ok = mbar_wait(&acc_full[buffer], (j / C::BUFFERS) & 1);
            if (!ok && lane == 0) atomicCAS(&g_gemm_error, 0, (23 << 8) | buffer);
            if (!__all_sync(0xffffffffu, ok)) break;
            tcgen05_fence_after();
            const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + buffer * C::BUFFER_COLUMNS;
            // The warps that share a quarter of the rows divide the columns in units of 16.
            constexpr int SHARERS = C::EPILOGUE_WARPS / 4;
            const int units = width / 16, sharer = (warp - 2) / 4;
            const int c_begin = (units * sharer / SHARERS) * 16, c_end = (units * (sharer + 1) / SHARERS) * 16;
#pragma unroll 1
            for (int c0 = c_begin; c0 < c_end; c0 += 16) {
                if (t0 + c0 >= p.tokens) break;
                if (!DUAL) {
                    float v[16];
                    tcgen05_ld16(lane_base + c0, v);
                    if (n < p.outs) {
                        float* out = static_cast<float*>(p.out);
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            if (t0 + c0 + c < p.tokens) out[static_cast<size_t>(t0 + c0 + c) * p.outs + n] = v[c];
                    }
                } else {
                    float gate[16], up[16];
                    tcgen05_ld16(lane_base + c0, gate);
                    tcgen05_ld16(lane_base + C::TILE_T + c0, up);
                    if (n < p.outs) {
                        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
                        for (int c = 0; c < 16; ++c)
                            if (t0 + c0 + c < p.tokens) {
                                const float activated = __fdividef(gate[c], 1.0f + __expf(-gate[c]));
                                out[static_cast<size_t>(t0 + c0 + c) * p.outs + n] = __float2bfloat16_rn(activated * up[c]);
                            }
                    }
                }
            }
            tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(&acc_empty[buffer], 0);  // this warp has read its rows of the buffer
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    cluster_sync();  // neither CTA leaves while the other may still read its shared or tensor memory
    if (warp == 1) tcgen05_dealloc_pair(tmem_base, C::TMEM_COLUMNS);
}

// -------------------------------------------------------------------------------- host

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &status) == cudaSuccess &&
            status == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(entry);
    }
    return fn;
}

// A [rows][inner] bfloat16 matrix, tiles of box_rows x 64 in the 128-byte swizzle.  `out` is
// 128 bytes.  Elements outside the matrix read as zero.
ME_EXPORT int me_make_tensor_map(void* out, const void* base, unsigned long long rows, unsigned long long inner,
                                 unsigned int box_rows) {
    EncodeTiledFn encode = encode_tiled();
    if (!encode) return ME_ERR_UNSUPPORTED;
    if (inner % 8 != 0 || reinterpret_cast<uintptr_t>(base) % 16 != 0 || box_rows > 256) return ME_ERR_ARGUMENT;
    alignas(64) CUtensorMap map;
    const cuuint64_t dims[2] = {inner, rows};
    const cuuint64_t strides[1] = {inner * 2};
    const cuuint32_t box[2] = {BLOCK_K, box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    const CUresult result = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                   element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (result != CUDA_SUCCESS) return ME_ERR_ARGUMENT;
    memcpy(out, &map, sizeof(map));
    return 0;
}

template <int BLOCK_T, bool DUAL>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, int splits, cudaStream_t stream) {
    using C = Config<BLOCK_T, DUAL>;
    auto kernel = gemm_tcgen05_kernel<BLOCK_T, DUAL>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, C::SMEM_BYTES)) return e;
    dim3 grid((p.tokens + BLOCK_T - 1) / BLOCK_T, (p.outs + BLOCK_N - 1) / BLOCK_N, splits);
    return launch_kernel(kernel, grid, GEMM_THREADS, C::SMEM_BYTES, stream, map_w, map_x, p);
}

// out[s][t][n] (float32) = sum over the k blocks of split s of x[t][k] * w[n][k].
ME_EXPORT int me_gemm_tcgen05(const void* map_w, const void* map_x, float* out, int tokens, int outs, int inner,
                              int block_t, int splits, cudaStream_t stream) {
    if (tokens <= 0 || outs <= 0) return 0;
    alignas(64) CUtensorMap w, x;
    memcpy(&w, map_w, sizeof(w));
    memcpy(&x, map_x, sizeof(x));
    GemmParams p{out, tokens, outs, (inner + BLOCK_K - 1) / BLOCK_K, 0, 0, 0, 0, 1};
    if (splits < 1 || splits > p.k_blocks) return ME_ERR_ARGUMENT;
    p.k_blocks_per_split = (p.k_blocks + splits - 1) / splits;
    if ((splits - 1) * p.k_blocks_per_split >= p.k_blocks) return ME_ERR_ARGUMENT;  // an empty split
    switch (block_t) {
        case 16: return launch<16, false>(w, x, p, splits, stream);
        case 32: return launch<32, false>(w, x, p, splits, stream);
        case 64: return launch<64, false>(w, x, p, splits, stream);
        case 128: return launch<128, false>(w, x, p, splits, stream);
        case 256: return launch<256, false>(w, x, p, splits, stream);
        default: return ME_ERR_ARGUMENT;
    }
}


template <bool DUAL>
static int launch_pair(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, cudaStream_t stream, int splits = 1) {
    using C = PairConfig<DUAL>;
    auto kernel = gemm_tcgen05_pair_kernel<DUAL>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, C::SMEM_BYTES)) return e;
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    GemmParams q = p;
    q.k_blocks_per_split = (p.k_blocks + splits - 1) / splits;
    q.token_tiles = (p.tokens + PAIR_T - 1) / PAIR_T;
    const int tiles = q.token_tiles * ((p.outs + 2 * BLOCK_N - 1) / (2 * BLOCK_N));
    const int pairs = sms / 2 > 0 ? sms / 2 : 1;
    q.full_tiles = tiles / pairs * pairs;
    // A narrow tile still streams its whole weight tile, so it costs well over its share of a full
    // tile's time; cutting pays only when the last wave is so empty that two or four parts of every
    // tile in it run side by side (measured: 6 % on the gate-up product of a 2,048-token prompt;
    // cutting a half-full wave in three or four made the products 20-60 % slower).
    q.tail_parts = 1;
    while (q.tail_parts < 4 && (tiles - q.full_tiles) * q.tail_parts * 2 <= pairs) q.tail_parts *= 2;
    if (tiles < pairs || splits > 1) { q.full_tiles = tiles; q.tail_parts = 1; }  // a single, partly filled wave: nothing to gain
    const int clusters = q.full_tiles + (tiles - q.full_tiles) * q.tail_parts;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * clusters, splits, 1);
    config.blockDim = dim3(GEMM_THREADS);
    config.dynamicSmemBytes = C::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = 2;
    return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map_w, map_x, q));
}

// out[s][t][n] (float32) = the part of x[t] . w[n] over the k blocks of split s, by CTA pairs: for
// products of a few hundred tokens, whose tiles alone do not fill the GPU.  A pair takes a third
// less out of L2 per flop than two lone CTAs, which is what bounds those products.
ME_EXPORT int me_gemm_tcgen05_pair_split(const void* map_w, const void* map_x, float* out, int tokens, int outs, int inner,
                                         int splits, cudaStream_t stream) {
    if (tokens <= 0 || outs <= 0) return 0;
    alignas(64) CUtensorMap w, x;
    memcpy(&w, map_w, sizeof(w));
    memcpy(&x, map_x, sizeof(x));
    GemmParams p{out, tokens, outs, (inner + BLOCK_K - 1) / BLOCK_K, 0, 0, 0, 0, 1};
    if (splits < 1 || splits > p.k_blocks) return ME_ERR_ARGUMENT;
    if ((splits - 1) * ((p.k_blocks + splits - 1) / splits) >= p.k_blocks) return ME_ERR_ARGUMENT;  // an empty split
    return launch_pair<false>(w, x, p, stream, splits);
}

template <bool DUAL>
static int launch_persistent(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, int group, cudaStream_t stream) {
    using C = PersistentConfig<DUAL>;
    auto kernel = gemm_tcgen05_persistent_kernel<DUAL>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, C::SMEM_BYTES)) return e;
    int device = 0, sms = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
    GemmParams q = p;
    q.token_tiles = (p.tokens + C::TILE_T - 1) / C::TILE_T;
    q.feature_tiles = (p.outs + 2 * BLOCK_N - 1) / (2 * BLOCK_N);
    q.group = group > 0 ? group : q.token_tiles;
    const int tiles = q.token_tiles * q.feature_tiles;
    const int pairs = sms / 2 > 0 ? sms / 2 : 1;
    // The tiles of a last round that is less than half full are cut in 2 or 4 narrower ones that
    // run side by side (see the pair kernel's launcher for what was measured).
    q.full_tiles = tiles / pairs * pairs;
    q.tail_parts = 1;
    while (q.tail_parts < 4 && (tiles - q.full_tiles) * q.tail_parts * 2 <= pairs) q.tail_parts *= 2;
    if (tiles <= pairs) return launch_pair<DUAL>(map_w, map_x, p, stream);  // one tile per pair: nothing to overlap
    q.items = q.full_tiles + (tiles - q.full_tiles) * q.tail_parts;
    const int clusters = q.items < pairs ? q.items : pairs;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * clusters, 1, 1);
    config.blockDim = dim3(C::THREADS);
    config.dynamicSmemBytes = C::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = 2;
    return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map_w, map_x, q));
}

// out[t][n] (float32) = x[t] . w[n] by persistent CTA pairs.  Weight and activation maps have
// boxes of 128 rows.
ME_EXPORT int me_gemm_tcgen05_persistent(const void* map_w, const void* map_x, float* out, int tokens, int outs,
                                         int inner, int group, cudaStream_t stream) {
    if (tokens <= 0 || outs <= 0) return 0;
    alignas(64) CUtensorMap w, x;
    memcpy(&w, map_w, sizeof(w));
    memcpy(&x, map_x, sizeof(x));
    GemmParams p{out, tokens, outs, (inner + BLOCK_K - 1) / BLOCK_K, 0, 0, 0, 0, 1, 0, 0, 0};
    return launch_persistent<false>(w, x, p, group, stream);
}

// act[t][n] (bfloat16) = silu(x . w[n]) * (x . w[dual_row_offset + n]) by persistent CTA pairs.
// Weight and activation maps have boxes of 128 rows.
ME_EXPORT int me_gemm_tcgen05_persistent_swiglu(const void* map_w, const void* map_x, void* act, int tokens, int outs,
                                                int inner, int dual_row_offset, int group, cudaStream_t stream) {
    if (tokens <= 0 || outs <= 0) return 0;
    alignas(64) CUtensorMap w, x;
    memcpy(&w, map_w, sizeof(w));
    memcpy(&x, map_x, sizeof(x));
    GemmParams p{act, tokens, outs, (inner + BLOCK_K - 1) / BLOCK_K, 0, dual_row_offset, 0, 0, 1, 0, 0, 0};
    return launch_persistent<true>(w, x, p, group, stream);
}

// act[t][n] (bfloat16) = silu(x . w[n]) * (x . w[dual_row_offset + n]) for n < outs.
ME_EXPORT int me_gemm_tcgen05_swiglu(const void* map_w, const void* map_x, void* act, int tokens, int outs, int inner,
                                     int dual_row_offset, int block_t, cudaStream_t stream) {
    if (tokens <= 0 || outs <= 0) return 0;
    alignas(64) CUtensorMap w, x;
    memcpy(&w, map_w, sizeof(w));
    memcpy(&x, map_x, sizeof(x));
    GemmParams p{act, tokens, outs, (inner + BLOCK_K - 1) / BLOCK_K, 0, dual_row_offset, 0, 0, 1};
    p.k_blocks_per_split = p.k_blocks;
    if (block_t == 256) return launch<256, true>(w, x, p, 1, stream);  // both accumulators fill all 512 TMEM columns
    if (block_t == 128) return launch<128, true>(w, x, p, 1, stream);
    return ME_ERR_ARGUMENT;
}

template <int BLOCK_T>
static int launch_stacked(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, cudaStream_t stream) {
    using C = StackedConfig<BLOCK_T, 1>;
    auto kernel = gemm_tcgen05_stacked_swiglu_kernel<BLOCK_T, 1>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, C::SMEM_BYTES)) return e;
    dim3 grid((p.tokens + BLOCK_T - 1) / BLOCK_T, (p.outs + STACK_ROWS - 1) / STACK_ROWS, 1);
    return launch_kernel(kernel, grid, GEMM_THREADS, C::SMEM_BYTES, stream, map_w, map_x, p);
}

// The same with the reduction cut in two halves, one per CTA of a cluster of two.
template <int BLOCK_T>
static int launch_stacked_halves(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmParams& p, cudaStream_t stream) {
    using C = StackedConfig<BLOCK_T, 2>;
    auto kernel = gemm_tcgen05_stacked_swiglu_kernel<BLOCK_T, 2>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, C::SMEM_BYTES)) return e;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(2 * ((p.tokens + BLOCK_T - 1) / BLOCK_T), (p.outs + STACK_ROWS - 1) / STACK_ROWS, 1);
    config.blockDim = dim3(GEMM_THREADS);
    config.dynamicSmemBytes = C::SMEM_BYTES;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = 2;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = 2;
    return static_cast<int>(cudaLaunchKernelEx(&config, kernel, map_w, map_x, p));
}

// act[t][n] (bfloat16) = silu(x . w[n]) * (x . w[dual_row_offset + n]) for few tokens (block_t 16,
// 32 or 64), the reduction in one CTA or (`halves` 2, block_t 16) in the two CTAs of a cluster.
// The weight map has boxes of 64 rows.
ME_EXPORT int me_gemm_tcgen05_stacked_swiglu(const void* map_w, const void* map_x, void* act, int tokens, int outs,
                                             int inner, int dual_row_offset, int block_t, int halves, cudaStream_t stream) {
    if (tokens <= 0 || outs <= 0) return 0;
    alignas(64) CUtensorMap w, x;
    memcpy(&w, map_w, sizeof(w));
    memcpy(&x, map_x, sizeof(x));
    GemmParams p{act, tokens, outs, (inner + BLOCK_K - 1) / BLOCK_K, 0, dual_row_offset, 0, 0, 1, 0};
    if (halves == 2) return block_t == 16 ? launch_stacked_halves<16>(w, x, p, stream) : ME_ERR_ARGUMENT;
    if (halves != 1) return ME_ERR_ARGUMENT;
    switch (block_t) {
        case 16: return launch_stacked<16>(w, x, p, stream);
        case 32: return launch_stacked<32>(w, x, p, stream);
        case 64: return launch_stacked<64>(w, x, p, stream);
        default: return ME_ERR_ARGUMENT;
    }
}

// ------------------------------------------------------------- the give-up path, exercised
//
// A CTA with the warp roles of the product kernels whose copies never arrive: no TMA is issued, so
// the MMA warp's wait for its first stage runs out after `polls` polls, it records the failure and
// commits nothing; the epilogue warps' wait for the accumulator runs out in turn; all warps meet,
// the tensor memory is given back, and the CTA returns normally.  Nothing faults, traps or hangs:
// a test calls this to see that a wait that runs out leaves the error word set, the context usable
// and tensor memory free for the next product.  `returned` (one int) is set to 1 at the very end.
__global__ void __launch_bounds__(GEMM_THREADS) gemm_wait_probe_kernel(uint32_t polls, int* returned) {
    __shared__ uint64_t full, accum;
    __shared__ uint32_t tmem_holder;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(&full, 1);
        mbar_init(&accum, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(&tmem_holder, 32);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = tmem_holder;
    if (warp == 0) {
        // the producer: its copy is never issued
    } else if (warp == 1) {
        if (lane == 0 && !mbar_wait(&full, 0, polls)) atomicCAS(&g_gemm_error, 0, (40 << 8));
        // no MMA was issued, so nothing is committed to `accum`
    } else {
        bool ok = mbar_wait(&accum, 0, polls);
        if (!ok && lane == 0) atomicCAS(&g_gemm_error, 0, (41 << 8));
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem_base, 32);
    if (threadIdx.x == 0) *returned = 1;
}

ME_EXPORT int me_gemm_wait_probe(int polls, int* returned, cudaStream_t stream) {
    if (polls < 1 || polls > (1 << 20) || returned == nullptr) return ME_ERR_ARGUMENT;
    return launch_kernel(gemm_wait_probe_kernel, 1, GEMM_THREADS, 0, stream, static_cast<uint32_t>(polls), returned);
}

// The first failure a kernel of this library recorded since the last call (0: none); clears it.
ME_EXPORT int me_gemm_take_error(int* code) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(code, g_gemm_error, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (*code != 0) e = cudaMemcpyToSymbol(g_gemm_error, &zero, sizeof(int));
    return static_cast<int>(e);
}
