// Causal attention of prompt portions over the paged cache on the 5th-generation tensor cores:
// both products of attention run as tcgen05.mma with accumulators in tensor memory.
//
// One CTA takes 128 consecutive new tokens of one (request, query head) and walks the request's
// keys in tiles of 128 that start at multiples of 128 in absolute position:
//
//   S = Q K^T      tcgen05.mma, A = Q tile and B = K tile from shared memory (K-major, 128-byte
//                  swizzle as TMA wrote them), D = S in tensor memory columns [0, 128)
//   P = softmax    256 threads, two per query row (tensor-memory lane = row, 64 score columns
//                  each): the scores are read once with tcgen05.ld and stay in registers for
//                  the row maximum (the two threads of a row exchange theirs through shared
//                  memory) and for exp2 and the row sum in float32; P is rounded to bfloat16 and
//                  stored with tcgen05.st over the first 64 columns of S
//   O += P V       tcgen05.mma with A = P read from tensor memory and B = V tile from shared
//                  memory as an MN-major operand (V is [key][dim]: rows run along the reduction),
//                  D = O in columns [128, 256), accumulated over the tiles
//
// When the maximum of a row has grown by more than 2^8 over the value its probabilities are taken
// relative to, O is rescaled in tensor memory (ld, multiply, st) before the next P V product;
// otherwise the older reference stays (a probability may then exceed 1) and the softmax of a tile
// waits for no product but its own scores.  Keys and values come from the
// cache by TMA, one box per page and 64-dimension half, addressed through the request's block
// table; queries likewise.  Keys beyond the request's length are read from its last page (finite
// values) and masked by position.
//
// Roles (320 threads): warp 0 issues TMA, warp 1 owns tensor memory and issues the MMAs, warps 2-9
// are the softmax rows (a row's time is a chain of dependent instructions of one thread: two
// threads per row halve it).  Shared memory is 96 KB and tensor memory 256 columns, so two CTAs share
// an SM and one's softmax overlaps the other's products.  Every wait is bounded (see tcgen05.cuh).
//
// Formula and conventions as in attention_bf16.cu (YuvGev00/mini-engine:
// src/mini_engine/attention.py:84-86,160-175; probabilities rounded to the value dtype before the
// second product, :173).  head_dim is 128; pages of 8 to 128 tokens; no window.
#include "tcgen05.cuh"

constexpr int TC_ROWS = 128;   // query rows per CTA
constexpr int TC_KEYS = 128;   // keys per tile
constexpr int TC_DIM = 128;    // head_dim
constexpr int TC_THREADS = 320;
constexpr int TC_SOFTMAX_THREADS = 256;
constexpr int TC_HALF_BYTES = 128 * 64 * 2;  // a 128-row, 64-column bfloat16 block
constexpr int TC_TMEM_COLUMNS = 256;
constexpr float TC_LOG2E = 1.4426950408889634f;

__device__ int g_attention_error = 0;

struct TcAttnParams {
    const int* block_table;   // [entries][table_width]
    const int* cu_tokens;     // [entries + 1]
    const int* context_lens;  // [entries]
    const int* entry_ids;     // the batch entries this launch covers (grid.z of them), or null: all
    __nv_bfloat16* out;       // [tokens][heads][128]
    float scale_log2;
    int heads, kv_heads, page_size, table_width;
};

// 2^x by the special-function unit alone (about 2 ulp; the result is rounded to bfloat16 anyway).
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Named barrier 1 of the 256 softmax threads, which also tells every one of them whether any
// arrived with `flag` set.
__device__ __forceinline__ bool softmax_barrier_any(bool flag) {
    uint32_t any;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "barrier.red.or.pred q, 1, 256, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(any)
        : "r"(static_cast<uint32_t>(flag))
        : "memory");
    return any != 0;
}

// max(a, b, c) in one instruction.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// The high halves of two float32 values side by side: both cut to bfloat16 (toward zero) by one
// byte permutation on the integer pipe.  The conversion instruction rounds to nearest but runs on
// the special-function unit, which the exponentials already fill.
__device__ __forceinline__ uint32_t cut_bf16x2(float lo, float hi) {
    return __byte_perm(__float_as_uint(lo), __float_as_uint(hi), 0x7632);
}

// Cutting loses half a bfloat16 step on average, 2^-8 / m of a value with mantissa m; over
// mantissas spread evenly in the exponent (what exponentials of spread-out scores give) that is
// 0.7213 * 2^-8 = 0.28 %.  The probabilities are therefore formed CUT_GAIN too large, so that what
// is left after the cut is right on average, and the row sums, which add the uncut values, are
// divided by the same factor at the end.
constexpr float CUT_GAIN = 1.0f + 0.7213475f / 256.0f;
constexpr float CUT_GAIN_LOG2 = 0.0040598f;  // log2(CUT_GAIN)

// 2^x for two values on the multiply-add pipe alone: x = n + r with n the nearest integer (the add
// of 1.5 * 2^23 leaves n in the low mantissa bits) and r in [-0.5, 0.5]; 2^r by a cubic whose
// relative error is below 8e-5 (the result is cut to bfloat16, step 4e-3); n goes into the
// exponent field by one shift-and-add.  Values below 2^-126 come out as 2^-126.
__device__ __forceinline__ float2 poly_exp2_pair(float2 x) {
    x.x = fmaxf(x.x, -126.0f);
    x.y = fmaxf(x.y, -126.0f);
    const float2 magic = make_float2(12582912.0f, 12582912.0f), minus_magic = make_float2(-12582912.0f, -12582912.0f);
    const float2 t = __fadd2_rn(x, magic);
    const float2 n = __fadd2_rn(t, minus_magic);
    const float2 r = __ffma2_rn(n, make_float2(-1.0f, -1.0f), x);
    float2 p = __ffma2_rn(make_float2(0.05517098f, 0.05517098f), r, make_float2(0.24260943f, 0.24260943f));
    p = __ffma2_rn(p, r, make_float2(0.69326097f, 0.69326097f));
    p = __ffma2_rn(p, r, make_float2(0.99992818f, 0.99992818f));
    return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(t.x) << 23)),
                       __int_as_float(__float_as_int(p.y) + (__float_as_int(t.y) << 23)));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    uint32_t packed;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(hi), "f"(lo));
    return packed;
}

__global__ void __launch_bounds__(TC_THREADS, 2)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_tile = tiles;                      // two halves of [128 rows][64 dims]
    uint8_t* k_tile = tiles + 2 * TC_HALF_BYTES;  // two halves of [128 keys][64 dims]
    uint8_t* v_tile = tiles + 4 * TC_HALF_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + 6 * TC_HALF_BYTES);
    uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 2, *v_full = bars + 3, *v_empty = bars + 4,
             *s_full = bars + 5, *p_full = bars + 6, *o_full = bars + 7;  // o_full: two, by the tile's parity
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 9);
    float* exchange = reinterpret_cast<float*>(bars + 10);  // [2 tile parities][2 column halves][128 rows]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Later blocks of a request see more keys and take longer in proportion.  The grid is (heads,
    // blocks, requests) and CTAs start in that order, so the longest blocks of all heads start
    // first and the short ones fill the SMs' slots as they come free.
    const int head = blockIdx.x, q_block = gridDim.y - 1 - blockIdx.y;

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        mbar_init(k_full, 1);
        mbar_init(k_empty, 1);
        mbar_init(v_full, 1);
        mbar_init(v_empty, 1);
        mbar_init(s_full, 1);
        mbar_init(p_full, TC_SOFTMAX_THREADS);
        mbar_init(o_full, 1);
        mbar_init(o_full + 1, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(tmem_holder, TC_TMEM_COLUMNS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_s = *tmem_holder;   // S, then P over its first 64 columns
    const uint32_t tmem_o = tmem_s + 128;

    pdl_trigger();
    pdl_wait();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.z] : blockIdx.z;
    const int token0 = p.cu_tokens[entry];
    const int new_tokens = p.cu_tokens[entry + 1] - token0;
    const bool has_work = q_block * TC_ROWS < new_tokens;  // uniform for the CTA
    const int context = p.context_lens[entry];
    const int rows_valid = min(TC_ROWS, new_tokens - q_block * TC_ROWS);
    const int pos0 = context - new_tokens + q_block * TC_ROWS;  // position of row 0
    const int tiles_count = has_work ? (pos0 + rows_valid - 1) / TC_KEYS + 1 : 0;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        // The whole warp takes part: lane g looks up page g of the tile in the block table (one
        // coalesced load for the tile, one tile ahead of its use) and issues that page's copies.
        if (has_work) {
            const int kv_head = head / (p.heads / p.kv_heads);
            const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;
            const int pages_per_tile = TC_KEYS / p.page_size;
            const int last_page_index = (context - 1) / p.page_size;
            const int page_bytes = p.page_size * 128;  // one page of one 64-dimension half
            if (lane == 0) {
                mbar_expect_tx(q_full, 2 * TC_HALF_BYTES);
                tma_load_2d(q_tile, &map_q, head * TC_DIM, token0 + q_block * TC_ROWS, q_full);
                tma_load_2d(q_tile + TC_HALF_BYTES, &map_q, head * TC_DIM + 64, token0 + q_block * TC_ROWS, q_full);
            }
            const bool loads = lane < pages_per_tile;
            int page = loads ? table[min(lane, last_page_index)] : 0;
            bool ok = true;
            for (int j = 0; j < tiles_count && ok; ++j) {
                const uint32_t parity = j & 1;
                const int next_page = (loads && j + 1 < tiles_count) ? table[min((j + 1) * pages_per_tile + lane, last_page_index)] : 0;
                const int row = (page * p.kv_heads + kv_head) * p.page_size;
                for (int which = 0; which < 2 && ok; ++which) {  // keys, then values
                    uint64_t* empty = which ? v_empty : k_empty;
                    uint64_t* full = which ? v_full : k_full;
                    uint8_t* tile = which ? v_tile : k_tile;
                    const CUtensorMap* map = which ? &map_v : &map_k;
                    if (lane == 0) {
                        ok = mbar_wait(empty, parity ^ 1);
                        if (ok) mbar_expect_tx(full, 2 * TC_HALF_BYTES);
                        else atomicCAS(&g_attention_error, 0, (1 << 8) | which);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (ok && loads) {
                        tma_load_2d(tile + lane * page_bytes, map, 0, row, full);
                        tma_load_2d(tile + TC_HALF_BYTES + lane * page_bytes, map, 64, row, full);
                    }
                }
                page = next_page;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && has_work) {
            constexpr uint32_t idesc_s = make_idesc(TC_KEYS);        // S[128 x 128] = Q K^T, K-major operands
            constexpr uint32_t idesc_o = make_idesc(TC_DIM, true);   // O[128 x 128] += P V, V is MN-major
            bool ok = mbar_wait(q_full, 0);
            if (!ok) atomicCAS(&g_attention_error, 0, 2 << 8);
            for (int j = 0; j < tiles_count && ok; ++j) {
                const uint32_t parity = j & 1;
                // The S columns are free once the previous P V product has read P out of them: the
                // MMAs of a CTA execute in the order of their issue, so this one needs no wait for it.
                ok = mbar_wait(k_full, parity);
                if (!ok) { atomicCAS(&g_attention_error, 0, (2 << 8) | 1); break; }
                tcgen05_fence_after();
#pragma unroll
                for (int kk = 0; kk < TC_DIM / 16; ++kk) {
                    const uint32_t offset = (kk / 4) * TC_HALF_BYTES + (kk % 4) * 32;
                    tcgen05_mma_bf16(tmem_s, smem_desc_sw128(smem_u32(q_tile) + offset),
                                     smem_desc_sw128(smem_u32(k_tile) + offset), idesc_s, kk > 0 ? 1u : 0u);
                }
                tcgen05_commit(s_full);
                tcgen05_commit(k_empty);
                ok = mbar_wait(p_full, parity) && mbar_wait(v_full, parity);
                if (!ok) { atomicCAS(&g_attention_error, 0, (2 << 8) | 2); break; }
                tcgen05_fence_after();
#pragma unroll
                for (int kk = 0; kk < TC_KEYS / 16; ++kk) {
                    // 16 keys = 16 rows of 128 bytes; the second 64 dimensions are one half further
                    const uint64_t v_desc = smem_desc_sw128_mn(smem_u32(v_tile) + kk * 16 * 128, TC_HALF_BYTES);
                    tcgen05_mma_bf16_ts(tmem_o, tmem_s + kk * 8, v_desc, idesc_o, (j > 0 || kk > 0) ? 1u : 0u);
                }
                tcgen05_commit(o_full + (j & 1));
                tcgen05_commit(v_empty);
            }
        }
    } else if (has_work) {
        // ------------------------------------------------------------------ softmax rows
        const int quarter = warp & 3;      // this warp's tensor-memory lanes are [32 * quarter, +32)
        const int half = (warp - 2) >> 2;  // its 64 of the 128 score (and output) columns
        const int row = quarter * 32 + lane;
        const int row_pos = pos0 + row;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const int col0 = half * 64;
        float row_max = -INFINITY, row_sum = 0.0f;  // the maximum of the whole row; the sum of this thread's columns
        // A wait that ran out must not leave other threads at a named barrier: a thread that saw
        // one keeps walking to the next barrier, where all 256 learn of it and leave together.
        bool ok = true;
        int j = 0;
        for (; j < tiles_count; ++j) {
            const uint32_t parity = j & 1;
            ok = ok && mbar_wait(s_full, parity);
            tcgen05_fence_after();
            const int first_key = j * TC_KEYS + col0;
            // Only the last tile or two of a block hold keys that some row must not see; every other
            // tile takes the path without per-element position tests.
            const bool masked_tile = j * TC_KEYS + TC_KEYS - 1 > pos0;
            uint32_t raw[64];
            tcgen05_ld32_nowait(tmem_s + lane_base + col0, raw);
            tcgen05_ld32_nowait(tmem_s + lane_base + col0 + 32, raw + 32);
            tcgen05_wait_ld();
            tcgen05_pin32(raw);
            tcgen05_pin32(raw + 32);
            float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};  // four chains, not one of 64 links
            if (masked_tile) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (first_key + i <= row_pos) best[i & 3] = fmaxf(best[i & 3], __uint_as_float(raw[i]));
            } else {
#pragma unroll
                for (int i = 0; i < 64; i += 2)  // two scores per instruction
                    best[(i >> 1) & 3] = fmax3(best[(i >> 1) & 3], __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
            }
            float tile_max = fmaxf(fmaxf(best[0], best[1]), fmaxf(best[2], best[3]));
            // The row's other thread: through shared memory, one named barrier per tile (the buffer
            // alternates with the tile's parity, so a slot is read before it is written again).
            float* slot = exchange + parity * 256;
            slot[half * 128 + row] = tile_max;
            if (softmax_barrier_any(!ok)) break;
            tile_max = fmaxf(tile_max, slot[(half ^ 1) * 128 + row]) * p.scale_log2;  // the scale is positive
            // The row's reference value `row_max` follows its true maximum lazily: only when the
            // maximum of some row of the warp has grown by more than 2^8 is O rescaled (and the
            // second product of the tile before waited for); until then probabilities are taken
            // relative to the older reference and may exceed 1, which float32 sums and bfloat16's
            // range hold with room to spare.  Both threads of a row decide alike: their warps
            // hold the same rows.
            const float new_max = fmaxf(row_max, tile_max);
            if (j == 0) {
                row_max = new_max;
            } else if (__any_sync(0xffffffffu, new_max - row_max > 8.0f)) {
                ok = ok && mbar_wait(o_full + ((j - 1) & 1), ((j - 1) >> 1) & 1);  // the MMAs run in order: all of O is complete
                tcgen05_fence_after();
                const float rescale = exp2f(row_max - new_max);
                row_sum *= rescale;
                row_max = new_max;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    float o[16];
                    tcgen05_ld16(tmem_o + lane_base + col0 + c * 16, o);
                    uint32_t scaled[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) scaled[i] = __float_as_uint(o[i] * rescale);
                    tcgen05_st16(tmem_o + lane_base + col0 + c * 16, scaled);
                }
            }
            const float base = row_max == -INFINITY ? 0.0f : row_max;
            // exp2(score * scale - base) for two scores at a time: the multiply-add and the sum use
            // the two-wide float32 instructions, so a pair costs one fma, two ex2, one add, one pack.
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), base2 = make_float2(-base, -base);
            float2 partial[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t packed[16];
                if (masked_tile) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int key = first_key + c * 32 + i;
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw[c * 32 + i]), __uint_as_float(raw[c * 32 + i + 1])), scale2, base2);
                        const float2 pr = make_float2(key <= row_pos ? fast_exp2(x.x) : 0.0f, key + 1 <= row_pos ? fast_exp2(x.y) : 0.0f);
                        partial[(i >> 1) & 1] = __fadd2_rn(partial[(i >> 1) & 1], pr);
                        packed[i / 2] = pack_bf16x2(pr.x, pr.y);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw[c * 32 + i]), __uint_as_float(raw[c * 32 + i + 1])), scale2, base2);
                        const float2 pr = make_float2(fast_exp2(x.x), fast_exp2(x.y));
                        partial[(i >> 1) & 1] = __fadd2_rn(partial[(i >> 1) & 1], pr);
                        packed[i / 2] = pack_bf16x2(pr.x, pr.y);
                    }
                }
                // P columns [16 (2 half + c), +16) hold keys [64 half + 32 c, +32).  Both threads of
                // the row have read their scores (the barrier above) before either writes P over them.
                tcgen05_st16(tmem_s + lane_base + (half * 2 + c) * 16, packed);
            }
            row_sum += (partial[0].x + partial[0].y) + (partial[1].x + partial[1].y);
            tcgen05_wait_st();
            tcgen05_fence_before();
            if (ok) mbar_arrive(p_full);
        }
        if (j == tiles_count)  // else: left at a barrier, all together
            ok = ok && mbar_wait(o_full + ((tiles_count - 1) & 1), ((tiles_count - 1) >> 1) & 1);
        // The row's sum is the sum of its two threads' (one more exchange; every thread reaches it).
        float* slot = exchange + (tiles_count & 1) * 256;
        slot[half * 128 + row] = row_sum;
        ok = !softmax_barrier_any(!ok || j < tiles_count);
        if (!ok && threadIdx.x == 64) atomicCAS(&g_attention_error, 0, 3 << 8);
        row_sum += slot[(half ^ 1) * 128 + row];
        if (ok) {
            tcgen05_fence_after();
            const float inv = 1.0f / row_sum;
            __nv_bfloat16* dst = p.out + (static_cast<size_t>(token0 + q_block * TC_ROWS + row) * p.heads + head) * TC_DIM + col0;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                float o[32];
                tcgen05_ld32(tmem_o + lane_base + col0 + c * 32, o);  // collective: every lane takes part
                if (row < rows_valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 chunk;
                        chunk.x = pack_bf16x2(o[i] * inv, o[i + 1] * inv);
                        chunk.y = pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv);
                        chunk.z = pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv);
                        chunk.w = pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = chunk;
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem_s, TC_TMEM_COLUMNS);
}

// ------------------------------------------------ two query heads of one KV group per CTA
//
// The kernel above keeps the tensor pipe a third busy: a CTA's tile is one dependent chain (scores,
// softmax, second product) and only the SM's other CTA fills the gaps.  Here one CTA carries two such
// chains that never wait for each other and share everything they can: the 128 new tokens of TWO
// query heads of the same KV group.  Both heads read the same keys and values, so one K tile and one
// V tile in shared memory (two stages each) feed four products per tile, and both heads have the same
// positions, hence the same masks and the same number of tiles.  Tensor memory holds S_a, S_b, O_a and
// O_b (512 columns, the whole of it: one CTA per SM).  A softmax thread owns a whole row of one head
// (128 scores in registers), so no two threads exchange anything: each of the two groups of 128
// threads talks to the MMA warp through its own barriers only.  The MMA warp issues
//     S_a(0), S_b(0);  then per tile j:  O_a += P_a V(j),  S_a(j+1),  O_b += P_b V(j),  S_b(j+1)
// so that while group a turns S_a(j+1) into probabilities the pipe runs O_b(j) and S_b(j+1), and
// the other way round.  A head's rows hand their probabilities over a quarter of the tile's keys at
// a time (barriers p_part[head][quarter]), and the two MMAs of a quarter are issued as soon as it
// is there: three quarters of O += P V run under the row's own exponentials instead of after them
// (8,192 tokens: 497 -> 475 us).  Lazy rescaling, masking by position and page addressing as above.
//
// What bounds it (clock stamps of one CTA, 2,048 to 8,192 tokens, before the hand-over in quarters): a
// tile of 128 keys of both heads takes 3,600 cycles; its 32 MMAs need 2,048 of the pipe (64 each, which
// is what a CTA that only issues MMAs gets, also beside warps that read and write tensor memory and
// compute exponentials: csrc/mma_rate.cu); each head's rows take 35 for the load of the scores, 250 to
// 315 for the maximum and 1,430 to 1,600 for the exponentials, and wait 1,650 for their next scores.
// So a head's tile is the chain scores -> maximum -> exponentials -> O += P V -> the next tile's
// scores (queued behind the other head's products) -> barrier -> scores, and the two heads' chains
// fill each other's gaps only in part.  The special-function unit takes four lanes a cycle per
// scheduler, so the 128 exponentials of a row are 1,024 cycles of its warp whatever else is done
// (measured alone: 9.1 cycles per score with the sum and the packing).  Tried from here and dropped:
// 2^x by a cubic on the multiply-add pipe costs 10.5 cycles per score there (the two-wide float32
// instructions issue at half rate), so more than a quarter of the exponentials moved over is a loss
// (503 us at 8,192 tokens with a quarter, 514 with none, 513 with half, 559 with three quarters); two
// threads per row halve a warp's exponentials but not the unit's (514 us); steps of 64 keys with two
// score buffers per head, so that rows never wait for a product, lost because an MMA of 64 keys
// holds its issuer as long as one of 128 (648 us); one CTA per SM that walks a list of items (longest
// first, to and fro over the CTAs) with the barriers' phases running on from item to item, so that an
// item's queries, first keys and first scores come while the item before is normalised and stored: 2
// to 3 % at 4,096 and 8,192 tokens, nothing at 2,048, and entries of unequal length would leave such a
// fixed list unbalanced where the hardware hands this kernel's CTAs out as SMs come free; an MMA warp
// that issues whatever is ready, head by head, instead of the fixed order a, b, a, b: 3,197 us against
// 1,818 us at 16,384 tokens, because the fixed order is what keeps the two heads half a tile apart, and
// heads in step compute their exponentials at the same time on the same units and leave the pipe idle
// meanwhile.  Clock stamps of all CTAs at 2,048 tokens: 60,000 to 77,000 cycles a CTA in 43 to 52 us, that is 1.48 GHz
// of 1.965 (the SMs run this kernel under the power limit).
constexpr int DUO_THREADS = 320;       // warp 0 TMA, warp 1 MMA, warps 2-5 rows of head a, warps 6-9 rows of head b
constexpr int DUO_TMEM_COLUMNS = 512;
constexpr int DUO_TILE_BYTES = 2 * TC_HALF_BYTES;  // a 128 x 128 bfloat16 tile as two 64-column halves
constexpr int DUO_SMEM_BYTES = 6 * DUO_TILE_BYTES + 1024 + 256;
#ifndef DUO_POLY
#define DUO_POLY 1  // of every four pairs of exponentials, how many the multiply-add pipe computes
#endif

__global__ void __launch_bounds__(DUO_THREADS, 1)
attention_tcgen05_duo_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                             const __grid_constant__ CUtensorMap map_v, TcAttnParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* q_tiles = tiles;                       // [2 heads][2 halves][128 rows][64 dims]
    uint8_t* k_tiles = tiles + 2 * DUO_TILE_BYTES;  // [2 stages][2 halves][128 keys][64 dims]
    uint8_t* v_tiles = tiles + 4 * DUO_TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + 6 * DUO_TILE_BYTES);
    uint64_t *q_full = bars, *k_full = bars + 1, *k_empty = bars + 3, *v_full = bars + 5, *v_empty = bars + 7,
             *s_full = bars + 9, *o_full = bars + 11,  // o_full[2 heads][2 tile parities]
             *p_part = bars + 15;                      // p_part[2 heads][4 quarters of a tile's keys]
    uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 23);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int head0 = 2 * blockIdx.x, q_block = gridDim.y - 1 - blockIdx.y;  // the longest blocks start first

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) {
            mbar_init(k_full + i, 1);
            mbar_init(k_empty + i, 1);
            mbar_init(v_full + i, 1);
            mbar_init(v_empty + i, 1);
            mbar_init(s_full + i, 1);
        }
        for (int i = 0; i < 8; ++i) mbar_init(p_part + i, 128);
        for (int i = 0; i < 4; ++i) mbar_init(o_full + i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tcgen05_alloc(tmem_holder, DUO_TMEM_COLUMNS);
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    const uint32_t tmem_base = *tmem_holder;  // S_a, S_b at columns 0 and 128 (P over the first 64 of each), O_a, O_b at 256 and 384

    pdl_trigger();
    pdl_wait();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.z] : blockIdx.z;
    const int token0 = p.cu_tokens[entry];
    const int new_tokens = p.cu_tokens[entry + 1] - token0;
    const bool has_work = q_block * TC_ROWS < new_tokens;  // uniform for the CTA
    const int context = p.context_lens[entry];
    const int rows_valid = min(TC_ROWS, new_tokens - q_block * TC_ROWS);
    const int pos0 = context - new_tokens + q_block * TC_ROWS;  // position of row 0
    const int tiles_count = has_work ? (pos0 + rows_valid - 1) / TC_KEYS + 1 : 0;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (has_work) {
            const int kv_head = head0 / (p.heads / p.kv_heads);
            const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;
            const int pages_per_tile = TC_KEYS / p.page_size;
            const int last_page_index = (context - 1) / p.page_size;
            const int page_bytes = p.page_size * 128;  // one page of one 64-dimension half
            if (lane == 0) {
                mbar_expect_tx(q_full, 2 * DUO_TILE_BYTES);
                for (int h = 0; h < 2; ++h)
                    for (int half = 0; half < 2; ++half)
                        tma_load_2d(q_tiles + h * DUO_TILE_BYTES + half * TC_HALF_BYTES, &map_q,
                                    (head0 + h) * TC_DIM + half * 64, token0 + q_block * TC_ROWS, q_full);
            }
            const bool loads = lane < pages_per_tile;
            int page = loads ? table[min(lane, last_page_index)] : 0;
            bool ok = true;
            for (int j = 0; j < tiles_count && ok; ++j) {
                const int stage = j & 1;
                const uint32_t parity = (j >> 1) & 1;
                const int next_page = (loads && j + 1 < tiles_count) ? table[min((j + 1) * pages_per_tile + lane, last_page_index)] : 0;
                const int row = (page * p.kv_heads + kv_head) * p.page_size;
                for (int which = 0; which < 2 && ok; ++which) {  // keys, then values
                    uint64_t* empty = (which ? v_empty : k_empty) + stage;
                    uint64_t* full = (which ? v_full : k_full) + stage;
                    uint8_t* tile = (which ? v_tiles : k_tiles) + stage * DUO_TILE_BYTES;
                    const CUtensorMap* map = which ? &map_v : &map_k;
                    if (lane == 0) {
                        ok = mbar_wait(empty, parity ^ 1);
                        if (ok) mbar_expect_tx(full, DUO_TILE_BYTES);
                        else atomicCAS(&g_attention_error, 0, (11 << 8) | which);
                    }
                    ok = __shfl_sync(0xffffffffu, ok, 0);
                    if (ok && loads) {
                        tma_load_2d(tile + lane * page_bytes, map, 0, row, full);
                        tma_load_2d(tile + TC_HALF_BYTES + lane * page_bytes, map, 64, row, full);
                    }
                }
                page = next_page;
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && has_work) {
            constexpr uint32_t idesc_s = make_idesc(TC_KEYS);       // S[128 x 128] = Q K^T, K-major operands
            constexpr uint32_t idesc_o = make_idesc(TC_DIM, true);  // O[128 x 128] += P V, V is MN-major
            // An MMA instruction holds the thread that issues it for 54 cycles whatever its size, and
            // the pipe needs 64 for 128 x 128 x 16: what the thread does besides must stay under ten
            // cycles an MMA or the pipe waits for it.  So the operands' descriptors are made once (their
            // address field is additive: a k step further is a constant more) and the first MMA of a
            // product, which overwrites, is its own instruction instead of a predicate computed each time.
            constexpr uint64_t NEXT_TILE = DUO_TILE_BYTES >> 4;  // the second head's queries, the second stage
            const uint64_t q_desc = smem_desc_sw128(smem_u32(q_tiles)), k_desc = smem_desc_sw128(smem_u32(k_tiles));
            const uint64_t v_desc = smem_desc_sw128_mn(smem_u32(v_tiles), TC_HALF_BYTES);
            auto scores = [&](int h, int stage) {
                const uint64_t q = q_desc + h * NEXT_TILE, k = k_desc + stage * NEXT_TILE;
                const uint32_t d = tmem_base + h * 128;
#pragma unroll
                for (int kk = 0; kk < TC_DIM / 16; ++kk) {
                    constexpr uint32_t HALF_STEP = TC_HALF_BYTES >> 4;
                    const uint64_t offset = (kk / 4) * HALF_STEP + (kk % 4) * 2;  // in units of 16 bytes
                    if (kk == 0) tcgen05_mma_bf16_overwrite(d, q + offset, k + offset, idesc_s);
                    else tcgen05_mma_bf16_add(d, q + offset, k + offset, idesc_s);
                }
                tcgen05_commit(s_full + h);
            };
            // O_h (+)= P_h V: the rows hand their probabilities over a quarter of the keys at a time, and
            // the two MMAs of a quarter are issued as soon as it is there, under the exponentials of the next.
            auto outputs = [&](int h, int stage, int j) -> bool {
                const uint64_t v = v_desc + stage * NEXT_TILE;
                const uint32_t d = tmem_base + 256 + h * 128, a = tmem_base + h * 128;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    if (!mbar_wait(p_part + h * 4 + c, j & 1)) return false;
                    tcgen05_fence_after();
                    if (c == 0 && j == 0) tcgen05_mma_bf16_ts_overwrite(d, a, v, idesc_o);
                    else tcgen05_mma_bf16_ts_add(d, a + (2 * c) * 8, v + (2 * c) * (16 * 128 >> 4), idesc_o);
                    tcgen05_mma_bf16_ts_add(d, a + (2 * c + 1) * 8, v + (2 * c + 1) * (16 * 128 >> 4), idesc_o);
                }
                tcgen05_commit(o_full + h * 2 + (j & 1));
                return true;
            };
            bool ok = mbar_wait(q_full, 0) && mbar_wait(k_full, 0);
            if (!ok) atomicCAS(&g_attention_error, 0, 12 << 8);
            if (ok) {
                tcgen05_fence_after();
                scores(0, 0);
                scores(1, 0);
                tcgen05_commit(k_empty);
            }
            for (int j = 0; j < tiles_count && ok; ++j) {
                const int stage = j & 1, next = stage ^ 1;
                const uint32_t stage_parity = (j >> 1) & 1, next_parity = ((j + 1) >> 1) & 1;
                const bool more = j + 1 < tiles_count;
                // head a: its probabilities of tile j are ready; then its scores of tile j + 1.  The
                // MMAs of a CTA run in the order of their issue, so the scores cannot overwrite the
                // probabilities that the product before them still reads.
                ok = mbar_wait(v_full + stage, stage_parity) && outputs(0, stage, j);
                if (!ok) { atomicCAS(&g_attention_error, 0, (12 << 8) | 1); break; }
                if (more) {
                    ok = mbar_wait(k_full + next, next_parity);
                    if (!ok) { atomicCAS(&g_attention_error, 0, (12 << 8) | 2); break; }
                    tcgen05_fence_after();
                    scores(0, next);
                }
                // head b likewise; after its products the stages of V(j) and K(j + 1) are free
                ok = outputs(1, stage, j);
                if (!ok) { atomicCAS(&g_attention_error, 0, (12 << 8) | 3); break; }
                tcgen05_commit(v_empty + stage);
                if (more) {
                    scores(1, next);
                    tcgen05_commit(k_empty + next);
                }
            }
        }
    } else if (has_work) {
        // ------------------------------------------------------------------ softmax rows
        const int h = (warp - 2) >> 2;  // which of the two heads
        const int quarter = warp & 3;   // this warp's tensor-memory lanes are [32 * quarter, +32)
        const int row = quarter * 32 + lane;
        const int row_pos = pos0 + row;
        const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t tmem_s = tmem_base + h * 128 + lane_base, tmem_o = tmem_base + 256 + h * 128 + lane_base;
        uint64_t* my_o_full = o_full + h * 2;
        float row_max = -INFINITY, row_sum = 0.0f;
        bool ok = true;
        for (int j = 0; j < tiles_count; ++j) {
            ok = __all_sync(0xffffffffu, mbar_wait(s_full + h, j & 1));
            if (!ok) break;
            tcgen05_fence_after();
            const int first_key = j * TC_KEYS;
            const bool masked_tile = first_key + TC_KEYS - 1 > pos0;  // some row must not see some key of the tile
            uint32_t raw[128];
#pragma unroll
            for (int c = 0; c < 4; ++c) tcgen05_ld32_nowait(tmem_s + c * 32, raw + c * 32);
            tcgen05_wait_ld();
#pragma unroll
            for (int c = 0; c < 4; ++c) tcgen05_pin32(raw + c * 32);
            float best[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
            if (masked_tile) {
#pragma unroll
                for (int i = 0; i < 128; ++i)
                    if (first_key + i <= row_pos) best[i & 3] = fmaxf(best[i & 3], __uint_as_float(raw[i]));
            } else {
#pragma unroll
                for (int i = 0; i < 128; i += 2)
                    best[(i >> 1) & 3] = fmax3(best[(i >> 1) & 3], __uint_as_float(raw[i]), __uint_as_float(raw[i + 1]));
            }
            const float tile_max = fmaxf(fmaxf(best[0], best[1]), fmaxf(best[2], best[3])) * p.scale_log2;  // the scale is positive
            // The reference value of the row follows its maximum lazily, as in the kernel above.
            const float new_max = fmaxf(row_max, tile_max);
            if (j == 0) {
                row_max = new_max;
            } else if (__any_sync(0xffffffffu, new_max - row_max > 8.0f)) {
                ok = __all_sync(0xffffffffu, mbar_wait(my_o_full + ((j - 1) & 1), ((j - 1) >> 1) & 1));  // the MMAs run in order: all of O is complete
                if (!ok) break;
                tcgen05_fence_after();
                const float rescale = exp2f(row_max - new_max);
                row_sum *= rescale;
                row_max = new_max;
#pragma unroll 1
                for (int c = 0; c < 8; ++c) {
                    float o[16];
                    tcgen05_ld16(tmem_o + c * 16, o);
                    uint32_t scaled[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) scaled[i] = __float_as_uint(o[i] * rescale);
                    tcgen05_st16(tmem_o + c * 16, scaled);
                }
            }
            const float base = row_max == -INFINITY ? 0.0f : row_max;
            // exp2(score * scale - base) * CUT_GAIN.  DUO_POLY of every four pairs of exponentials go
            // through the multiply-add pipe instead of the special-function unit, and the
            // probabilities are cut to bfloat16 on the integer pipe.
            const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), base2 = make_float2(CUT_GAIN_LOG2 - base, CUT_GAIN_LOG2 - base);
            float2 partial[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t packed[16];
                if (masked_tile) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const int key = first_key + c * 32 + i;
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw[c * 32 + i]), __uint_as_float(raw[c * 32 + i + 1])), scale2, base2);
                        const float2 pr = make_float2(key <= row_pos ? fast_exp2(x.x) : 0.0f, key + 1 <= row_pos ? fast_exp2(x.y) : 0.0f);
                        partial[(i >> 1) & 1] = __fadd2_rn(partial[(i >> 1) & 1], pr);
                        packed[i / 2] = cut_bf16x2(pr.x, pr.y);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(raw[c * 32 + i]), __uint_as_float(raw[c * 32 + i + 1])), scale2, base2);
                        const float2 pr = ((i >> 1) % 4) < DUO_POLY ? poly_exp2_pair(x) : make_float2(fast_exp2(x.x), fast_exp2(x.y));
                        partial[(i >> 1) & 1] = __fadd2_rn(partial[(i >> 1) & 1], pr);
                        packed[i / 2] = cut_bf16x2(pr.x, pr.y);
                    }
                }
                // P columns [16 c, +16) hold keys [32 c, +32); this thread has read its whole row of S.
                // The quarter before has had this quarter's exponentials to land in tensor memory.
                if (c > 0) {
                    tcgen05_wait_st();
                    tcgen05_fence_before();
                    mbar_arrive(p_part + h * 4 + c - 1);
                }
                tcgen05_st16(tmem_s + c * 16, packed);
            }
            row_sum += (partial[0].x + partial[0].y) + (partial[1].x + partial[1].y);
            tcgen05_wait_st();
            tcgen05_fence_before();
            mbar_arrive(p_part + h * 4 + 3);
        }
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(my_o_full + ((tiles_count - 1) & 1), ((tiles_count - 1) >> 1) & 1));
        if (!ok && lane == 0) atomicCAS(&g_attention_error, 0, 13 << 8);
        if (ok) {
            tcgen05_fence_after();
            const float inv = CUT_GAIN / row_sum;
            __nv_bfloat16* dst = p.out + (static_cast<size_t>(token0 + q_block * TC_ROWS + row) * p.heads + head0 + h) * TC_DIM;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                float o[32];
                tcgen05_ld32(tmem_o + c * 32, o);  // collective: every lane takes part
                if (row < rows_valid) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 chunk;
                        chunk.x = pack_bf16x2(o[i] * inv, o[i + 1] * inv);
                        chunk.y = pack_bf16x2(o[i + 2] * inv, o[i + 3] * inv);
                        chunk.z = pack_bf16x2(o[i + 4] * inv, o[i + 5] * inv);
                        chunk.w = pack_bf16x2(o[i + 6] * inv, o[i + 7] * inv);
                        *reinterpret_cast<uint4*>(dst + c * 32 + i) = chunk;
                    }
                }
            }
        }
    }
    tcgen05_fence_before();
    __syncthreads();
    if (warp == 1) tcgen05_dealloc(tmem_base, DUO_TMEM_COLUMNS);
}

// -------------------------------------------------------------------------------- host

// q, k and v are described by TMA maps made with me_make_tensor_map (gemm_tcgen05.cu): q as
// [tokens][heads * 128] with boxes of 128 rows, the page arrays as [(pages * kv_heads *
// page_size)][128] with boxes of page_size rows.
ME_EXPORT int me_attention_tcgen05(const void* map_q, const void* map_k, const void* map_v, const int* block_table,
                                   const int* cu_tokens, const int* context_lens, void* out, float scale, int entries,
                                   int max_new_tokens, int heads, int kv_heads, int head_dim, int page_size,
                                   int table_width, const int* entry_ids, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (head_dim != TC_DIM || kv_heads < 1 || heads % kv_heads) return ME_ERR_UNSUPPORTED;
    if (page_size < 8 || page_size > TC_KEYS || TC_KEYS % page_size) return ME_ERR_UNSUPPORTED;
    alignas(64) CUtensorMap q, k, v;
    memcpy(&q, map_q, sizeof(q));
    memcpy(&k, map_k, sizeof(k));
    memcpy(&v, map_v, sizeof(v));
    TcAttnParams p{block_table, cu_tokens, context_lens, entry_ids, static_cast<__nv_bfloat16*>(out), scale * TC_LOG2E,
                   heads, kv_heads, page_size, table_width};
    const int blocks = (max_new_tokens + TC_ROWS - 1) / TC_ROWS;
    if ((heads / kv_heads) % 2 == 0) {  // two query heads of a KV group per CTA
        static SharedMemoryOptIn duo_opt_in;
        if (const int e = duo_opt_in(attention_tcgen05_duo_kernel, DUO_SMEM_BYTES)) return e;
        return launch_kernel(attention_tcgen05_duo_kernel, dim3(heads / 2, blocks, entries), DUO_THREADS, DUO_SMEM_BYTES,
                             stream, q, k, v, p);
    }
    constexpr int SMEM = 6 * TC_HALF_BYTES + 1024 + 256 + 2 * 2 * 128 * 4;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(attention_tcgen05_kernel, SMEM)) return e;
    return launch_kernel(attention_tcgen05_kernel, dim3(heads, blocks, entries), TC_THREADS, SMEM, stream, q, k, v, p);
}

ME_EXPORT int me_attention_take_error(int* code) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(code, g_attention_error, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (*code != 0) e = cudaMemcpyToSymbol(g_attention_error, &zero, sizeof(int));
    return static_cast<int>(e);
}
