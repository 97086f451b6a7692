// Causal grouped-query attention over the paged cache in bfloat16 with tensor-core products
// and a 32-bit online softmax, for head sizes 64 and 128.
//
// Two kernels share the tile code:
//   * portions (any number of new tokens per request): one CTA per (request, query head,
//     64 consecutive new tokens); it walks the request's keys in tiles of 64 that start at
//     multiples of 64 in absolute position, double-buffered through shared memory.
//   * decode (one new token per request): one CTA per (request, KV head, 128 keys); all query
//     heads of the group share the keys that are read; each of its four warps takes 32 keys;
//     the CTA writes one partial (max, sum, unnormalised output) per head to scratch memory,
//     and a second kernel merges a request's partials in ascending key order.  The split
//     depends on positions only, never on the batch.
//
// Formula (YuvGev00/mini-engine: src/mini_engine/attention.py:84-86,160-175, the online softmax
// of src/mini_engine/triton_attention.py:56-82): query head h reads KV head h / group;
// s = (q . k) * scale; a query at position p sees keys at positions <= p (and > p - window);
// out = softmax(s) V.  Scores, maxima, sums and the output accumulate in float32; the
// probabilities are rounded to bfloat16 for the second product, as the reference's
// `p.to(v.dtype)` does.
//
// Pages are [page][kv_head][slot][head_dim]; a key's address comes from the request's block
// table, so any page size works.  Keys outside the visible range are zero-filled in shared
// memory (never read from the cache), so stale contents of reused pages cannot leak.
#include <string.h>

#include "tcgen05.cuh"

constexpr int BLOCK_M = 64;   // query rows per CTA (portions)
constexpr int BLOCK_KEYS = 64;  // keys per tile
constexpr int ATTN_THREADS = 128;
constexpr int DECODE_WARP_KEYS = 32;
constexpr int DECODE_CHUNK = 4 * DECODE_WARP_KEYS;  // keys per decode CTA
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
    const __nv_bfloat16* q;        // [tokens][heads][D]
    const __nv_bfloat16* k_pages;  // [pages][kv_heads][page_size][D]
    const __nv_bfloat16* v_pages;
    const int* block_table;   // [entries][table_width]
    const int* cu_tokens;     // [entries + 1]
    const int* context_lens;  // [entries]
    __nv_bfloat16* out;       // [tokens][heads][D]
    float* partials;          // decode: [entries][heads][max_splits][D + 2]
    int* counters;            // decode: [entries][kv_heads] arrival counts, all zero between launches; or null
    const int* entry_ids;     // the batch entries this launch covers (grid.z of them), or null: all, in order
    float scale_log2;         // scale * log2(e)
    int heads, kv_heads, page_size, table_width, window, max_splits;
    int page_shift;  // log2(page_size) when it is a power of two, else -1
    int tiles_per_cta;  // decode: consecutive 128-key tiles that one CTA walks
};

// ------------------------------------------------------------------------ small helpers

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// 16-byte chunks of a row are permuted by the row's low bits so that the eight rows an
// ldmatrix reads fall into different banks.
template <int D>
__device__ __forceinline__ int swizzled(int row, int chunk) {
    return row * (D / 8) + (chunk ^ (row & 7));
}

__device__ __forceinline__ void cp_async_16(void* dst, const void* src, bool valid) {
    const int bytes = valid ? 16 : 0;  // 0: the destination is filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Element offset of a key's row inside the page arrays (the same for keys and values), or -1
// when the key is outside [lowest, last_key] or its page was given back.
__device__ __forceinline__ long long key_row_offset(const AttnParams& p, const int* table, int key, int lowest,
                                                    int last_key, int kv_head, int head_dim) {
    if (key < lowest || key > last_key) return -1;
    int page_index, slot;
    if (p.page_shift >= 0) {
        page_index = key >> p.page_shift;
        slot = key & (p.page_size - 1);
    } else {
        page_index = key / p.page_size;
        slot = key - page_index * p.page_size;
    }
    const int page = table[page_index];
    if (page < 0) return -1;
    return ((static_cast<long long>(page) * p.kv_heads + kv_head) * p.page_size + slot) * head_dim;
}

// One warp: scores of its 16 query rows against KEYS keys.  `q_frag` holds the rows' A fragments.
template <int D, int KEYS>
__device__ __forceinline__ void scores_tile(float (&s)[KEYS / 8][4], const uint32_t (&q_frag)[D / 16][4],
                                            const __nv_bfloat16* k_tile, int lane) {
#pragma unroll
    for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) s[n][i] = 0.0f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
        for (int pair = 0; pair < KEYS / 16; ++pair) {  // two 8-key tiles per ldmatrix.x4
            uint32_t b[4];
            const int key = pair * 16 + (lane & 7) + (lane >> 4) * 8;
            const int chunk = kk * 2 + ((lane >> 3) & 1);
            ldmatrix_x4(b, k_tile + swizzled<D>(key, chunk) * 8);
            mma_bf16(s[pair * 2], q_frag[kk], b[0], b[1]);
            mma_bf16(s[pair * 2 + 1], q_frag[kk], b[2], b[3]);
        }
    }
}

// One warp: acc[16 x D] += P[16 x KEYS] V[KEYS x D], P taken from the score registers.
template <int D, int KEYS>
__device__ __forceinline__ void accumulate_pv(float (&acc)[D / 8][4], const float (&s)[KEYS / 8][4],
                                              const __nv_bfloat16* v_tile, int lane) {
#pragma unroll
    for (int kk = 0; kk < KEYS / 16; ++kk) {  // 16 keys per step
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int pair = 0; pair < D / 16; ++pair) {  // two 8-dim tiles per ldmatrix.x4.trans
            uint32_t b[4];
            const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            const int chunk = pair * 2 + (lane >> 4);
            ldmatrix_x4_trans(b, v_tile + swizzled<D>(key, chunk) * 8);
            mma_bf16(acc[pair * 2], a, b[0], b[1]);
            mma_bf16(acc[pair * 2 + 1], a, b[2], b[3]);
        }
    }
}

// Masks the scores of one tile, updates the running maximum and sum of the thread's two rows
// (row `g` and row `g + 8` of the warp's 16) and turns the scores into probabilities.
// `row_pos[i]` is the absolute position of row i's query; keys are visible in
// [row_pos - window + 1, row_pos] (window <= 0: from 0).
template <int D, int KEYS>
__device__ __forceinline__ void softmax_step(float (&s)[KEYS / 8][4], float (&acc)[D / 8][4], float (&row_max)[2],
                                             float (&row_sum)[2], const int (&row_pos)[2], int first_key,
                                             int window, float scale_log2, int lane) {
    const int col0 = first_key + 2 * (lane & 3);
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int key = col0 + n * 8 + (i & 1);
            const int r = i >> 1;
            const bool visible = key <= row_pos[r] && (window <= 0 || key > row_pos[r] - window);
            s[n][i] = visible ? s[n][i] * scale_log2 : -INFINITY;
            tile_max[r] = fmaxf(tile_max[r], s[n][i]);
        }
    float rescale[2], base[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 1));
        tile_max[r] = fmaxf(tile_max[r], __shfl_xor_sync(0xffffffffu, tile_max[r], 2));
        const float new_max = fmaxf(row_max[r], tile_max[r]);
        base[r] = new_max == -INFINITY ? 0.0f : new_max;  // a row that has seen nothing yet
        rescale[r] = exp2f(row_max[r] - base[r]);         // 0 while row_max is -inf
        row_max[r] = new_max;
        row_sum[r] *= rescale[r];
    }
#pragma unroll
    for (int n = 0; n < KEYS / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float prob = exp2f(s[n][i] - base[i >> 1]);
            s[n][i] = prob;
            row_sum[i >> 1] += prob;
        }
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] *= rescale[i >> 1];
}

// --------------------------------------------------------------------- portions kernel

template <int D>
__global__ void __launch_bounds__(ATTN_THREADS) attention_portions_kernel(AttnParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem);  // [64][D]
    __nv_bfloat16* kv_tiles = q_tile + BLOCK_M * D;                  // [2 stages][K | V][64][D]
    constexpr int CHUNKS = D / 8;
    constexpr int ROWS_PER_PASS = ATTN_THREADS / CHUNKS;
    constexpr int PASSES = BLOCK_KEYS / ROWS_PER_PASS;

    // Later blocks of a request see more keys: start them first so that the grid's tail is short.
    const int head = blockIdx.y, q_block = gridDim.x - 1 - blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.z] : blockIdx.z;
    const int token0 = p.cu_tokens[entry];
    const int new_tokens = p.cu_tokens[entry + 1] - token0;
    if (q_block * BLOCK_M >= new_tokens) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rows_valid = min(BLOCK_M, new_tokens - q_block * BLOCK_M);
    const int pos0 = p.context_lens[entry] - new_tokens + q_block * BLOCK_M;  // position of row 0
    const int last_key = pos0 + rows_valid - 1;
    const int lowest = p.window > 0 ? max(pos0 - p.window + 1, 0) : 0;
    const int kv_head = head / (p.heads / p.kv_heads);
    const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;
    const int my_chunk = threadIdx.x % CHUNKS, my_row = threadIdx.x / CHUNKS;

    // Queries of this block -> shared memory (rows past the end are zero).
    {
        const __nv_bfloat16* q_src = p.q + (static_cast<size_t>(token0 + q_block * BLOCK_M) * p.heads + head) * D;
#pragma unroll
        for (int pass = 0; pass < BLOCK_M / ROWS_PER_PASS; ++pass) {
            const int row = pass * ROWS_PER_PASS + my_row;
            const bool valid = row < rows_valid;
            cp_async_16(q_tile + swizzled<D>(row, my_chunk) * 8,
                        valid ? q_src + static_cast<size_t>(row) * p.heads * D + my_chunk * 8 : p.q, valid);
        }
    }
    const int first_tile = lowest / BLOCK_KEYS, last_tile = last_key / BLOCK_KEYS;
    auto prefetch = [&](int tile, int s) {
        __nv_bfloat16* k_tile = kv_tiles + s * 2 * BLOCK_KEYS * D;
        __nv_bfloat16* v_tile = k_tile + BLOCK_KEYS * D;
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {
            const int row = pass * ROWS_PER_PASS + my_row;
            const long long offset = key_row_offset(p, table, tile * BLOCK_KEYS + row, lowest, last_key, kv_head, D);
            const bool valid = offset >= 0;
            const long long at = valid ? offset + my_chunk * 8 : 0;
            cp_async_16(k_tile + swizzled<D>(row, my_chunk) * 8, p.k_pages + at, valid);
            cp_async_16(v_tile + swizzled<D>(row, my_chunk) * 8, p.v_pages + at, valid);
        }
    };
    prefetch(first_tile, 0);
    cp_async_commit();

    uint32_t q_frag[D / 16][4];
    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    const int row_pos[2] = {pos0 + warp * 16 + (lane >> 2), pos0 + warp * 16 + (lane >> 2) + 8};

    for (int tile = first_tile; tile <= last_tile; ++tile) {
        const int s = (tile - first_tile) & 1;
        if (tile < last_tile) {
            prefetch(tile + 1, s ^ 1);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (tile == first_tile) {
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(q_frag[kk], q_tile + swizzled<D>(row, kk * 2 + (lane >> 4)) * 8);
            }
        }
        const __nv_bfloat16* k_tile = kv_tiles + s * 2 * BLOCK_KEYS * D;
        float scores[BLOCK_KEYS / 8][4];
        scores_tile<D, BLOCK_KEYS>(scores, q_frag, k_tile, lane);
        softmax_step<D, BLOCK_KEYS>(scores, acc, row_max, row_sum, row_pos, tile * BLOCK_KEYS, p.window, p.scale_log2, lane);
        accumulate_pv<D, BLOCK_KEYS>(acc, scores, k_tile + BLOCK_KEYS * D, lane);
        __syncthreads();  // the next iteration's prefetch overwrites the other stage's reader
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = warp * 16 + (lane >> 2) + r * 8;
        if (row >= rows_valid) continue;
        const float inv = 1.0f / row_sum[r];
        __nv_bfloat16* dst = p.out + (static_cast<size_t>(token0 + q_block * BLOCK_M + row) * p.heads + head) * D;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const int col = n * 8 + 2 * (lane & 3);
            *reinterpret_cast<uint32_t*>(dst + col) = pack_bf16(acc[n][r * 2] * inv, acc[n][r * 2 + 1] * inv);
        }
    }
}

// ----------------------------------------------------------------------- decode kernels

// grid (splits, kv_heads, entries).  Rows of the score tile are the query heads of the group
// (at most 16; the rest of the 16 rows are zero).  A CTA takes `tiles_per_cta` consecutive tiles of
// 128 keys (32 per warp); while a warp multiplies one tile's keys, its values and the next tile's
// keys are on their way, so loads never stop.  Three CTAs fit an SM.
constexpr int MAX_DECODE_TILES = 8;

template <int D>
__device__ __forceinline__ void merge_head(const AttnParams& p, int entry, int head, int first, int last, int lane);

// First failure that a decode kernel recorded: 1 = a bounded wait ran out, 2 = a context needed
// more partial-result slots than the launch was given (its last keys were left out).
__device__ int g_decode_error = 0;

// The range of partial-result slots of one (entry, head) in the kernel below: one per span of
// keys that the query can see, clamped to the slots that exist.  A context that needs more was
// given too few splits by the caller: its keys beyond are not read, which is recorded.
__device__ __forceinline__ void decode_slot_range(const AttnParams& p, int position, int lowest, int span, int& first,
                                                  int& last) {
    last = position / span;
    if (last >= p.max_splits) {
        atomicCAS(&g_decode_error, 0, 2);
        last = p.max_splits - 1;
    }
    first = min(lowest / span, last);
}

template <int D>
__global__ void __launch_bounds__(ATTN_THREADS, 3) attention_decode_kernel(AttnParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int KEYS = DECODE_WARP_KEYS;
    constexpr int CHUNKS = D / 8;
    constexpr int ROWS_PER_PASS = 32 / CHUNKS;
    constexpr int WARP_TILE = 2 * KEYS * D;  // elements of one warp's K and V tiles
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem);  // [16][D]
    __nv_bfloat16* kv_tiles = q_tile + 16 * D;                       // [4 warps][K | V][KEYS][D]

    const int kv_head = blockIdx.y, split = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.z] : blockIdx.z;
    const int position = p.context_lens[entry] - 1;  // the query's position; it sees keys <= position
    const int lowest = p.window > 0 ? max(position - p.window + 1, 0) : 0;
    const int span = p.tiles_per_cta * DECODE_CHUNK;
    const int cta_start = split * span;
    if (cta_start > position || cta_start + span <= lowest) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = p.heads / p.kv_heads;
    const int token = p.cu_tokens[entry];
    const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;

    for (int idx = threadIdx.x; idx < 16 * CHUNKS; idx += ATTN_THREADS) {
        const int row = idx / CHUNKS, chunk = idx % CHUNKS;
        const bool valid = row < group;
        const __nv_bfloat16* src = p.q + (static_cast<size_t>(token) * p.heads + kv_head * group + row) * D + chunk * 8;
        cp_async_16(q_tile + swizzled<D>(row, chunk) * 8, valid ? src : p.q, valid);
    }
    __nv_bfloat16* k_tile = kv_tiles + warp * WARP_TILE;
    __nv_bfloat16* v_tile = k_tile + KEYS * D;
    // Lane r resolves key row r of a tile; the copies fetch the offsets by shuffle.  The offsets of
    // the next tile are resolved while the current tile is multiplied.
    auto resolve = [&](int t) {
        return key_row_offset(p, table, cta_start + t * DECODE_CHUNK + warp * KEYS + lane, lowest, position, kv_head, D);
    };
    auto issue = [&](__nv_bfloat16* tile, const __nv_bfloat16* pages, long long mine) {
#pragma unroll
        for (int pass = 0; pass < KEYS / ROWS_PER_PASS; ++pass) {
            const int row = pass * ROWS_PER_PASS + lane / CHUNKS;
            const long long offset = __shfl_sync(0xffffffffu, mine, row);
            cp_async_16(tile + swizzled<D>(row, lane % CHUNKS) * 8, pages + (offset >= 0 ? offset + (lane % CHUNKS) * 8 : 0),
                        offset >= 0);
        }
    };
    // Tiles of this CTA that hold visible keys.
    const int tiles = min(p.tiles_per_cta, (position - cta_start) / DECODE_CHUNK + 1);
    long long offset_now = resolve(0);
    issue(k_tile, p.k_pages, offset_now);
    cp_async_commit();  // group: queries + keys of tile 0
    issue(v_tile, p.v_pages, offset_now);
    cp_async_commit();  // group: values of tile 0

    float acc[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[n][i] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};
    uint32_t q_frag[D / 16][4];
    const int row_pos[2] = {position, position};

#pragma unroll 1
    for (int t = 0; t < tiles; ++t) {
        const bool more = t + 1 < tiles;
        const long long offset_next = more ? resolve(t + 1) : -1;
        cp_async_wait<1>();  // everything but the newest group (this tile's values) has landed
        if (t == 0) {
            __syncthreads();  // the queries were loaded by all threads
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
                ldmatrix_x4(q_frag[kk], q_tile + swizzled<D>(row, kk * 2 + (lane >> 4)) * 8);
            }
        } else {
            __syncwarp();
        }
        const int first_key = cta_start + t * DECODE_CHUNK + warp * KEYS;
        float scores[KEYS / 8][4];
        scores_tile<D, KEYS>(scores, q_frag, k_tile, lane);
        softmax_step<D, KEYS>(scores, acc, row_max, row_sum, row_pos, first_key, p.window, p.scale_log2, lane);
        __syncwarp();  // every lane has read the keys: the next tile's keys may overwrite them
        if (more) issue(k_tile, p.k_pages, offset_next);
        cp_async_commit();
        cp_async_wait<1>();  // this tile's values have landed (the next keys may still be in flight)
        __syncwarp();
        accumulate_pv<D, KEYS>(acc, scores, v_tile, lane);
        __syncwarp();
        if (more) issue(v_tile, p.v_pages, offset_next);
        cp_async_commit();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 1);
        row_sum[r] += __shfl_xor_sync(0xffffffffu, row_sum[r], 2);
    }
    __syncwarp();  // every lane is done reading this warp's tiles: they now hold the warp's partial

    // Per-warp partial [16][D + 2] float32 over the warp's own K and V tiles.
    float* mine = reinterpret_cast<float*>(k_tile);
    constexpr int STRIDE = D + 2;
    static_assert(16 * STRIDE * 4 <= WARP_TILE * 2, "the partial must fit the warp's tiles");
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = (lane >> 2) + r * 8;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            const int col = n * 8 + 2 * (lane & 3);
            mine[row * STRIDE + col] = acc[n][r * 2];
            mine[row * STRIDE + col + 1] = acc[n][r * 2 + 1];
        }
        if ((lane & 3) == 0) {
            mine[row * STRIDE + D] = row_max[r];
            mine[row * STRIDE + D + 1] = row_sum[r];
        }
    }
    __syncthreads();

    // Merge the four warps and write the CTA's partial.
    for (int idx = threadIdx.x; idx < group * STRIDE; idx += ATTN_THREADS) {
        const int row = idx / STRIDE, col = idx % STRIDE;
        float warp_max[4], total_max = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            warp_max[w] = reinterpret_cast<const float*>(kv_tiles + w * WARP_TILE)[row * STRIDE + D];
            total_max = fmaxf(total_max, warp_max[w]);
        }
        float value = 0.0f;
        if (col == D) {
            value = total_max;
        } else {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                if (warp_max[w] == -INFINITY) continue;
                const float* part = reinterpret_cast<const float*>(kv_tiles + w * WARP_TILE);
                value += part[row * STRIDE + col] * exp2f(warp_max[w] - total_max);
            }
        }
        const int head = kv_head * group + row;
        p.partials[((static_cast<size_t>(entry) * p.heads + head) * p.max_splits + split) * STRIDE + col] = value;
    }
    if (p.counters == nullptr) return;  // a separate kernel merges

    // The CTA that finishes last among those of this (request, KV head) merges all their partials,
    // always in ascending order of the keys, so the result does not depend on who is last.
    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    int first_slot, last_slot;
    decode_slot_range(p, position, lowest, span, first_slot, last_slot);
    if (threadIdx.x == 0) {
        const int active = last_slot - first_slot + 1;  // the CTAs of this (request, KV head) that got here
        int* counter = p.counters + entry * p.kv_heads + kv_head;
        const int ticket = atomicAdd(counter, 1);
        is_last = ticket == active - 1;
        if (is_last) *counter = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int row = warp; row < group; row += 4) merge_head<D>(p, entry, kv_head * group + row, first_slot, last_slot, lane);
}

// One warp merges the partials of one (entry, head) in ascending order of their keys and writes
// the head's output.  Each lane owns D / 32 output elements.  Partials are taken eight at a time,
// all of a batch's loads in flight together; between batches the running maximum rescales what
// has been summed.
template <int D>
__device__ __forceinline__ void merge_head(const AttnParams& p, int entry, int head, int first, int last, int lane) {
    constexpr int STRIDE = D + 2;
    constexpr int PER_LANE = D / 32;
    constexpr int BATCH = 8;
    const float* base = p.partials + (static_cast<size_t>(entry) * p.heads + head) * p.max_splits * STRIDE;
    float value[PER_LANE], denom = 0.0f, total_max = -INFINITY;
#pragma unroll
    for (int i = 0; i < PER_LANE; ++i) value[i] = 0.0f;
    for (int s0 = first; s0 <= last; s0 += BATCH) {
        float m[BATCH], l[BATCH];
        float2 v[BATCH][PER_LANE / 2];
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            const float* part = base + min(s0 + j, last) * STRIDE;
            const float2 tail = __ldcg(reinterpret_cast<const float2*>(part + D));
            m[j] = s0 + j <= last ? tail.x : -INFINITY;
            l[j] = tail.y;
#pragma unroll
            for (int i = 0; i < PER_LANE / 2; ++i) v[j][i] = __ldcg(reinterpret_cast<const float2*>(part + lane * PER_LANE) + i);
        }
        float batch_max = m[0];
#pragma unroll
        for (int j = 1; j < BATCH; ++j) batch_max = fmaxf(batch_max, m[j]);
        if (batch_max == -INFINITY) continue;
        const float new_max = fmaxf(total_max, batch_max);
        const float keep = exp2f(total_max - new_max);  // 0 while nothing has been summed
        total_max = new_max;
        denom *= keep;
#pragma unroll
        for (int i = 0; i < PER_LANE; ++i) value[i] *= keep;
#pragma unroll
        for (int j = 0; j < BATCH; ++j) {
            const float weight = m[j] == -INFINITY ? 0.0f : exp2f(m[j] - new_max);
            denom += l[j] * weight;
#pragma unroll
            for (int i = 0; i < PER_LANE / 2; ++i) {
                value[2 * i] += v[j][i].x * weight;
                value[2 * i + 1] += v[j][i].y * weight;
            }
        }
    }
    const int token = p.cu_tokens[entry];
    __nv_bfloat16* dst = p.out + (static_cast<size_t>(token) * p.heads + head) * D + lane * PER_LANE;
    const float inv = 1.0f / denom;
#pragma unroll
    for (int i = 0; i < PER_LANE; i += 2)
        *reinterpret_cast<uint32_t*>(dst + i) = pack_bf16(value[i] * inv, value[i + 1] * inv);
}

// One warp per (entry, head), for callers that give the decode kernel no arrival counters.
template <int D>
__global__ void __launch_bounds__(128) attention_decode_merge_kernel(AttnParams p, int items) {
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    if (item >= items) return;
    const int listed = item / p.heads, head = item % p.heads;
    const int entry = p.entry_ids ? p.entry_ids[listed] : listed;
    const int position = p.context_lens[entry] - 1;
    const int lowest = p.window > 0 ? max(position - p.window + 1, 0) : 0;
    const int span = p.tiles_per_cta * DECODE_CHUNK;
    int first_slot, last_slot;
    decode_slot_range(p, position, lowest, span, first_slot, last_slot);
    merge_head<D>(p, entry, head, first_slot, last_slot, lane);
}

// ------------------------------------------------- decode kernel with TMA page loads
//
// grid (splits, kv_heads, entries).  The 128-key tiles that a request's query can see are divided
// evenly among the `splits` CTAs of its (request, KV head): the division depends on the request's
// own length (at least two tiles per CTA; CTAs left without tiles exit), so every CTA of a
// request has the same work whatever the longest request of the batch is, and `splits` is chosen
// from the batch size alone.  Built for few instructions per key:
// eight warps of 16 keys each; a warp's keys and values arrive as TMA boxes of whole page rows in
// the 128-byte swizzle, one mbarrier each for K and V; the products are transposed so that the 16
// rows of an mma tile are keys or head dimensions, never padding:
//     S^T [16 keys x 8 heads] = K [16 x D] Q^T [D x 8]
//     O^T [D x 8 heads]      += V^T [D x 16 keys] P^T [16 x 8]
// P^T's B fragments come from S^T's accumulators through movmatrix.  Groups of up to 8 query
// heads, pages of a power of two >= 8 keys.  Rows of V outside the visible range are zeroed in
// shared memory before the second product, so what a reused page still holds there cannot leak.
// With one split the CTA writes the output itself; else partials as in the kernel above.
constexpr int TMA_WARP_KEYS = 16;
constexpr int TMA_MIN_TILES = 2;  // a CTA takes at least this many tiles: a partial more costs more than a tile

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

template <int D, int WARPS>
constexpr int tma_decode_smem_bytes() {
    return 1024 + WARPS * 2 * (D / 64) * TMA_WARP_KEYS * 128 + 8 * D * 2 + WARPS * 2 * 8;
}

template <int D, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, WARPS == 8 ? 3 : 4)
attention_decode_tma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                            AttnParams p) {
    extern __shared__ uint8_t raw_smem[];
    constexpr int TILE_KEYS = WARPS * TMA_WARP_KEYS;       // keys that the CTA takes at a time
    constexpr int THREADS = WARPS * 32;
    constexpr int HALVES = D / 64;                         // 64-element (128-byte) column blocks of a row
    constexpr int HALF_BYTES = TMA_WARP_KEYS * 128;        // one column block of a warp's 16 keys
    constexpr int OPERAND_BYTES = HALVES * HALF_BYTES;     // a warp's K (or V) tile
    constexpr int STRIDE = D + 2;
    static_assert(8 * STRIDE * 4 <= 2 * OPERAND_BYTES, "a warp's partial must fit its tiles");
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_smem) + 1023) & ~uintptr_t(1023));
    __nv_bfloat16* q_tile = reinterpret_cast<__nv_bfloat16*>(smem + WARPS * 2 * OPERAND_BYTES);  // [8][D]
    uint64_t* bars = reinterpret_cast<uint64_t*>(q_tile + 8 * D);

    const int kv_head = blockIdx.y, split = blockIdx.x, splits = gridDim.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    uint8_t* k_tile = smem + warp * 2 * OPERAND_BYTES;
    uint8_t* v_tile = k_tile + OPERAND_BYTES;
    uint64_t* k_bar = bars + warp * 2;
    uint64_t* v_bar = k_bar + 1;
    if (lane == 0) {
        mbar_init(k_bar, 1);
        mbar_init(v_bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // The batch's description (entry list, block table, lengths) was written before the step's
    // first kernel started, so it is read ahead of the wait for the previous kernel; only the
    // queries and the newest keys and values come from that kernel.
    pdl_trigger();
    const int entry = p.entry_ids ? p.entry_ids[blockIdx.z] : blockIdx.z;
    const int* table = p.block_table + static_cast<size_t>(entry) * p.table_width;
    const int position = p.context_lens[entry] - 1;  // the query's position; it sees keys <= position
    const int token = p.cu_tokens[entry];
    const int lowest = p.window > 0 ? max(position - p.window + 1, 0) : 0;
    const int group = p.heads / p.kv_heads;
    // This CTA's tiles [tile, tile_end) among the request's visible ones.
    const int lowest_tile = lowest / TILE_KEYS, tile_count = position / TILE_KEYS - lowest_tile + 1;
    const int per_cta = max((tile_count + splits - 1) / splits, TMA_MIN_TILES);
    const int active = (tile_count + per_cta - 1) / per_cta;  // CTAs of this (request, KV head) with work
    int tile = lowest_tile + split * per_cta;
    const int tile_end = min(tile + per_cta, lowest_tile + tile_count);

    // Lane j holds the page of box j of a run of tiles of this warp: box = (tile, half of the 16
    // keys when pages hold 8).  The run is renewed when the walk leaves it.
    const int box_rows = min(p.page_size, TMA_WARP_KEYS);
    const int boxes = TMA_WARP_KEYS / box_rows;  // 1 or 2
    const int run_tiles = 32 / boxes;
    int run_start = tile, my_page = -1;
    auto load_pages = [&]() {
        const int mine = run_start + lane / boxes;
        const int index = (mine * TILE_KEYS + warp * TMA_WARP_KEYS + (lane % boxes) * box_rows) >> p.page_shift;
        my_page = mine < tile_end && index < p.table_width ? table[index] : -1;
    };
    if (split < active) load_pages();
    __syncwarp();  // the warp's barriers are initialised

    auto first_key_of = [&](int t) { return t * TILE_KEYS + warp * TMA_WARP_KEYS; };
    auto visible = [&](int t) {  // this warp's 16 keys of tile t hold something the query sees
        const int first = first_key_of(t);
        return t < tile_end && first <= position && first + TMA_WARP_KEYS > lowest;
    };
    // Lanes 0 .. boxes * HALVES - 1 each fetch one box of a tile: `box_rows` rows of 64 elements.
    auto issue = [&](int t, uint8_t* dst, const CUtensorMap* map, uint64_t* bar) {
        if (t - run_start >= run_tiles) {
            run_start = t;
            load_pages();
        }
        const int box = lane / HALVES, half = lane % HALVES;
        const int first = first_key_of(t) + box * box_rows;
        const int page = __shfl_sync(0xffffffffu, my_page, (t - run_start) * boxes + (box < boxes ? box : 0));
        const bool wanted = lane < boxes * HALVES && page >= 0 && first <= position && first + box_rows > lowest;
        const uint32_t count = __popc(__ballot_sync(0xffffffffu, wanted));
        if (lane == 0) mbar_expect_tx(bar, count * box_rows * 128);
        __syncwarp();
        if (wanted) {
            const int row = (page * p.kv_heads + kv_head) * p.page_size + (first & (p.page_size - 1));
            tma_load_2d(dst + half * HALF_BYTES + box * box_rows * 128, map, half * 64, row, bar);
        }
    };
    // The keys and values of a tile that does not hold the query's own position were written in
    // earlier steps, which are complete: the CTA's first tile is then on its way before the wait
    // for the previous kernel (which writes the newest key and value, and the queries).
    bool fetching = false;
    if (split < active) {
        while (tile < tile_end && !visible(tile)) ++tile;  // a window may start inside the first tile
        if (tile < tile_end && tile != position / TILE_KEYS) {
            issue(tile, k_tile, &k_map, k_bar);
            issue(tile, v_tile, &v_map, v_bar);
            fetching = true;
        }
    }
    pdl_wait();
    if (split >= active) return;
    if (!fetching && tile < tile_end) {
        issue(tile, k_tile, &k_map, k_bar);
        issue(tile, v_tile, &v_map, v_bar);
    }

    // Queries of the group: rows beyond it are zero.
    for (int idx = threadIdx.x; idx < 8 * (D / 8); idx += THREADS) {
        const int row = idx / (D / 8), chunk = idx % (D / 8);
        uint4 value = make_uint4(0u, 0u, 0u, 0u);
        if (row < group)
            value = *reinterpret_cast<const uint4*>(p.q + (static_cast<size_t>(token) * p.heads + kv_head * group + row) * D + chunk * 8);
        *reinterpret_cast<uint4*>(q_tile + swizzled<D>(row, chunk) * 8) = value;
    }
    __syncthreads();

    uint32_t q_frag[D / 16][2];  // B fragments of Q^T: [k = 16 elements][n = 8 heads]
#pragma unroll
    for (int kk = 0; kk < D / 16; kk += 2) {
        uint32_t r[4];
        ldmatrix_x4(r, q_tile + swizzled<D>(lane & 7, kk * 2 + (lane >> 3)) * 8);
        q_frag[kk][0] = r[0], q_frag[kk][1] = r[1], q_frag[kk + 1][0] = r[2], q_frag[kk + 1][1] = r[3];
    }

    float acc[D / 16][4];  // O^T: rows 16 i + lane / 4 (+ 8), heads 2 (lane % 4) (+ 1)
#pragma unroll
    for (int i = 0; i < D / 16; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;
    float row_max[2] = {-INFINITY, -INFINITY}, row_sum[2] = {0.0f, 0.0f};  // of heads 2 (lane % 4) and + 1
    uint32_t phase = 0;
    bool failed = false;

    // ldmatrix addresses inside a tile: row r, 16-byte chunk c of column block h live at
    // h * HALF_BYTES + r * 128 + ((c ^ (r & 7)) << 4).
    const int k_row = lane & 15, k_hi = lane >> 4;
    const int v_row = (lane & 7) + ((lane >> 4) << 3), v_hi = (lane >> 3) & 1;
#pragma unroll 1
    for (; visible(tile); ++tile) {
        const bool more = visible(tile + 1);
        const int first_key = first_key_of(tile);
        if (!__all_sync(0xffffffffu, mbar_wait(k_bar, phase))) {
            failed = true;
            break;
        }
        float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
            uint32_t a[4];
            const int chunk = kk * 2 + k_hi;
            ldmatrix_x4(a, k_tile + (chunk >> 3) * HALF_BYTES + k_row * 128 + (((chunk & 7) ^ (k_row & 7)) << 4));
            mma_bf16(s, a, q_frag[kk][0], q_frag[kk][1]);
        }
        __syncwarp();  // every lane has read the keys: the next tile's keys may overwrite them
        if (more) issue(tile + 1, k_tile, &k_map, k_bar);

        // Online softmax over the 16 keys, per head column.
        const int key0 = first_key + (lane >> 2);
        const bool seen0 = key0 <= position && key0 >= lowest, seen1 = key0 + 8 <= position && key0 + 8 >= lowest;
        float rescale[2];
        uint32_t packed[2];
        {
            float prob[4];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const float a = seen0 ? s[j] * p.scale_log2 : -INFINITY;
                const float b = seen1 ? s[j + 2] * p.scale_log2 : -INFINITY;
                float tile_max = fmaxf(a, b);
                tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
                tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 8));
                tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
                const float new_max = fmaxf(row_max[j], tile_max);
                const float base = new_max == -INFINITY ? 0.0f : new_max;  // a head that has seen nothing yet
                rescale[j] = exp2f(row_max[j] - base);                     // 0 while row_max is -inf
                row_max[j] = new_max;
                prob[j] = exp2f(a - base);
                prob[j + 2] = exp2f(b - base);
                row_sum[j] = row_sum[j] * rescale[j] + prob[j] + prob[j + 2];
            }
            packed[0] = movmatrix_trans(pack_bf16(prob[0], prob[1]));  // keys 0-7 of the tile
            packed[1] = movmatrix_trans(pack_bf16(prob[2], prob[3]));  // keys 8-15
        }
        if (__any_sync(0xffffffffu, rescale[0] != 1.0f || rescale[1] != 1.0f)) {
#pragma unroll
            for (int i = 0; i < D / 16; ++i) {
                acc[i][0] *= rescale[0], acc[i][2] *= rescale[0];
                acc[i][1] *= rescale[1], acc[i][3] *= rescale[1];
            }
        }
        if (!__all_sync(0xffffffffu, mbar_wait(v_bar, phase))) {
            failed = true;
            break;
        }
        const bool ragged = first_key < lowest || first_key + TMA_WARP_KEYS - 1 > position;
        if (ragged) {  // zero the value rows that the query must not see (or that were never fetched)
            for (int idx = lane; idx < TMA_WARP_KEYS * HALVES * 8; idx += 32) {
                const int row = idx / (HALVES * 8), rest = idx % (HALVES * 8);
                const int key = first_key + row;
                if (key < lowest || key > position)
                    *reinterpret_cast<uint4*>(v_tile + (rest >> 3) * HALF_BYTES + row * 128 + ((rest & 7) << 4)) =
                        make_uint4(0u, 0u, 0u, 0u);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // before a TMA box lands there again
            __syncwarp();
        }
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            uint32_t a[4];
            const int chunk = i * 2 + v_hi;
            ldmatrix_x4_trans(a, v_tile + (chunk >> 3) * HALF_BYTES + v_row * 128 + (((chunk & 7) ^ (v_row & 7)) << 4));
            mma_bf16(acc[i], a, packed[0], packed[1]);
        }
        __syncwarp();
        if (more) issue(tile + 1, v_tile, &v_map, v_bar);
        phase ^= 1u;
    }
    if (failed && lane == 0) atomicCAS(&g_decode_error, 0, 1);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        row_sum[j] += __shfl_xor_sync(0xffffffffu, row_sum[j], 4);
        row_sum[j] += __shfl_xor_sync(0xffffffffu, row_sum[j], 8);
        row_sum[j] += __shfl_xor_sync(0xffffffffu, row_sum[j], 16);
    }
    __syncwarp();  // every lane is done reading this warp's tiles: they now hold the warp's partial

    // Per-warp partial [8 heads][D + 2] float32 over the warp's own K and V tiles.
    float* mine = reinterpret_cast<float*>(k_tile);
    {
        const int head = 2 * (lane & 3), dim = lane >> 2;
#pragma unroll
        for (int i = 0; i < D / 16; ++i) {
            mine[head * STRIDE + i * 16 + dim] = acc[i][0];
            mine[(head + 1) * STRIDE + i * 16 + dim] = acc[i][1];
            mine[head * STRIDE + i * 16 + dim + 8] = acc[i][2];
            mine[(head + 1) * STRIDE + i * 16 + dim + 8] = acc[i][3];
        }
        if (lane < 4) {
            mine[head * STRIDE + D] = row_max[0], mine[head * STRIDE + D + 1] = row_sum[0];
            mine[(head + 1) * STRIDE + D] = row_max[1], mine[(head + 1) * STRIDE + D + 1] = row_sum[1];
        }
    }
    __syncthreads();

    // Merge the eight warps (ascending keys): the CTA's partial, or with one split the output.
    const bool direct = splits == 1;
    for (int idx = threadIdx.x; idx < group * STRIDE; idx += THREADS) {
        const int row = idx / STRIDE, col = idx % STRIDE;
        float weight[WARPS], total_max = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            weight[w] = reinterpret_cast<const float*>(smem + w * 2 * OPERAND_BYTES)[row * STRIDE + D];
            total_max = fmaxf(total_max, weight[w]);
        }
        float value = 0.0f, denom = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            if (weight[w] == -INFINITY) continue;
            const float* part = reinterpret_cast<const float*>(smem + w * 2 * OPERAND_BYTES);
            const float scale = exp2f(weight[w] - total_max);
            value += part[row * STRIDE + (col == D ? D + 1 : col)] * scale;
            if (direct) denom += part[row * STRIDE + D + 1] * scale;
        }
        if (col == D) value = total_max;
        const int head = kv_head * group + row;
        if (!direct)
            p.partials[((static_cast<size_t>(entry) * p.heads + head) * p.max_splits + split) * STRIDE + col] = value;
        else if (col < D)
            p.out[(static_cast<size_t>(token) * p.heads + head) * D + col] = __float2bfloat16(value / denom);
    }
    if (direct || p.counters == nullptr) return;  // nothing to merge, or a separate kernel merges

    __shared__ int is_last;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        int* counter = p.counters + entry * p.kv_heads + kv_head;
        const int ticket = atomicAdd(counter, 1);
        is_last = ticket == active - 1;
        if (is_last) *counter = 0;  // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int row = warp; row < group; row += WARPS) merge_head<D>(p, entry, kv_head * group + row, 0, active - 1, lane);
}

// One warp per (entry, head) merges the partials of the kernel above when it got no counters.
template <int D, int WARPS>
__global__ void __launch_bounds__(128) attention_decode_tma_merge_kernel(AttnParams p, int items) {
    constexpr int TILE_KEYS = WARPS * TMA_WARP_KEYS;
    const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    pdl_trigger();
    pdl_wait();
    if (item >= items) return;
    const int listed = item / p.heads, head = item % p.heads;
    const int entry = p.entry_ids ? p.entry_ids[listed] : listed;
    const int position = p.context_lens[entry] - 1;
    const int lowest = p.window > 0 ? max(position - p.window + 1, 0) : 0;
    const int tile_count = position / TILE_KEYS - lowest / TILE_KEYS + 1;
    const int per_cta = max((tile_count + p.max_splits - 1) / p.max_splits, TMA_MIN_TILES);
    merge_head<D>(p, entry, head, 0, (tile_count + per_cta - 1) / per_cta - 1, lane);
}

// -------------------------------------------------------------------------------- host

template <int D>
static int launch_portions(const AttnParams& p, int entries, int max_new_tokens, cudaStream_t stream) {
    constexpr int SMEM = (BLOCK_M * D + 4 * BLOCK_KEYS * D) * 2;
    auto kernel = attention_portions_kernel<D>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, SMEM)) return e;
    dim3 grid((max_new_tokens + BLOCK_M - 1) / BLOCK_M, p.heads, entries);
    return launch_kernel(kernel, grid, ATTN_THREADS, SMEM, stream, p);
}

template <int D>
static int launch_decode(const AttnParams& p, int entries, cudaStream_t stream) {
    constexpr int SMEM = (16 * D + 8 * DECODE_WARP_KEYS * D) * 2;
    auto kernel = attention_decode_kernel<D>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, SMEM)) return e;
    dim3 grid(p.max_splits, p.kv_heads, entries);
    const int status = launch_kernel(kernel, grid, ATTN_THREADS, SMEM, stream, p);
    if (status != 0 || p.counters != nullptr) return status;
    const int items = entries * p.heads;
    return launch_kernel(attention_decode_merge_kernel<D>, (items + 3) / 4, 128, 0, stream, p, items);
}

template <int D, int WARPS>
static int launch_decode_tma(const CUtensorMap& k_map, const CUtensorMap& v_map, const AttnParams& p, int entries,
                             cudaStream_t stream) {
    constexpr int SMEM = tma_decode_smem_bytes<D, WARPS>();
    auto kernel = attention_decode_tma_kernel<D, WARPS>;
    static SharedMemoryOptIn opt_in;
    if (const int e = opt_in(kernel, SMEM)) return e;
    dim3 grid(p.max_splits, p.kv_heads, entries);
    const int status = launch_kernel(kernel, grid, WARPS * 32, SMEM, stream, k_map, v_map, p);
    if (status != 0 || p.counters != nullptr || p.max_splits == 1) return status;
    const int items = entries * p.heads;
    return launch_kernel(attention_decode_tma_merge_kernel<D, WARPS>, (items + 3) / 4, 128, 0, stream, p, items);
}

static int shift_of(int page_size) {
    for (int shift = 0; shift < 31; ++shift)
        if ((1 << shift) == page_size) return shift;
    return -1;
}

static bool sizes_ok(int head_dim, int heads, int kv_heads) {
    return (head_dim == 64 || head_dim == 128) && kv_heads > 0 && heads % kv_heads == 0;
}

// Any mix of portions and single tokens.  grid.x covers the longest portion.  `entry_ids` lists
// the batch entries to run (`entries` of them), or is null for all of them in order; the partial
// results and counters of the decode kernel are indexed by the entry's number in the batch.
ME_EXPORT int me_attention_portions_bf16(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                         const int* cu_tokens, const int* context_lens, void* out, float scale,
                                         int entries, int max_new_tokens, int heads, int kv_heads, int head_dim,
                                         int page_size, int table_width, int window, const int* entry_ids,
                                         cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (!sizes_ok(head_dim, heads, kv_heads)) return ME_ERR_UNSUPPORTED;
    AttnParams p{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_pages),
                 static_cast<const __nv_bfloat16*>(v_pages), block_table, cu_tokens, context_lens,
                 static_cast<__nv_bfloat16*>(out), nullptr, nullptr, entry_ids, scale * LOG2E, heads, kv_heads,
                 page_size, table_width, window, 0, shift_of(page_size), 1};
    return head_dim == 128 ? launch_portions<128>(p, entries, max_new_tokens, stream)
                           : launch_portions<64>(p, entries, max_new_tokens, stream);
}

// Every entry brings exactly one token.  `partials` is scratch of
// entries * heads * max_splits * (head_dim + 2) floats; a CTA walks `tiles_per_cta` (1..8) tiles
// of 128 keys, and max_splits covers the longest context that this launch may meet:
// ceil(max_context / (128 * tiles_per_cta)).  `counters` is entries * kv_heads ints that are zero
// before the launch (the kernel leaves them zero again): the last CTA of a (request, KV head) then
// merges the partials itself; with null a second kernel does.
ME_EXPORT int me_attention_decode_bf16_tiled(const void* q, const void* k_pages, const void* v_pages,
                                             const int* block_table, const int* cu_tokens, const int* context_lens,
                                             void* out, float* partials, int* counters, float scale, int entries, int max_splits,
                                             int tiles_per_cta, int heads, int kv_heads, int head_dim, int page_size,
                                             int table_width, int window, const int* entry_ids, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (!sizes_ok(head_dim, heads, kv_heads) || heads / kv_heads > 16 || max_splits < 1) return ME_ERR_UNSUPPORTED;
    if (tiles_per_cta < 1 || tiles_per_cta > MAX_DECODE_TILES) return ME_ERR_ARGUMENT;
    AttnParams p{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_pages),
                 static_cast<const __nv_bfloat16*>(v_pages), block_table, cu_tokens, context_lens,
                 static_cast<__nv_bfloat16*>(out), partials, counters, entry_ids, scale * LOG2E, heads, kv_heads,
                 page_size, table_width, window, max_splits, shift_of(page_size), tiles_per_cta};
    return head_dim == 128 ? launch_decode<128>(p, entries, stream) : launch_decode<64>(p, entries, stream);
}

// Every entry brings one token, through the TMA kernel.  `k_map` and `v_map` are 128-byte TMA
// descriptors of the page arrays seen as [(pages * kv_heads * page_size)][head_dim] with boxes of
// min(page_size, 16) rows by 64 elements in the 128-byte swizzle.  `splits` CTAs share the keys
// of one (request, KV head); `partials` holds entries * heads * splits * (head_dim + 2) floats and
// `counters` entries * kv_heads zeros (both unused with one split).  Groups of up to 8 query
// heads, pages of a power of two of at least 8 keys; other sizes are refused.
// `warps`: 8 (tiles of 128 keys, three CTAs to an SM) or 6 (tiles of 96 keys, four to an SM).
ME_EXPORT int me_attention_decode_bf16_tma(const void* k_map, const void* v_map, const void* q, const int* block_table,
                                           const int* cu_tokens, const int* context_lens, void* out, float* partials,
                                           int* counters, float scale, int entries, int splits, int warps, int heads,
                                           int kv_heads, int head_dim, int page_size, int table_width, int window,
                                           const int* entry_ids, cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (!sizes_ok(head_dim, heads, kv_heads) || heads / kv_heads > 8) return ME_ERR_UNSUPPORTED;
    if (shift_of(page_size) < 3) return ME_ERR_UNSUPPORTED;
    if (splits < 1 || splits > 65535 || (splits > 1 && partials == nullptr)) return ME_ERR_ARGUMENT;
    if (warps != 8 && warps != 6) return ME_ERR_ARGUMENT;
    AttnParams p{static_cast<const __nv_bfloat16*>(q), nullptr, nullptr, block_table, cu_tokens, context_lens,
                 static_cast<__nv_bfloat16*>(out), partials, counters, entry_ids, scale * LOG2E, heads, kv_heads,
                 page_size, table_width, window, splits, shift_of(page_size), 0};
    CUtensorMap maps[2];
    memcpy(&maps[0], k_map, sizeof(CUtensorMap));
    memcpy(&maps[1], v_map, sizeof(CUtensorMap));
    if (warps == 8)
        return head_dim == 128 ? launch_decode_tma<128, 8>(maps[0], maps[1], p, entries, stream)
                               : launch_decode_tma<64, 8>(maps[0], maps[1], p, entries, stream);
    return head_dim == 128 ? launch_decode_tma<128, 6>(maps[0], maps[1], p, entries, stream)
                           : launch_decode_tma<64, 6>(maps[0], maps[1], p, entries, stream);
}

// First failure that a decode kernel recorded since the last call, or 0: 1 = a wait that ran out,
// 2 = `max_splits` did not cover a context (its output lacks the keys beyond).
ME_EXPORT int me_attention_bf16_take_error(int* code) {
    int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbol(code, g_decode_error, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (*code != 0) e = cudaMemcpyToSymbol(g_decode_error, &zero, sizeof(int));
    return static_cast<int>(e);
}

// The same with one tile of 128 keys per CTA: max_splits = ceil(max_context / 128).
ME_EXPORT int me_attention_decode_bf16(const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                       const int* cu_tokens, const int* context_lens, void* out, float* partials,
                                       float scale, int entries, int max_splits, int heads, int kv_heads, int head_dim,
                                       int page_size, int table_width, int window, cudaStream_t stream) {
    return me_attention_decode_bf16_tiled(q, k_pages, v_pages, block_table, cu_tokens, context_lens, out, partials,
                                          nullptr, scale, entries, max_splits, 1, heads, kv_heads, head_dim, page_size,
                                          table_width, window, nullptr, stream);
}

// ------------------------------------------------- decode attention without allocation

#include "attention_bf16_noalloc.h"

// Scratch of the allocation-free entry point: partial results of the split decode kernel.
// It lives in the library's image, so every GPU on which this library is loaded holds these
// 8 MiB from the first use of the library until the process exits.
static __device__ __align__(256) float g_noalloc_partials[ME_NOALLOC_MAX_PARTIAL_FLOATS];

// In host code `g_noalloc_partials` names a host-side shadow of the device array, not device
// memory, so it must never be handed to a kernel.  The device address is looked up once per
// device, with that device current, and remembered here.
static float* g_noalloc_address[ME_NOALLOC_MAX_DEVICES] = {};

ME_EXPORT int me_attention_decode_bf16_noalloc(const void* q, const void* k_pages, const void* v_pages,
                                               const int* block_table, const int* cu_tokens, const int* context_lens,
                                               void* out, float scale, int entries, int max_splits, int heads,
                                               int kv_heads, int head_dim, int page_size, int table_width, int window,
                                               cudaStream_t stream) {
    if (entries <= 0) return 0;
    if (max_splits < 1 || heads < 1) return ME_ERR_ARGUMENT;
    const long long needed = static_cast<long long>(entries) * heads * max_splits * (head_dim + 2);
    if (needed > ME_NOALLOC_MAX_PARTIAL_FLOATS) return ME_ERR_NOALLOC_TOO_LARGE;
    int device = -1;
    cudaError_t status = cudaGetDevice(&device);
    if (status != cudaSuccess) return static_cast<int>(status);
    if (device < 0 || device >= ME_NOALLOC_MAX_DEVICES) return ME_ERR_ARGUMENT;
    if (g_noalloc_address[device] == nullptr) {
        void* address = nullptr;
        status = cudaGetSymbolAddress(&address, g_noalloc_partials);
        if (status != cudaSuccess) return static_cast<int>(status);
        g_noalloc_address[device] = static_cast<float*>(address);
    }
    return me_attention_decode_bf16(q, k_pages, v_pages, block_table, cu_tokens, context_lens, out,
                                    g_noalloc_address[device], scale, entries, max_splits, heads, kv_heads, head_dim,
                                    page_size, table_width, window, stream);
}
