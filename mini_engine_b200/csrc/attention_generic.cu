// Causal grouped-query attention over the paged cache for any head size: one warp per
// (token, query head).  It is the attention of the float32 path and of bfloat16 head sizes
// that the tensor-core kernels do not take.
//
// Formula (YuvGev00/mini-engine, src/mini_engine/attention.py:84-86,160-175 and the online
// softmax of src/mini_engine/triton_attention.py:56-82): query head h reads KV head h / group;
// s = (q . k) * scale; the query at position p sees keys at positions <= p (and > p - window
// when a window is given); out = softmax(s) V.
//
// Keys are visited in tiles of 32 whose boundaries are multiples of 32 in *absolute position*
// and are combined in ascending order, so the arithmetic of a query depends only on its own
// position: the same bits come out whether the token arrived in a whole prompt, in a
// two-token portion or as a decoded token, and whatever else is in the batch.
#include "common.cuh"

struct AttnArgs {
    const void* q;         // [tokens][heads][head_dim]
    const void* k_pages;   // [pages][kv_heads][page_size][head_dim]
    const void* v_pages;
    const int* block_table;  // [entries][table_width]
    const int* entry_of_token;
    const int* positions;
    void* out;  // [tokens][heads][head_dim]
    float scale;
    int tokens, heads, kv_heads, head_dim, page_size, table_width, window;
};

constexpr int ATTN_WARPS = 4;
constexpr int MAX_DIM_PER_LANE = 16;  // head_dim <= 512

template <typename T>
__global__ void __launch_bounds__(ATTN_WARPS * 32) paged_attention_generic_kernel(AttnArgs a) {
    extern __shared__ float q_staged[];  // [ATTN_WARPS][head_dim]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = static_cast<long long>(blockIdx.x) * ATTN_WARPS + warp;
    if (item >= static_cast<long long>(a.tokens) * a.heads) return;
    const int token = static_cast<int>(item / a.heads), head = static_cast<int>(item % a.heads);
    const int d = a.head_dim;
    pdl_trigger();
    pdl_wait();
    const int kv_head = head / (a.heads / a.kv_heads);
    const int position = a.positions[token];
    const int* table = a.block_table + static_cast<size_t>(a.entry_of_token[token]) * a.table_width;
    const T* k_pages = static_cast<const T*>(a.k_pages);
    const T* v_pages = static_cast<const T*>(a.v_pages);

    float* q = q_staged + warp * d;
    const T* q_src = static_cast<const T*>(a.q) + (static_cast<size_t>(token) * a.heads + head) * d;
    for (int i = lane; i < d; i += 32) q[i] = to_float(q_src[i]);
    __syncwarp();

    const int lowest = a.window > 0 ? max(position - a.window + 1, 0) : 0;
    float running_max = -INFINITY, denom = 0.0f;
    float acc[MAX_DIM_PER_LANE];
#pragma unroll
    for (int i = 0; i < MAX_DIM_PER_LANE; ++i) acc[i] = 0.0f;

    for (int tile = (lowest / 32) * 32; tile <= position; tile += 32) {
        const int key = tile + lane;
        const bool valid = key >= lowest && key <= position;
        long long base = -1;  // element offset of this lane's key row, -1 when masked
        if (valid) {
            const int page = table[key / a.page_size];
            if (page >= 0)
                base = ((static_cast<long long>(page) * a.kv_heads + kv_head) * a.page_size + key % a.page_size) * d;
        }
        float score = -INFINITY;
        if (base >= 0) {
            const T* k_row = k_pages + base;
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(q[i], to_float(k_row[i]), dot);
            score = dot * a.scale;
        }
        const float new_max = fmaxf(running_max, warp_max(score));
        if (new_max == -INFINITY) continue;  // nothing visible yet (uniform across the warp)
        const float p = base >= 0 ? expf(score - new_max) : 0.0f;
        const float rescale = expf(running_max - new_max);  // 0 on the first tile (exp(-inf))
        denom = denom * rescale + warp_sum(p);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < MAX_DIM_PER_LANE; ++i) acc[i] *= rescale;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const long long bj = __shfl_sync(0xffffffffu, base, j);
            if (bj < 0) continue;  // uniform across the warp
            const T* v_row = v_pages + bj;
#pragma unroll
            for (int i = 0; i < MAX_DIM_PER_LANE; ++i) {
                const int e = lane + 32 * i;
                if (e < d) acc[i] = fmaf(pj, to_float(v_row[e]), acc[i]);
            }
        }
    }
    T* out = static_cast<T*>(a.out) + (static_cast<size_t>(token) * a.heads + head) * d;
    const float inv = 1.0f / denom;
#pragma unroll
    for (int i = 0; i < MAX_DIM_PER_LANE; ++i) {
        const int e = lane + 32 * i;
        if (e < d) out[e] = from_float<T>(acc[i] * inv);
    }
}

ME_EXPORT int me_paged_attention_generic(const void* q, const void* k_pages, const void* v_pages,
                                         const int* block_table, const int* entry_of_token,
                                         const int* positions, void* out, int type, float scale, int tokens,
                                         int heads, int kv_heads, int head_dim, int page_size, int table_width,
                                         int window, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim > 32 * MAX_DIM_PER_LANE || heads % kv_heads) return ME_ERR_UNSUPPORTED;
    AttnArgs a{q, k_pages, v_pages, block_table, entry_of_token, positions, out, scale,
               tokens, heads, kv_heads, head_dim, page_size, table_width, window};
    const long long items = static_cast<long long>(tokens) * heads;
    const int blocks = static_cast<int>((items + ATTN_WARPS - 1) / ATTN_WARPS);
    const size_t smem = static_cast<size_t>(ATTN_WARPS) * head_dim * sizeof(float);
    if (type == ME_BF16)
        return launch_kernel(paged_attention_generic_kernel<__nv_bfloat16>, blocks, ATTN_WARPS * 32, smem, stream, a);
    return launch_kernel(paged_attention_generic_kernel<float>, blocks, ATTN_WARPS * 32, smem, stream, a);
}
