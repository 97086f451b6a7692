// Memory-bound kernels between the matrix products: embedding lookup, residual sum fused
// with RMSNorm, the SwiGLU gate on partial sums, and per-head q/k norm + rotary + cache
// write.  Statistics, angles and sums are 32-bit; outputs are rounded once.
//
// Formulas restate YuvGev00/mini-engine: src/mini_engine/model.py:59-69 (RMSNorm),
// :72-90 (rotary, rotate-half), :113-116 (norm before rotation, v untouched), :130 (SwiGLU),
// src/mini_engine/attention.py:118-121 (new K/V go to their slots before attention reads).
#include "common.cuh"

#include <algorithm>

// ------------------------------------------------------------------------------ embedding

// One block per token.  VEC: the width is a multiple of 8 and both pointers are 16-byte aligned;
// a thread then moves eight elements per step.
template <typename T, bool VEC>
__global__ void embedding_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                 float* __restrict__ out, int hidden, int vocab, float multiplier) {
    const int token = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int id = ids[token];
    float* row_out = out + static_cast<size_t>(token) * hidden;
    if (id < 0 || id >= vocab) {  // the host validates ids; never read outside the table
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) row_out[i] = 0.0f;
        return;
    }
    const T* row = table + static_cast<size_t>(id) * hidden;
    if (VEC) {
        for (int i = threadIdx.x * 8; i < hidden; i += blockDim.x * 8) {
            float v[8];
            if (sizeof(T) == 2) {
                const uint4 raw = *reinterpret_cast<const uint4*>(row + i);
                const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = __bfloat1622float2(pairs[j]);
                    v[2 * j] = f.x, v[2 * j + 1] = f.y;
                }
            } else {
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = to_float(row[i + j]);
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] *= multiplier;  // 1 for a model without embedding scaling: exact
            *reinterpret_cast<float4*>(row_out + i) = make_float4(v[0], v[1], v[2], v[3]);
            *reinterpret_cast<float4*>(row_out + i + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) row_out[i] = to_float(row[i]) * multiplier;
    }
}

// out[t][:] = table[ids[t]][:] * multiplier, widened to float32.
ME_EXPORT int me_embedding(const void* table, int table_type, const int* ids, float* out, int tokens,
                           int hidden, int vocab, float multiplier, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const bool vec = hidden % 8 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
    const int threads = vec ? std::min(512, std::max(32, (hidden / 8 + 31) / 32 * 32)) : (hidden >= 1024 ? 256 : 128);
    if (table_type == ME_BF16) {
        const auto* t = static_cast<const __nv_bfloat16*>(table);
        return vec ? launch_kernel(embedding_kernel<__nv_bfloat16, true>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier)
                   : launch_kernel(embedding_kernel<__nv_bfloat16, false>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier);
    }
    const auto* t = static_cast<const float*>(table);
    return vec ? launch_kernel(embedding_kernel<float, true>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier)
               : launch_kernel(embedding_kernel<float, false>, tokens, threads, 0, stream, t, ids, out, hidden, vocab, multiplier);
}

// ------------------------------------------------------------- what a head may do to logits

// logits[r][v] = cap(logits[r][v] * scale + bias[v]) with cap(y) = soft_cap * tanh(y / soft_cap) when
// soft_cap > 0, in place; `bias` may be null.  For heads that have a bias, a logit scale or a
// soft cap; a plain head never launches this.
__global__ void logits_finish_kernel(float* __restrict__ logits, const float* __restrict__ bias, float scale,
                                     float soft_cap, int vocab) {
    pdl_trigger();
    pdl_wait();
    float* row = logits + static_cast<size_t>(blockIdx.y) * vocab;
    for (int v = blockIdx.x * blockDim.x + threadIdx.x; v < vocab; v += gridDim.x * blockDim.x) {
        float y = row[v] * scale;
        if (bias != nullptr) y += bias[v];
        if (soft_cap > 0.0f) y = soft_cap * tanhf(y / soft_cap);
        row[v] = y;
    }
}

ME_EXPORT int me_logits_finish(float* logits, const float* bias, float scale, float soft_cap, int rows, int vocab,
                               cudaStream_t stream) {
    if (rows <= 0 || vocab <= 0) return 0;
    if (rows > 65535) return ME_ERR_ARGUMENT;
    const int blocks = std::min((vocab + 255) / 256, 1024);
    return launch_kernel(logits_finish_kernel, dim3(blocks, rows), 256, 0, stream, logits, bias, scale, soft_cap, vocab);
}

// --------------------------------------------------------------- residual sum + RMSNorm

constexpr int MAX_UNROLLED_SPLITS = 8;

__device__ __forceinline__ void store4(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
__device__ __forceinline__ void store4(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&lo);
    packed.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = packed;
}

// One block per output row.  x_row = x[src] + sum_s pending[s][src] (ascending s); when
// `rows` is null the sum is written back to x (the residual stream advances), otherwise only
// the listed rows are read and x is left alone.  out = weight * x_row * rsqrt(mean(x_row^2) + eps).
// VEC: hidden is a multiple of 4 and every pointer is 16-byte aligned; all loads of a thread are
// then issued before any of them is used, which is what matters when only a few rows run.
//
// The sum of squares is defined over LANES "lanes" (256, 512 or 1024, chosen from the width
// alone): lane v adds the squares of its columns 4v..4v+3 (+ 4 LANES j) in ascending order, the 32
// lanes of a warp are added by a butterfly, and the warps' sums in ascending order.  A block of
// THREADS = LANES threads has one lane per thread (every load of a short row in flight at once:
// few rows); a block of THREADS < LANES threads plays LANES / THREADS lanes per thread with one
// partial sum each, which gives the same bits with more blocks per SM (many rows).
template <typename OutT, bool VEC, int LANES, int THREADS>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ pending, int splits, size_t split_stride,
                   const float* __restrict__ weight, float eps, OutT* __restrict__ out,
                   const int* __restrict__ rows, int hidden) {
    constexpr int PLAYED = LANES / THREADS;  // lanes per thread
    extern __shared__ float row_cache[];  // [hidden]
    __shared__ float warp_partial[LANES / 32];
    const int out_row = blockIdx.x;
    pdl_trigger();
    // The norm's weight and the step's row list do not come from the previous kernel: fetch them
    // ahead of the wait.
    const int src = rows ? rows[out_row] : out_row;
    float4 first_weight = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (VEC && threadIdx.x * 4 < hidden) first_weight = *reinterpret_cast<const float4*>(weight + threadIdx.x * 4);
    pdl_wait();
    float* x_row = x + static_cast<size_t>(src) * hidden;
    const float* pending_row = pending + static_cast<size_t>(src) * hidden;
    const bool write_back = !rows && splits > 0;
    float sum_sq[PLAYED];
#pragma unroll
    for (int k = 0; k < PLAYED; ++k) sum_sq[k] = 0.0f;
    if (VEC && splits <= MAX_UNROLLED_SPLITS) {
        for (int base = 0; base < hidden; base += LANES * 4) {
#pragma unroll
            for (int k = 0; k < PLAYED; ++k) {
                const int i = base + (k * THREADS + threadIdx.x) * 4;
                if (i >= hidden) continue;
                float4 v = *reinterpret_cast<const float4*>(x_row + i);
                float4 part[MAX_UNROLLED_SPLITS];
#pragma unroll
                for (int s = 0; s < MAX_UNROLLED_SPLITS; ++s)
                    if (s < splits) part[s] = *reinterpret_cast<const float4*>(pending_row + s * split_stride + i);
#pragma unroll
                for (int s = 0; s < MAX_UNROLLED_SPLITS; ++s)
                    if (s < splits) { v.x += part[s].x; v.y += part[s].y; v.z += part[s].z; v.w += part[s].w; }
                *reinterpret_cast<float4*>(row_cache + i) = v;
                if (write_back) *reinterpret_cast<float4*>(x_row + i) = v;
                sum_sq[k] = fmaf(v.x, v.x, sum_sq[k]);
                sum_sq[k] = fmaf(v.y, v.y, sum_sq[k]);
                sum_sq[k] = fmaf(v.z, v.z, sum_sq[k]);
                sum_sq[k] = fmaf(v.w, v.w, sum_sq[k]);
            }
        }
    } else {
        for (int base = 0; base < hidden; base += LANES) {
#pragma unroll
            for (int k = 0; k < PLAYED; ++k) {
                const int i = base + k * THREADS + threadIdx.x;
                if (i >= hidden) continue;
                float v = x_row[i];
                for (int s = 0; s < splits; ++s) v += pending_row[s * split_stride + i];
                row_cache[i] = v;
                if (write_back) x_row[i] = v;
                sum_sq[k] = fmaf(v, v, sum_sq[k]);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < PLAYED; ++k) {
        const float warp_total = warp_sum(sum_sq[k]);
        if ((threadIdx.x & 31) == 0) warp_partial[k * (THREADS / 32) + (threadIdx.x >> 5)] = warp_total;
    }
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int w = 0; w < LANES / 32; ++w) total += warp_partial[w];
    const float inv = rsqrtf(total / static_cast<float>(hidden) + eps);
    OutT* out_ptr = out + static_cast<size_t>(out_row) * hidden;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < hidden; i += THREADS * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row_cache + i);
            const float4 w = i == threadIdx.x * 4 ? first_weight : *reinterpret_cast<const float4*>(weight + i);
            store4(out_ptr + i, make_float4(w.x * (v.x * inv), w.y * (v.y * inv), w.z * (v.z * inv), w.w * (v.w * inv)));
        }
    } else {
        for (int i = threadIdx.x; i < hidden; i += THREADS)
            out_ptr[i] = from_float<OutT>(weight[i] * (row_cache[i] * inv));
    }
}

template <typename OutT, bool VEC, int LANES, int THREADS>
static int launch_add_rmsnorm_threads(float* x, const float* pending, int splits, size_t split_stride,
                                      const float* weight, float eps, OutT* out, const int* rows, int count, int hidden,
                                      cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(hidden) * sizeof(float);
    auto kernel = add_rmsnorm_kernel<OutT, VEC, LANES, THREADS>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(kernel, count, THREADS, smem, stream, x, pending, splits, split_stride, weight, eps, out,
                         rows, hidden);
}

// Few rows: one lane per thread.  Many rows: 256 threads per row, more rows per SM.  The lanes
// (hence the bits of the result) depend on the width alone.
constexpr int NORM_MANY_ROWS = 256;

template <typename OutT, bool VEC, int LANES>
static int launch_add_rmsnorm_lanes(float* x, const float* pending, int splits, size_t split_stride, const float* weight,
                                    float eps, OutT* out, const int* rows, int count, int hidden, cudaStream_t stream) {
    if (count >= NORM_MANY_ROWS)
        return launch_add_rmsnorm_threads<OutT, VEC, LANES, 256>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream);
    return launch_add_rmsnorm_threads<OutT, VEC, LANES, LANES>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream);
}

template <typename OutT, bool VEC>
static int launch_add_rmsnorm(float* x, const float* pending, int splits, size_t split_stride, const float* weight,
                              float eps, OutT* out, const int* rows, int count, int hidden, cudaStream_t stream) {
    if (VEC && hidden > 2048)
        return launch_add_rmsnorm_lanes<OutT, VEC, 1024>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream);
    if (VEC && hidden > 1024)
        return launch_add_rmsnorm_lanes<OutT, VEC, 512>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream);
    return launch_add_rmsnorm_lanes<OutT, VEC, 256>(x, pending, splits, split_stride, weight, eps, out, rows, count, hidden, stream);
}

static bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

ME_EXPORT int me_add_rmsnorm(float* x, const float* pending, int splits, long long split_stride,
                             const float* weight, float eps, void* out, int out_type, const int* rows,
                             int count, int hidden, cudaStream_t stream) {
    if (count <= 0) return 0;
    if (static_cast<size_t>(hidden) * sizeof(float) > 200 * 1024) return ME_ERR_UNSUPPORTED;
    // Which path runs depends on the width and on the alignment of the engine's persistent
    // buffers only, never on the batch, so a row's statistics are the same bits in every step.
    const bool vec = hidden % 4 == 0 && aligned16(x) && aligned16(weight) && aligned16(out) &&
                     (pending == nullptr || (aligned16(pending) && split_stride % 4 == 0));
    const size_t stride = static_cast<size_t>(split_stride);
    if (out_type == ME_BF16) {
        auto* o = static_cast<__nv_bfloat16*>(out);
        return vec ? launch_add_rmsnorm<__nv_bfloat16, true>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream)
                   : launch_add_rmsnorm<__nv_bfloat16, false>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream);
    }
    auto* o = static_cast<float*>(out);
    return vec ? launch_add_rmsnorm<float, true>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream)
               : launch_add_rmsnorm<float, false>(x, pending, splits, stride, weight, eps, o, rows, count, hidden, stream);
}

// --------------------------------------------------------------------------------- SwiGLU

// partial[s][t][0..inter) are gate sums, [inter..2*inter) up sums.  out = silu(gate) * up.
template <typename OutT>
__global__ void swiglu_kernel(const float* __restrict__ partial, int splits, size_t split_stride,
                              OutT* __restrict__ out, int tokens, int inter) {
    const size_t total = static_cast<size_t>(tokens) * inter;
    pdl_trigger();
    pdl_wait();
    for (size_t idx = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; idx < total;
         idx += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t t = idx / inter;
        const size_t i = idx - t * inter;
        const float* base = partial + t * 2 * inter;
        float gate = 0.0f, up = 0.0f;
        for (int s = 0; s < splits; ++s) {
            gate += base[s * split_stride + i];
            up += base[s * split_stride + inter + i];
        }
        const float activated = gate / (1.0f + expf(-gate));
        out[idx] = from_float<OutT>(activated * up);
    }
}

ME_EXPORT int me_swiglu(const float* partial, int splits, long long split_stride, void* out, int out_type,
                        int tokens, int inter, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const size_t total = static_cast<size_t>(tokens) * inter;
    const int threads = 256;
    const int blocks = static_cast<int>(std::min<size_t>((total + threads - 1) / threads, 148 * 16));
    if (out_type == ME_BF16)
        return launch_kernel(swiglu_kernel<__nv_bfloat16>, blocks, threads, 0, stream, partial, splits,
                             (size_t)split_stride, static_cast<__nv_bfloat16*>(out), tokens, inter);
    return launch_kernel(swiglu_kernel<float>, blocks, threads, 0, stream, partial, splits, (size_t)split_stride,
                         static_cast<float*>(out), tokens, inter);
}

// ------------------------------------------------- per-head norm + rotary + cache write

// One warp per (token, head) over the columns of qkv = [q heads | k heads | v heads].
//   q heads: optional RMSNorm over head_dim, optional rotation, written to q_out[t][h][:].
//   k heads: the same, written to the token's slot of k_pages (or to k_dense[t][h][:]).
//   v heads: copied to the slot of v_pages (or v_dense).
// Pages are [page][kv_head][slot in page][head_dim]; slot_mapping[t] = page * page_size + slot,
// negative for a token whose keys are not to be stored.
struct QkvArgs {
    const float* qkv;     // [splits][tokens][(heads + 2 kv_heads) * head_dim]
    int splits;
    size_t split_stride;
    const float* q_weight;  // [head_dim] or null: no norm
    const float* k_weight;
    float eps;
    const float2* cos_sin;  // [tokens][rotary_dim / 2] (cos, sin) of each token's angles, or null: no rotation
    const int* positions;
    const int* slot_mapping;  // null: dense outputs
    void* q_out;
    void* k_pages;
    void* v_pages;
    void* k_dense;
    void* v_dense;
    int tokens, heads, kv_heads, head_dim, page_size;
    int rotary_dim;  // the first rotary_dim elements of a head are rotated (in halves of rotary_dim / 2), the rest pass through
    const float* bias;  // [(heads + 2 kv_heads) * head_dim] added to the projections' sums, or null
};

constexpr int QKV_WARPS = 4;
constexpr int MAX_HEAD_DIM = 512;

template <typename OutT>
__global__ void __launch_bounds__(QKV_WARPS * 32) qk_norm_rope_store_kernel(QkvArgs a) {
    extern __shared__ float staged[];  // [QKV_WARPS][head_dim]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = a.heads + 2 * a.kv_heads;
    const long long item = static_cast<long long>(blockIdx.x) * QKV_WARPS + warp;
    if (item >= static_cast<long long>(a.tokens) * heads_total) return;
    const int token = static_cast<int>(item / heads_total);
    const int column_head = static_cast<int>(item % heads_total);
    const int d = a.head_dim, half = a.rotary_dim / 2;
    float* vec = staged + warp * d;
    pdl_trigger();
    pdl_wait();

    const size_t row_width = static_cast<size_t>(heads_total) * d;
    const float* src = a.qkv + static_cast<size_t>(token) * row_width + static_cast<size_t>(column_head) * d;
    float sum_sq = 0.0f;
    for (int i = lane; i < d; i += 32) {
        float v = 0.0f;
        for (int s = 0; s < a.splits; ++s) v += src[s * a.split_stride + i];
        if (a.bias) v += a.bias[static_cast<size_t>(column_head) * d + i];
        vec[i] = v;
        sum_sq = fmaf(v, v, sum_sq);
    }
    const bool is_q = column_head < a.heads;
    const bool is_k = !is_q && column_head < a.heads + a.kv_heads;
    const float* weight = is_q ? a.q_weight : (is_k ? a.k_weight : nullptr);
    float inv = 1.0f;
    if (weight) {
        sum_sq = warp_sum(sum_sq);
        inv = rsqrtf(sum_sq / static_cast<float>(d) + a.eps);
    }
    __syncwarp();

    OutT* dst;
    if (is_q) {
        dst = static_cast<OutT*>(a.q_out) + (static_cast<size_t>(token) * a.heads + column_head) * d;
    } else {
        const int kv_head = is_k ? column_head - a.heads : column_head - a.heads - a.kv_heads;
        if (a.slot_mapping) {
            const int slot = a.slot_mapping[token];
            if (slot < 0) return;
            const size_t page = slot / a.page_size, offset = slot % a.page_size;
            OutT* pages = static_cast<OutT*>(is_k ? a.k_pages : a.v_pages);
            dst = pages + ((page * a.kv_heads + kv_head) * a.page_size + offset) * d;
        } else {
            OutT* dense = static_cast<OutT*>(is_k ? a.k_dense : a.v_dense);
            dst = dense + (static_cast<size_t>(token) * a.kv_heads + kv_head) * d;
        }
    }
    const bool rotate = (is_q || is_k) && a.cos_sin != nullptr;
    const float2* angles = a.cos_sin + static_cast<size_t>(token) * half;
    for (int i = lane; i < d; i += 32) {
        float value = weight ? weight[i] * (vec[i] * inv) : vec[i];
        if (rotate && i < a.rotary_dim) {
            // rotate-half: out[i] = x[i] cos - x[i + half] sin (i < half); x[i] cos + x[i - half] sin.
            const int j = i < half ? i + half : i - half;
            const float other = weight ? weight[j] * (vec[j] * inv) : vec[j];
            const float2 angle = angles[i < half ? i : i - half];
            const float cosine = angle.x, sine = angle.y;
            value = i < half ? value * cosine - other * sine : value * cosine + other * sine;
        }
        dst[i] = from_float<OutT>(value);
    }
}

// The same for head_dim == 128: each lane owns four consecutive elements, all partial sums are
// loaded before they are added, and the rotation partner (64 elements away) is 16 lanes away.
// A warp takes HEADS consecutive heads of one token and requests all of them before it uses any:
// with one partial sum (prompts) four heads per warp keep enough loads in flight to fill HBM.
template <typename OutT, int HEADS, int MAX_SPLITS>
__global__ void __launch_bounds__(QKV_WARPS * 32) qk_norm_rope_store_128_kernel(QkvArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads_total = a.heads + 2 * a.kv_heads;
    const int groups = heads_total / HEADS;  // the launcher makes sure this divides
    const long long item = static_cast<long long>(blockIdx.x) * QKV_WARPS + warp;
    if (item >= static_cast<long long>(a.tokens) * groups) return;
    const int token = static_cast<int>(item / groups);
    const int first_head = static_cast<int>(item % groups) * HEADS;
    constexpr int D = 128;
    pdl_trigger();
    // Weights and the step's slot list do not come from the previous kernel: fetch them ahead of the wait.
    const float4 one = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
    const float4 q_w = a.q_weight ? *reinterpret_cast<const float4*>(a.q_weight + lane * 4) : one;
    const float4 k_w = a.k_weight ? *reinterpret_cast<const float4*>(a.k_weight + lane * 4) : one;
    const int slot = a.slot_mapping ? a.slot_mapping[token] : 0;
    pdl_wait();
    const float* src = a.qkv + static_cast<size_t>(token) * heads_total * D + static_cast<size_t>(first_head) * D + lane * 4;
    float4 part[HEADS][MAX_SPLITS];
#pragma unroll
    for (int u = 0; u < HEADS; ++u)
#pragma unroll
        for (int s = 0; s < MAX_SPLITS; ++s)
            if (s < a.splits) part[u][s] = *reinterpret_cast<const float4*>(src + u * D + s * a.split_stride);
    float4 first = make_float4(1.0f, 0.0f, 1.0f, 0.0f), second = first;
    if (a.cos_sin != nullptr) {
        const float4* angles = reinterpret_cast<const float4*>(a.cos_sin + static_cast<size_t>(token) * (D / 2) + (lane & 15) * 4);
        first = angles[0];   // (cos, sin) of four consecutive frequencies
        second = angles[1];
    }
#pragma unroll
    for (int u = 0; u < HEADS; ++u) {
        const int column_head = first_head + u;
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
        for (int s = 0; s < MAX_SPLITS; ++s)
            if (s < a.splits) { v.x += part[u][s].x; v.y += part[u][s].y; v.z += part[u][s].z; v.w += part[u][s].w; }
        if (a.bias) {
            const float4 b = *reinterpret_cast<const float4*>(a.bias + static_cast<size_t>(column_head) * D + lane * 4);
            v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
        }
        const bool is_q = column_head < a.heads;
        const bool is_k = !is_q && column_head < a.heads + a.kv_heads;
        const float* weight = is_q ? a.q_weight : (is_k ? a.k_weight : nullptr);
        if (weight) {
            float sum_sq = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
            sum_sq = warp_sum(sum_sq);
            const float inv = rsqrtf(sum_sq / static_cast<float>(D) + a.eps);
            const float4 w = is_q ? q_w : k_w;
            v = make_float4(w.x * (v.x * inv), w.y * (v.y * inv), w.z * (v.z * inv), w.w * (v.w * inv));
        }
        if ((is_q || is_k) && a.cos_sin != nullptr) {
            const float4 other = make_float4(__shfl_xor_sync(0xffffffffu, v.x, 16), __shfl_xor_sync(0xffffffffu, v.y, 16),
                                             __shfl_xor_sync(0xffffffffu, v.z, 16), __shfl_xor_sync(0xffffffffu, v.w, 16));
            const float sign = lane < 16 ? -1.0f : 1.0f;  // first half: x cos - partner sin; second: x cos + partner sin
            v.x = v.x * first.x + sign * other.x * first.y;
            v.y = v.y * first.z + sign * other.y * first.w;
            v.z = v.z * second.x + sign * other.z * second.y;
            v.w = v.w * second.z + sign * other.w * second.w;
        }
        OutT* dst;
        if (is_q) {
            dst = static_cast<OutT*>(a.q_out) + (static_cast<size_t>(token) * a.heads + column_head) * D;
        } else {
            const int kv_head = is_k ? column_head - a.heads : column_head - a.heads - a.kv_heads;
            if (a.slot_mapping) {
                if (slot < 0) continue;
                const size_t page = slot / a.page_size, offset = slot % a.page_size;
                OutT* pages = static_cast<OutT*>(is_k ? a.k_pages : a.v_pages);
                dst = pages + ((page * a.kv_heads + kv_head) * a.page_size + offset) * D;
            } else {
                OutT* dense = static_cast<OutT*>(is_k ? a.k_dense : a.v_dense);
                dst = dense + (static_cast<size_t>(token) * a.kv_heads + kv_head) * D;
            }
        }
        store4(dst + lane * 4, v);
    }
}

// (cos, sin) of position * inv_freq for every token of the step, once per step for all layers
// (src/mini_engine/model.py:79-83,183 of YuvGev00/mini-engine builds its tables once per step too).
__global__ void rope_table_kernel(const float* __restrict__ inv_freq, const int* __restrict__ positions,
                                  float2* __restrict__ out, int tokens, int half) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * half) return;
    const int token = idx / half, i = idx % half;
    float sine, cosine;
    sincosf(static_cast<float>(positions[token]) * inv_freq[i], &sine, &cosine);
    out[idx] = make_float2(cosine, sine);
}

ME_EXPORT int me_rope_table(const float* inv_freq, const int* positions, float* out, int tokens, int half,
                            cudaStream_t stream) {
    if (tokens <= 0) return 0;
    const int total = tokens * half;
    return launch_kernel(rope_table_kernel, (total + 255) / 256, 256, 0, stream, inv_freq, positions,
                         reinterpret_cast<float2*>(out), tokens, half);
}

ME_EXPORT int me_qk_norm_rope_store(const float* qkv, int splits, long long split_stride, const float* q_weight,
                                    const float* k_weight, float eps, const float* cos_sin,
                                    const int* positions, const int* slot_mapping, void* q_out, void* k_pages,
                                    void* v_pages, void* k_dense, void* v_dense, int out_type, int tokens,
                                    int heads, int kv_heads, int head_dim, int page_size, int rotary_dim,
                                    const float* bias, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (head_dim > MAX_HEAD_DIM || head_dim % 2) return ME_ERR_UNSUPPORTED;
    if (rotary_dim < 0 || rotary_dim > head_dim || rotary_dim % 2) return ME_ERR_ARGUMENT;
    QkvArgs a{qkv, splits, (size_t)split_stride, q_weight, k_weight, eps, reinterpret_cast<const float2*>(cos_sin), positions, slot_mapping,
              q_out, k_pages, v_pages, k_dense, v_dense, tokens, heads, kv_heads, head_dim, page_size, rotary_dim, bias};
    const long long items = static_cast<long long>(tokens) * (heads + 2 * kv_heads);
    const int blocks = static_cast<int>((items + QKV_WARPS - 1) / QKV_WARPS);
    const size_t smem = static_cast<size_t>(QKV_WARPS) * head_dim * sizeof(float);
    // The choice depends on the model's sizes and the engine's buffers only, never on the batch.
    const bool vec = head_dim == 128 && rotary_dim == head_dim && splits <= MAX_UNROLLED_SPLITS && split_stride % 4 == 0 && aligned16(qkv) &&
                     aligned16(q_out) && aligned16(k_pages) && aligned16(v_pages) && aligned16(k_dense) &&
                     aligned16(v_dense) && aligned16(q_weight) && aligned16(k_weight) && aligned16(cos_sin) && aligned16(bias);
    if (vec) {
        // The number of heads per warp depends on the number of partial sums and on the model's
        // head counts only, never on the batch.
        const bool four = splits == 1 && (heads + 2 * kv_heads) % 4 == 0;
        const long long warps = static_cast<long long>(tokens) * ((heads + 2 * kv_heads) / (four ? 4 : 1));
        const int vec_blocks = static_cast<int>((warps + QKV_WARPS - 1) / QKV_WARPS);
        if (out_type == ME_BF16)
            return four ? launch_kernel(qk_norm_rope_store_128_kernel<__nv_bfloat16, 4, 1>, vec_blocks, QKV_WARPS * 32, 0, stream, a)
                        : launch_kernel(qk_norm_rope_store_128_kernel<__nv_bfloat16, 1, MAX_UNROLLED_SPLITS>, vec_blocks, QKV_WARPS * 32, 0, stream, a);
        return four ? launch_kernel(qk_norm_rope_store_128_kernel<float, 4, 1>, vec_blocks, QKV_WARPS * 32, 0, stream, a)
                    : launch_kernel(qk_norm_rope_store_128_kernel<float, 1, MAX_UNROLLED_SPLITS>, vec_blocks, QKV_WARPS * 32, 0, stream, a);
    }
    if (out_type == ME_BF16)
        return launch_kernel(qk_norm_rope_store_kernel<__nv_bfloat16>, blocks, QKV_WARPS * 32, smem, stream, a);
    return launch_kernel(qk_norm_rope_store_kernel<float>, blocks, QKV_WARPS * 32, smem, stream, a);
}

// Dense [tokens][kv_heads][head_dim] keys and values into their slots of the pages.
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ k_dense, const T* __restrict__ v_dense,
                                const int* __restrict__ slot_mapping, T* __restrict__ k_pages,
                                T* __restrict__ v_pages, int kv_heads, int head_dim, int page_size) {
    const int token = blockIdx.x;
    pdl_trigger();
    pdl_wait();
    const int slot = slot_mapping[token];
    if (slot < 0) return;
    const size_t page = slot / page_size, offset = slot % page_size;
    const int width = kv_heads * head_dim;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const int head = i / head_dim, e = i % head_dim;
        const size_t dst = ((page * kv_heads + head) * page_size + offset) * head_dim + e;
        k_pages[dst] = k_dense[static_cast<size_t>(token) * width + i];
        v_pages[dst] = v_dense[static_cast<size_t>(token) * width + i];
    }
}

ME_EXPORT int me_kv_store(const void* k_dense, const void* v_dense, const int* slot_mapping, void* k_pages,
                          void* v_pages, int type, int tokens, int kv_heads, int head_dim, int page_size,
                          cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (type == ME_BF16)
        return launch_kernel(kv_store_kernel<__nv_bfloat16>, tokens, 128, 0, stream,
                             static_cast<const __nv_bfloat16*>(k_dense), static_cast<const __nv_bfloat16*>(v_dense),
                             slot_mapping, static_cast<__nv_bfloat16*>(k_pages), static_cast<__nv_bfloat16*>(v_pages),
                             kv_heads, head_dim, page_size);
    return launch_kernel(kv_store_kernel<float>, tokens, 128, 0, stream, static_cast<const float*>(k_dense),
                         static_cast<const float*>(v_dense), slot_mapping, static_cast<float*>(k_pages),
                         static_cast<float*>(v_pages), kv_heads, head_dim, page_size);
}
