// Choosing the next token from float32 logits [rows][vocab]: argmax, or a draw from
// softmax(logits / temperature).
//
// YuvGev00/mini-engine, src/mini_engine/engine.py:282-291: temperature 0 is argmax; otherwise
// probabilities are softmax(logits / max(T, 1e-5)) in 32-bit and one token is drawn.  The
// reference draws with a single engine-wide generator, so its streams depend on the batch;
// here the caller passes one uniform number per row (derived from the seed, the request and
// the index of the token), and the draw is the inverse of the cumulative distribution at that
// number, so a request's tokens do not depend on what else is in the batch.
#include "common.cuh"

constexpr int SAMPLE_THREADS = 1024;

// One block per row.  Each thread owns one contiguous chunk of the vocabulary, so the
// cumulative sums run in index order and ties resolve to the lowest index.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperatures,
              const float* __restrict__ uniforms, int* __restrict__ out, int vocab) {
    __shared__ float red_value[SAMPLE_THREADS / 32];
    __shared__ int red_index[SAMPLE_THREADS / 32];
    __shared__ float chunk_sums[SAMPLE_THREADS];
    __shared__ float row_max_shared;
    __shared__ int best_shared;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    pdl_wait();
    const float* x = logits + static_cast<size_t>(row) * vocab;
    const int chunk = (vocab + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(tid * chunk, vocab), end = min(begin + chunk, vocab);

    // 1. maximum and its lowest index.  Threads stride through the row together (coalesced
    //    loads); a thread meets its indices in ascending order, so "greater than" keeps the lowest.
    float best = -INFINITY;
    int best_index = vocab;
    for (int i = tid; i < vocab; i += SAMPLE_THREADS) {
        const float v = x[i];
        if (v > best || (best_index == vocab && !(v < best))) { best = v; best_index = i; }
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, best, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, best_index, offset);
        if (other > best || (other == best && other_index < best_index)) { best = other; best_index = other_index; }
    }
    if (lane == 0) { red_value[warp] = best; red_index[warp] = best_index; }
    __syncthreads();
    if (tid == 0) {
        float b = red_value[0];
        int bi = red_index[0];
        for (int w = 1; w < SAMPLE_THREADS / 32; ++w)
            if (red_value[w] > b || (red_value[w] == b && red_index[w] < bi)) { b = red_value[w]; bi = red_index[w]; }
        row_max_shared = b;
        best_shared = bi < vocab ? bi : 0;
    }
    __syncthreads();
    const float temperature = temperatures ? temperatures[row] : 0.0f;
    if (temperature == 0.0f) {
        if (tid == 0) out[row] = best_shared;
        return;
    }

    // 2. unnormalised probabilities, chunk by chunk
    const float inv_t = 1.0f / fmaxf(temperature, 1e-5f);
    const float row_max = row_max_shared;
    float local = 0.0f;
    for (int i = begin; i < end; ++i) local += expf((x[i] - row_max) * inv_t);
    chunk_sums[tid] = local;
    __syncthreads();

    // 3. the chunk in which the cumulative sum passes uniform * total, then the token in it
    if (tid == 0) {
        float total = 0.0f;
        for (int t = 0; t < SAMPLE_THREADS; ++t) total += chunk_sums[t];
        const float target = uniforms[row] * total;
        float before = 0.0f;
        int owner = 0;
        for (int t = 0; t < SAMPLE_THREADS; ++t) {
            if (chunk_sums[t] > 0.0f) owner = t;  // last non-empty chunk so far: fallback for rounding
            if (before + chunk_sums[t] > target) { owner = t; break; }
            before += chunk_sums[t];
        }
        const int b = min(owner * chunk, vocab), e = min(b + chunk, vocab);
        int chosen = e - 1;
        float cumulative = before;
        for (int i = b; i < e; ++i) {
            cumulative += expf((x[i] - row_max) * inv_t);
            if (cumulative > target) { chosen = i; break; }
        }
        out[row] = chosen;
    }
}

ME_EXPORT int me_sample(const float* logits, const float* temperatures, const float* uniforms, int* out,
                        int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return 0;
    return launch_kernel(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, temperatures, uniforms, out, vocab);
}
