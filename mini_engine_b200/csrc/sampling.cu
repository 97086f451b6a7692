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

// One block per row.  Cumulative sums run in index order (a warp per contiguous segment of the
// vocabulary, then a thread per few consecutive tokens of one segment), and ties resolve to the
// lowest index.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, const float* __restrict__ temperatures,
              const float* __restrict__ uniforms, int* __restrict__ out, int vocab) {
    __shared__ float red_value[SAMPLE_THREADS / 32];
    __shared__ int red_index[SAMPLE_THREADS / 32];
    __shared__ float segment_sums[SAMPLE_THREADS / 32];
    __shared__ float warp_totals[SAMPLE_THREADS / 32];
    __shared__ int first_passing, last_positive;
    __shared__ float row_max_shared;
    __shared__ int best_shared;
    const int row = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    pdl_trigger();
    pdl_wait();
    const float* x = logits + static_cast<size_t>(row) * vocab;

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
        first_passing = SAMPLE_THREADS;
        last_positive = 0;
    }
    __syncthreads();
    const float temperature = temperatures ? temperatures[row] : 0.0f;
    if (temperature == 0.0f) {
        if (tid == 0) out[row] = best_shared;
        return;
    }

    // 2. unnormalised probabilities: warp w owns the contiguous segment [w * segment, +segment)
    //    of the vocabulary and adds it up with coalesced loads.
    const float factor = 1.4426950408889634f / fmaxf(temperature, 1e-5f);  // log2(e) / T
    const float row_max = row_max_shared;
    const int segment = (vocab + SAMPLE_THREADS / 32 - 1) / (SAMPLE_THREADS / 32);
    const int seg_begin = min(warp * segment, vocab), seg_end = min(seg_begin + segment, vocab);
    float local = 0.0f;
    for (int i = seg_begin + lane; i < seg_end; i += 32) local += exp2f((x[i] - row_max) * factor);
    local = warp_sum(local);
    if (lane == 0) segment_sums[warp] = local;
    __syncthreads();

    // 3. the segment in which the cumulative sum passes uniform * total (every thread finds it
    //    alike).  Then the whole block goes over that one segment, a few consecutive tokens per
    //    thread: a prefix sum over the threads names the first thread at which the cumulative
    //    sum exceeds the target, and that thread walks its own tokens.
    float total = 0.0f;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) total += segment_sums[w];
    const float target = uniforms[row] * total;
    int owner = -1, last_nonempty = 0;
    float before = 0.0f, before_last = 0.0f, running = 0.0f;
    for (int w = 0; w < SAMPLE_THREADS / 32; ++w) {
        const float s = segment_sums[w];
        if (s > 0.0f) { last_nonempty = w; before_last = running; }
        if (owner < 0 && running + s > target) { owner = w; before = running; }
        running += s;
    }
    if (owner < 0) { owner = last_nonempty; before = before_last; }  // rounding at a uniform number near 1
    const int owner_begin = min(owner * segment, vocab), owner_end = min(owner_begin + segment, vocab);
    const int per_thread = (segment + SAMPLE_THREADS - 1) / SAMPLE_THREADS;
    const int begin = min(owner_begin + tid * per_thread, owner_end), end = min(begin + per_thread, owner_end);
    float mine = 0.0f;
    for (int i = begin; i < end; ++i) mine += exp2f((x[i] - row_max) * factor);
    float scan = mine;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const float below = __shfl_up_sync(0xffffffffu, scan, offset);
        if (lane >= offset) scan += below;
    }
    if (lane == 31) warp_totals[warp] = scan;
    __syncthreads();
    float exclusive = before;
    for (int w = 0; w < warp; ++w) exclusive += warp_totals[w];
    exclusive += scan - mine;
    if (mine > 0.0f) {
        if (exclusive + mine > target) atomicMin(&first_passing, tid);
        atomicMax(&last_positive, tid);
    }
    __syncthreads();
    // No thread passes only when rounding left the target at or above the last cumulative sum:
    // then the last token of the segment that has any probability is the draw.
    const bool passing = first_passing < SAMPLE_THREADS;
    if (tid != (passing ? first_passing : last_positive)) return;
    int chosen = -1, fallback = begin;
    float cumulative = exclusive;
    for (int i = begin; i < end && chosen < 0; ++i) {
        const float p = exp2f((x[i] - row_max) * factor);
        cumulative += p;
        if (p > 0.0f) {
            fallback = i;
            if (passing && cumulative > target) chosen = i;
        }
    }
    out[row] = chosen >= 0 ? chosen : fallback;
}

ME_EXPORT int me_sample(const float* logits, const float* temperatures, const float* uniforms, int* out,
                        int rows, int vocab, cudaStream_t stream) {
    if (rows <= 0) return 0;
    return launch_kernel(sample_kernel, rows, SAMPLE_THREADS, 0, stream, logits, temperatures, uniforms, out, vocab);
}

// out[i] = tokens[rows[i]]: the drawn tokens of the requests that go on, in the order of the next
// step, without a round trip to the host.
__global__ void pick_tokens_kernel(const int* __restrict__ tokens, const int* __restrict__ rows, int* __restrict__ out, int count) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = tokens[rows[i]];
}

ME_EXPORT int me_pick_tokens(const int* tokens, const int* rows, int* out, int count, cudaStream_t stream) {
    if (count <= 0) return 0;
    return launch_kernel(pick_tokens_kernel, (count + 127) / 128, 128, 0, stream, tokens, rows, out, count);
}
