// Attention whose softmax weights are mixed across heads ("talking heads"), over a paged cache with a
// sliding window that also keeps the first positions of a sequence, with key and value heads of
// different sizes and an optional per-head output gate.  Float or bfloat16 storage; scores, weights,
// the mixing and the sums over keys are float in both.
//
//   s_g(i, j) = scale * q_g(i) . k_c(j)                 c = g / (heads / kv_heads)
//   visible(i, j): j <= i and (i - j < window or j < keep_first)        (window 0: every j <= i)
//   w_g(i, .) = softmax over the visible j of s_g(i, .)
//   w'_h(i, j) = sum_g talk[h, g] w_g(i, j)             (talk absent: w' = w)
//   out_h(i) = out_scale * gate_h(i) * sum_j w'_h(i, j) v_c(j)          c = h / (heads / kv_heads)
//   gate_h(i) = 1 / (1 + exp(-gate_in[i, h]))           (gate_in absent: 1)
//
// Mixing needs every head's NORMALISED weight of a key at once, so a block owns one query token with all
// its heads and walks the visible keys twice: the first walk finds each head's maximum and sum, the
// second recomputes the scores, normalises them, mixes them across heads in shared memory and applies
// them to the values.  Keys are walked in chunks of 32 positions (a chunk lies within one cache page).
//
// Cache layout of one layer: k_pool[page][kv_head][page_size][head_dim],
// v_pool[page][kv_head][page_size][value_dim]; block_table[seq][i] is the page that holds positions
// [i*page_size, (i+1)*page_size) of that sequence.  Pages that hold only invisible positions are never read.
#include "common.cuh"

#include <math_constants.h>

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int kChunk = 32;
constexpr int kMaxAcc = 16;  // outputs per thread: heads * value_dim <= kMaxAcc * threads
constexpr int kMaxThreads = 512;

// Two neighbouring elements (the address is a multiple of two elements).
__device__ __forceinline__ void load_pair(const float* p, float& a, float& b) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    a = v.x, b = v.y;
}
__device__ __forceinline__ void load_pair(const __nv_bfloat16* p, float& a, float& b) {
    const uint32_t raw = *reinterpret_cast<const uint32_t*>(p);
    a = __uint_as_float(raw << 16), b = __uint_as_float(raw & 0xffff0000u);
}

template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q_shared, const T* __restrict__ k_row, int head_dim,
                                         bool vector_ok) {
    float sum = 0.0f;
    if (vector_ok) {
#pragma unroll 4
        for (int d = 0; d < head_dim; d += 8) {
            float kv[8];
            load8(k_row + d, kv);
            const float4 qa = *reinterpret_cast<const float4*>(q_shared + d), qb = *reinterpret_cast<const float4*>(q_shared + d + 4);
            sum = fmaf(qa.x, kv[0], sum), sum = fmaf(qa.y, kv[1], sum), sum = fmaf(qa.z, kv[2], sum), sum = fmaf(qa.w, kv[3], sum);
            sum = fmaf(qb.x, kv[4], sum), sum = fmaf(qb.y, kv[5], sum), sum = fmaf(qb.z, kv[6], sum), sum = fmaf(qb.w, kv[7], sum);
        }
    } else {
        for (int d = 0; d < head_dim; ++d) sum = fmaf(q_shared[d], Num<T>::load(k_row + d), sum);
    }
    return sum;
}

// Rotation of query and key heads (split-half pairs over the first rotary_dim coordinates, angles from
// the tables) and the cache write: keys rotated, values as they are.  q is rotated in place.
// grid (tokens); any block size.
template <typename T>
__global__ void rotate_store_kernel(T* __restrict__ q, int q_stride, const T* __restrict__ k, int k_stride,
                                    const T* __restrict__ v, int v_stride, const int* __restrict__ positions,
                                    const float* __restrict__ cos_table, const float* __restrict__ sin_table,
                                    T* __restrict__ k_pool, T* __restrict__ v_pool, const int* __restrict__ slot_mapping,
                                    int heads, int kv_heads, int head_dim, int value_dim, int rotary_dim, int page_size) {
    grid_launch_dependents();  // what follows may start its own preparations; it waits for this grid before it reads
    grid_dependency_wait();
    const int token = blockIdx.x;
    const int half = rotary_dim / 2;
    const int pos = positions[token];
    const float* cos_row = cos_table + (size_t)pos * half;
    const float* sin_row = sin_table + (size_t)pos * half;
    T* q_row = q + (size_t)token * q_stride;
    for (int item = threadIdx.x; item < heads * half; item += blockDim.x) {
        const int head = item / half, i = item % half;
        T* p = q_row + (size_t)head * head_dim;
        const float a = Num<T>::load(p + i), b = Num<T>::load(p + i + half);
        const float c = cos_row[i], s = sin_row[i];
        Num<T>::store(p + i, a * c - b * s);
        Num<T>::store(p + i + half, b * c + a * s);
    }
    const int slot = slot_mapping[token];
    if (slot < 0) return;  // a padding row stores nothing
    const size_t page = slot / page_size, offset = slot % page_size;
    const T* k_row = k + (size_t)token * k_stride;
    for (int item = threadIdx.x; item < kv_heads * head_dim; item += blockDim.x) {
        const int head = item / head_dim, d = item % head_dim;
        const T* p = k_row + (size_t)head * head_dim;
        float value;
        if (d < half) {
            value = Num<T>::load(p + d) * cos_row[d] - Num<T>::load(p + d + half) * sin_row[d];
        } else if (d < rotary_dim) {
            const int i = d - half;
            value = Num<T>::load(p + d) * cos_row[i] + Num<T>::load(p + i) * sin_row[i];
        } else {
            value = Num<T>::load(p + d);
        }
        Num<T>::store(k_pool + ((page * kv_heads + head) * page_size + offset) * head_dim + d, value);
    }
    const T* v_row = v + (size_t)token * v_stride;
    for (int item = threadIdx.x; item < kv_heads * value_dim; item += blockDim.x) {
        const int head = item / value_dim, d = item % value_dim;
        v_pool[((page * kv_heads + head) * page_size + offset) * value_dim + d] = v_row[(size_t)head * value_dim + d];
    }
}

// grid (max_q_len, sequences); block: a multiple of 32 threads with heads * value_dim <= kMaxAcc * threads.
// shared: q [heads * head_dim], weights [heads][32], mixed [heads][32], maxima [heads], sums [heads], talk [heads^2].
template <typename T>
__global__ void __launch_bounds__(kMaxThreads) talking_attention_rows_kernel(
    const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride, const T* __restrict__ k_pool,
    const T* __restrict__ v_pool, const int* __restrict__ block_table, int max_blocks, const int* __restrict__ cu_q,
    const int* __restrict__ kv_lens, const float* __restrict__ talk, const T* __restrict__ gate_in, int gate_stride,
    int heads, int kv_heads, int head_dim, int value_dim, int page_size, int window, int keep_first, float scale,
    float out_scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) float shared[];
    const int seq = blockIdx.y;
    const int q_begin = cu_q[seq];
    const int q_len = cu_q[seq + 1] - q_begin;
    const int j = blockIdx.x;
    if (j >= q_len) return;  // the whole block leaves
    const int row = q_begin + j;
    const int pos = kv_lens[seq] - q_len + j;
    const int window_first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kept_end = keep_first < window_first ? keep_first : window_first;  // [0, kept_end): kept first positions
    const int group = heads / kv_heads;
    const bool vector_ok = (head_dim % 8) == 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;

    float* q_shared = shared;
    float* weights = q_shared + heads * head_dim;
    float* mixed = weights + heads * kChunk;
    float* maxima = mixed + heads * kChunk;
    float* sums = maxima + heads;
    float* talk_shared = sums + heads;

    const T* q_row = q + (size_t)row * q_stride;
    for (int i = threadIdx.x; i < heads * head_dim; i += blockDim.x) q_shared[i] = Num<T>::load(q_row + i);
    if (talk != nullptr)
        for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) talk_shared[i] = talk[i];
    __syncthreads();
    const int* table = block_table + (size_t)seq * max_blocks;

    // first walk: every head's maximum and sum of exponentials over the visible keys (a warp owns a head)
    for (int head = warp; head < heads; head += warps) {
        const int kv_head = head / group;
        float running_max = -CUDART_INF_F, running_sum = 0.0f;
        for (int range = 0; range < 2; ++range) {
            const int begin = range == 0 ? 0 : window_first, end = range == 0 ? kept_end : pos + 1;
            for (int chunk = begin - begin % kChunk; chunk < end; chunk += kChunk) {
                const size_t page = table[chunk / page_size];
                const size_t base = (page * kv_heads + kv_head) * page_size + (chunk % page_size);
                const int p = chunk + lane;
                float score = -CUDART_INF_F;
                if (p >= begin && p < end)
                    score = dot_row<T>(q_shared + head * head_dim, k_pool + (base + lane) * head_dim, head_dim, vector_ok) * scale;
                const float new_max = fmaxf(running_max, warp_max(score));  // finite: the chunk holds a visible key
                const float e = expf(score - new_max);                      // exp(-inf) = 0 for an invisible key
                running_sum = running_sum * expf(running_max - new_max) + warp_sum(e);
                running_max = new_max;
            }
        }
        if (lane == 0) {
            maxima[head] = running_max;
            sums[head] = running_sum;
        }
    }
    __syncthreads();

    float acc[kMaxAcc];
#pragma unroll
    for (int i = 0; i < kMaxAcc; ++i) acc[i] = 0.0f;
    const int outputs = heads * value_dim;

    // second walk: normalised weights of a chunk for all heads, mixed across heads, applied to the values
    for (int range = 0; range < 2; ++range) {
        const int begin = range == 0 ? 0 : window_first, end = range == 0 ? kept_end : pos + 1;
        for (int chunk = begin - begin % kChunk; chunk < end; chunk += kChunk) {
            const size_t page = table[chunk / page_size];
            const size_t page_base = page * kv_heads * page_size + (chunk % page_size);
            for (int head = warp; head < heads; head += warps) {
                const size_t base = page_base + (size_t)(head / group) * page_size;
                const int p = chunk + lane;
                float weight = 0.0f;
                if (p >= begin && p < end) {
                    const float score =
                        dot_row<T>(q_shared + head * head_dim, k_pool + (base + lane) * head_dim, head_dim, vector_ok) * scale;
                    weight = expf(score - maxima[head]) / sums[head];
                }
                weights[head * kChunk + lane] = weight;
            }
            __syncthreads();
            const float* applied = weights;
            if (talk != nullptr) {
                for (int item = threadIdx.x; item < heads * kChunk; item += blockDim.x) {
                    const int head = item / kChunk, key = item % kChunk;
                    float sum = 0.0f;
                    for (int g = 0; g < heads; ++g) sum = fmaf(talk_shared[head * heads + g], weights[g * kChunk + key], sum);
                    mixed[item] = sum;
                }
                __syncthreads();
                applied = mixed;
            }
            const int first_key = begin > chunk ? begin - chunk : 0;
            const int last_key = end - chunk < kChunk ? end - chunk : kChunk;
#pragma unroll
            for (int i = 0; i < kMaxAcc; ++i) {
                const int o = threadIdx.x + i * blockDim.x;
                if (o < outputs) {
                    const int head = o / value_dim, d = o % value_dim;
                    const T* v_col = v_pool + (page_base + (size_t)(head / group) * page_size) * value_dim + d;
                    const float* w = applied + head * kChunk;
                    float sum = acc[i];
                    for (int key = first_key; key < last_key; ++key)
                        sum = fmaf(w[key], Num<T>::load(v_col + (size_t)key * value_dim), sum);
                    acc[i] = sum;
                }
            }
            __syncthreads();  // the next chunk overwrites the weights
        }
    }

    T* out_row = out + (size_t)row * out_stride;
#pragma unroll
    for (int i = 0; i < kMaxAcc; ++i) {
        const int o = threadIdx.x + i * blockDim.x;
        if (o < outputs) {
            float value = acc[i] * out_scale;
            if (gate_in != nullptr) {
                const float z = Num<T>::load(gate_in + (size_t)row * gate_stride + o / value_dim);
                value *= 1.0f / (1.0f + expf(-z));
            }
            Num<T>::store(out_row + o, value);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Decoding: one query token per sequence.  A block per token cannot keep a GPU busy with a handful of
// sequences, so the visible keys are cut into their chunks of 32 and every chunk gets a block, in two kernels:
//   scores: a block computes every head's scaled scores of its chunk (scratch [sequence][head][chunk][32]) and
//           the chunk's maximum and sum of exponentials per head (scratch [sequence][head][chunk][2]);
//   values: a block first folds all chunks' maxima and sums into every head's maximum and sum (in chunk order),
//           then normalises its own chunk's scores, mixes them across heads, applies them to its chunk of the
//           values, and writes its partial result (scratch [sequence][chunk][heads * value_dim]); the block
//           that finishes last (a ticket per sequence) adds the partial results in chunk order, applies gate
//           and scale and stores the token's result, and puts the ticket back to zero.
// The chunks of a sequence: those of the kept first positions [0, kept_end), then those of the window.

struct DecodeChunks {
    int pos, window_first, kept_end, kept_chunks, total;
    __device__ __forceinline__ DecodeChunks(int kv_len, int window, int keep_first) {
        pos = kv_len - 1;
        window_first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
        kept_end = keep_first < window_first ? keep_first : window_first;
        kept_chunks = (kept_end + kChunk - 1) / kChunk;
        total = kept_chunks + pos / kChunk - window_first / kChunk + 1;
    }
    // first position of chunk `index`, and the range of visible positions it is walked for
    __device__ __forceinline__ void chunk(int index, int& first, int& begin, int& end) const {
        if (index < kept_chunks) {
            first = index * kChunk;
            begin = 0;
            end = kept_end;
        } else {
            first = (window_first / kChunk + index - kept_chunks) * kChunk;
            begin = window_first;
            end = pos + 1;
        }
    }
};

// grid (most chunks of any sequence, sequences); block: a warp per head, at most 16.
template <typename T>
__global__ void __launch_bounds__(kMaxThreads) talking_decode_scores_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ cu_q, const int* __restrict__ kv_lens, float* __restrict__ scores, float* __restrict__ stats,
    int max_chunks, int heads, int kv_heads, int head_dim, int page_size, int window, int keep_first, float scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) float q_shared[];  // heads * head_dim
    const int seq = blockIdx.y, index = blockIdx.x;
    const DecodeChunks chunks(kv_lens[seq], window, keep_first);
    if (index >= chunks.total) return;
    int first, begin, end;
    chunks.chunk(index, first, begin, end);
    const T* q_row = q + (size_t)cu_q[seq] * q_stride;
    for (int i = threadIdx.x; i < heads * head_dim; i += blockDim.x) q_shared[i] = Num<T>::load(q_row + i);
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    const int group = heads / kv_heads;
    const bool vector_ok = (head_dim % 8) == 0;
    const size_t page = block_table[(size_t)seq * max_blocks + first / page_size];
    const int p = first + lane;
    const bool seen = p >= begin && p < end;
    for (int head = warp; head < heads; head += warps) {
        const size_t row = (page * kv_heads + head / group) * page_size + (first % page_size) + lane;
        float score = -CUDART_INF_F;
        if (seen) score = dot_row<T>(q_shared + head * head_dim, k_pool + row * head_dim, head_dim, vector_ok) * scale;
        const float top = warp_max(score);  // finite: a chunk that is walked holds a visible key
        const float sum = warp_sum(expf(score - top));
        const size_t at = ((size_t)seq * heads + head) * max_chunks + index;
        scores[at * kChunk + lane] = score;
        if (lane == 0) {
            stats[at * 2] = top;
            stats[at * 2 + 1] = sum;
        }
    }
}

// grid (most chunks of any sequence, sequences); block: as for the kernel with a block per token.
// shared: weights [heads][32], mixed [heads][32], maxima [heads], sums [heads], talk [heads^2].
template <typename T>
__global__ void __launch_bounds__(kMaxThreads) talking_decode_values_kernel(
    T* __restrict__ out, int out_stride, const T* __restrict__ v_pool, const int* __restrict__ block_table, int max_blocks,
    const int* __restrict__ cu_q, const int* __restrict__ kv_lens, const float* __restrict__ scores, const float* __restrict__ stats,
    float* __restrict__ partial, int* __restrict__ tickets, int max_chunks, const float* __restrict__ talk,
    const T* __restrict__ gate_in, int gate_stride, int heads, int kv_heads, int value_dim, int page_size, int window,
    int keep_first, float out_scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) float shared[];
    __shared__ int last_block;
    const int seq = blockIdx.y, index = blockIdx.x;
    const DecodeChunks chunks(kv_lens[seq], window, keep_first);
    if (index >= chunks.total) return;
    int first, begin, end;
    chunks.chunk(index, first, begin, end);
    float* weights = shared;
    float* mixed = weights + heads * kChunk;
    float* maxima = mixed + heads * kChunk;
    float* sums = maxima + heads;
    float* talk_shared = sums + heads;
    const int group = heads / kv_heads;
    const int outputs = heads * value_dim;

    // every head's maximum and sum over all chunks: a warp per head, a lane per chunk (and every 32nd after it);
    // the order of the additions depends on the number of chunks only
    for (int head = threadIdx.x >> 5; head < heads; head += blockDim.x >> 5) {
        const float2* of_head = reinterpret_cast<const float2*>(stats) + ((size_t)seq * heads + head) * max_chunks;
        const int lane = threadIdx.x & 31;
        float top = -CUDART_INF_F;
        for (int c = lane; c < chunks.total; c += 32) top = fmaxf(top, of_head[c].x);
        top = warp_max(top);
        float sum = 0.0f;
        for (int c = lane; c < chunks.total; c += 32) {
            const float2 pair = of_head[c];
            sum += pair.y * expf(pair.x - top);
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            maxima[head] = top;
            sums[head] = sum;
        }
    }
    if (talk != nullptr)
        for (int i = threadIdx.x; i < heads * heads; i += blockDim.x) talk_shared[i] = talk[i];
    __syncthreads();
    for (int item = threadIdx.x; item < heads * kChunk; item += blockDim.x) {
        const int head = item / kChunk, key = item % kChunk;
        const float score = scores[(((size_t)seq * heads + head) * max_chunks + index) * kChunk + key];
        weights[item] = expf(score - maxima[head]) / sums[head];  // exp(-inf) = 0 for an invisible key
    }
    __syncthreads();
    const float* applied = weights;
    if (talk != nullptr) {
        for (int item = threadIdx.x; item < heads * kChunk; item += blockDim.x) {
            const int head = item / kChunk, key = item % kChunk;
            float sum = 0.0f;
            for (int g = 0; g < heads; ++g) sum = fmaf(talk_shared[head * heads + g], weights[g * kChunk + key], sum);
            mixed[item] = sum;
        }
        __syncthreads();
        applied = mixed;
    }
    const size_t page = block_table[(size_t)seq * max_blocks + first / page_size];
    const size_t page_base = page * kv_heads * page_size + (first % page_size);
    const int first_key = begin > first ? begin - first : 0;
    const int last_key = end - first < kChunk ? end - first : kChunk;
    float* mine = partial + ((size_t)seq * max_chunks + index) * outputs;
    if ((value_dim & 1) == 0) {
        // A thread owns two neighbouring coordinates of one key/value head: it asks for all 32 keys' values at once
        // (one round trip to memory), then serves every query head of the group from its registers.
        const int half = value_dim / 2;
        for (int item = threadIdx.x; item < kv_heads * half; item += blockDim.x) {
            const int kv_head = item / half, d = 2 * (item % half);
            const T* v_col = v_pool + (page_base + (size_t)kv_head * page_size) * value_dim + d;
            float lo[kChunk], hi[kChunk];
#pragma unroll
            for (int key = 0; key < kChunk; ++key) {
                lo[key] = hi[key] = 0.0f;
                if (key >= first_key && key < last_key) load_pair(v_col + (size_t)key * value_dim, lo[key], hi[key]);
            }
            for (int head = kv_head * group; head < (kv_head + 1) * group; ++head) {
                const float* w = applied + head * kChunk;
                float sum_lo = 0.0f, sum_hi = 0.0f;
#pragma unroll
                for (int key = 0; key < kChunk; ++key) {  // (the weight of a key outside the range is zero)
                    sum_lo = fmaf(w[key], lo[key], sum_lo);
                    sum_hi = fmaf(w[key], hi[key], sum_hi);
                }
                *reinterpret_cast<float2*>(mine + head * value_dim + d) = make_float2(sum_lo, sum_hi);
            }
        }
    } else {
        for (int o = threadIdx.x; o < outputs; o += blockDim.x) {
            const int head = o / value_dim, d = o % value_dim;
            const T* v_col = v_pool + (page_base + (size_t)(head / group) * page_size) * value_dim + d;
            const float* w = applied + head * kChunk;
            float sum = 0.0f;
#pragma unroll 8
            for (int key = first_key; key < last_key; ++key) sum = fmaf(w[key], Num<T>::load(v_col + (size_t)key * value_dim), sum);
            mine[o] = sum;
        }
    }
    // the last block of the sequence to get here adds the chunks' parts, in chunk order
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) last_block = atomicAdd(tickets + seq, 1) == chunks.total - 1;
    __syncthreads();
    if (!last_block) return;
    __threadfence();
    const int row = cu_q[seq];
    const float* parts = partial + (size_t)seq * max_chunks * outputs;
    if ((value_dim & 3) == 0) {
        for (int o = 4 * threadIdx.x; o < outputs; o += 4 * blockDim.x) {  // four neighbouring coordinates of one head
            float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll 8
            for (int c = 0; c < chunks.total; ++c) {
                const float4 part = __ldcg(reinterpret_cast<const float4*>(parts + (size_t)c * outputs + o));
                sum.x += part.x, sum.y += part.y, sum.z += part.z, sum.w += part.w;
            }
            float factor = out_scale;
            if (gate_in != nullptr) factor /= 1.0f + expf(-Num<T>::load(gate_in + (size_t)row * gate_stride + o / value_dim));
            T* dst = out + (size_t)row * out_stride + o;
            Num<T>::store(dst, sum.x * factor);
            Num<T>::store(dst + 1, sum.y * factor);
            Num<T>::store(dst + 2, sum.z * factor);
            Num<T>::store(dst + 3, sum.w * factor);
        }
    } else {
        for (int o = threadIdx.x; o < outputs; o += blockDim.x) {
            float sum = 0.0f;
#pragma unroll 8
            for (int c = 0; c < chunks.total; ++c) sum += __ldcg(parts + (size_t)c * outputs + o);
            float value = sum * out_scale;
            if (gate_in != nullptr) {
                const float z = Num<T>::load(gate_in + (size_t)row * gate_stride + o / value_dim);
                value *= 1.0f / (1.0f + expf(-z));
            }
            Num<T>::store(out + (size_t)row * out_stride + o, value);
        }
    }
    if (threadIdx.x == 0) tickets[seq] = 0;  // as the next call expects it
}

}  // namespace mb

using namespace mb;

// q (rotated in place), k, v: [tokens, ...] rows with unit column stride and the row strides given (in
// elements); they may be column slices of one wider tensor.  slot_mapping[token]: page * page_size +
// offset of the token's cache position, or -1 for a row that stores nothing.
MB_EXPORT int mb_rotate_store(void* q, int q_stride, const void* k, int k_stride, const void* v, int v_stride, int dtype,
                              const int* positions, const float* cos_table, const float* sin_table, void* k_pool,
                              void* v_pool, const int* slot_mapping, int tokens, int heads, int kv_heads, int head_dim,
                              int value_dim, int rotary_dim, int page_size, cudaStream_t stream) {
    if (tokens <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        return fail("rotate_store: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    if (rotary_dim > 0 && (!cos_table || !sin_table || !positions))
        return fail("rotate_store: a rotation needs positions and cos/sin tables");
    if (!k_pool || !v_pool || !slot_mapping || page_size <= 0)
        return fail("rotate_store: needs pools, a slot mapping and a page size");
    if (rotary_dim == 0) {  // the tables are not read; any valid address serves
        cos_table = sin_table = reinterpret_cast<const float*>(slot_mapping);
    }
    const int work = kv_heads * (head_dim > value_dim ? head_dim : value_dim);
    const int threads = work >= 256 ? 256 : (work >= 128 ? 128 : 64);
    if (dtype == MB_F32)
        MB_LAUNCH("talking_attention", rotate_store_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true,
                  (float*)q, q_stride, (const float*)k, k_stride, (const float*)v, v_stride, positions, cos_table,
                  sin_table, (float*)k_pool, (float*)v_pool, slot_mapping, heads, kv_heads, head_dim, value_dim,
                  rotary_dim, page_size);
    else if (dtype == MB_BF16)
        MB_LAUNCH("talking_attention", rotate_store_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream,
                  true, (__nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, k_stride, (const __nv_bfloat16*)v,
                  v_stride, positions, cos_table, sin_table, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                  slot_mapping, heads, kv_heads, head_dim, value_dim, rotary_dim, page_size);
    else
        return fail("rotate_store: unknown dtype code %d", dtype);
    return check_launch("rotate_store");
}

// One query token per sequence (row cu_q[s] of q), the visible keys of every sequence cut into chunks of 32 with a
// block each.  most_positions: an upper bound of every sequence's cache length (it sizes grid and scratch).
// scratch: at least mb_talking_decode_scratch_floats(...) floats; tickets: `sequences` ints that are zero (the
// call leaves them zero).
MB_EXPORT size_t mb_talking_decode_chunks(int most_positions, int window, int keep_first) {
    const int span = (window > 0 && window < most_positions) ? window : most_positions;
    const int kept = keep_first < most_positions ? keep_first : most_positions;
    return (size_t)((span + kChunk - 2) / kChunk + 1 + (kept + kChunk - 1) / kChunk);
}

MB_EXPORT size_t mb_talking_decode_scratch_floats(int sequences, int heads, int value_dim, int most_positions, int window,
                                                  int keep_first) {
    const size_t chunks = mb_talking_decode_chunks(most_positions, window, keep_first);
    return (size_t)sequences * chunks * ((size_t)heads * (kChunk + 2) + (size_t)heads * value_dim) + 4;
}

MB_EXPORT int mb_talking_attention_decode(const void* q, int q_stride, void* out, int out_stride, int dtype, const void* k_pool,
                                          const void* v_pool, const int* block_table, int max_blocks, const int* cu_q,
                                          const int* kv_lens, int sequences, int most_positions, const float* talk,
                                          const void* gate_in, int gate_stride, int heads, int kv_heads, int head_dim,
                                          int value_dim, int page_size, int window, int keep_first, float scale, float out_scale,
                                          float* scratch, int* tickets, cudaStream_t stream) {
    if (sequences <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads)
        return fail("talking_attention: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (head_dim <= 0 || value_dim <= 0) return fail("talking_attention: head sizes must be positive");
    if (page_size <= 0 || page_size % kChunk) return fail("talking_attention: page_size %d must be a multiple of %d", page_size, kChunk);
    if (window < 0 || keep_first < 0 || most_positions <= 0) return fail("talking_attention: window, keep_first or positions out of range");
    if (sequences > 65535) return fail("talking_attention: %d sequences exceed the grid limit 65535", sequences);
    if (!scratch || !tickets) return fail("talking_attention: the decode form needs scratch memory and tickets");
    const int max_chunks = (int)mb_talking_decode_chunks(most_positions, window, keep_first);
    float* scores = scratch;
    float* stats = scores + (size_t)sequences * heads * max_chunks * kChunk;
    float* partial = stats + ((size_t)sequences * heads * max_chunks * 2 + 3) / 4 * 4;  // read 16 bytes at a time
    const dim3 grid(max_chunks, sequences);
    const size_t q_bytes = sizeof(float) * (size_t)heads * head_dim;
    const size_t smem = sizeof(float) * (2 * (size_t)heads * kChunk + 2 * heads + (size_t)heads * heads);
    if (q_bytes > 200 * 1024 || smem > 200 * 1024) return fail("talking_attention: %d heads of %d do not fit a block's shared memory", heads, head_dim);
    const int outputs = heads * value_dim;
    int threads = 128;
    while (threads < kMaxThreads && threads * 4 < outputs) threads *= 2;
    int score_threads = 32;
    while (score_threads < kMaxThreads && score_threads < 32 * heads) score_threads *= 2;
    cudaError_t status = cudaSuccess;
    if (dtype == MB_F32) {
        auto first = talking_decode_scores_kernel<float>;
        auto second = talking_decode_values_kernel<float>;
        if (q_bytes > 48 * 1024) status = cudaFuncSetAttribute(first, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)q_bytes);
        if (status == cudaSuccess && smem > 48 * 1024) status = cudaFuncSetAttribute(second, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("talking_attention: %s", cudaGetErrorString(status));
        MB_LAUNCH("talking_attention", first, dim3(grid), dim3(score_threads), q_bytes, stream, true, (const float*)q,
                  q_stride, (const float*)k_pool, block_table, max_blocks, cu_q, kv_lens, scores, stats, max_chunks,
                  heads, kv_heads, head_dim, page_size, window, keep_first, scale);
        MB_LAUNCH("talking_attention", second, dim3(grid), dim3(threads), smem, stream, true, (float*)out, out_stride,
                  (const float*)v_pool, block_table, max_blocks, cu_q, kv_lens, scores, stats, partial, tickets,
                  max_chunks, talk, (const float*)gate_in, gate_stride, heads, kv_heads, value_dim, page_size, window,
                  keep_first, out_scale);
    } else if (dtype == MB_BF16) {
        auto first = talking_decode_scores_kernel<__nv_bfloat16>;
        auto second = talking_decode_values_kernel<__nv_bfloat16>;
        if (q_bytes > 48 * 1024) status = cudaFuncSetAttribute(first, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)q_bytes);
        if (status == cudaSuccess && smem > 48 * 1024) status = cudaFuncSetAttribute(second, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (status != cudaSuccess) return fail("talking_attention: %s", cudaGetErrorString(status));
        MB_LAUNCH("talking_attention", first, dim3(grid), dim3(score_threads), q_bytes, stream, true,
                  (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k_pool, block_table, max_blocks, cu_q,
                  kv_lens, scores, stats, max_chunks, heads, kv_heads, head_dim, page_size, window, keep_first, scale);
        MB_LAUNCH("talking_attention", second, dim3(grid), dim3(threads), smem, stream, true, (__nv_bfloat16*)out,
                  out_stride, (const __nv_bfloat16*)v_pool, block_table, max_blocks, cu_q, kv_lens, scores, stats,
                  partial, tickets, max_chunks, talk, (const __nv_bfloat16*)gate_in, gate_stride, heads, kv_heads,
                  value_dim, page_size, window, keep_first, out_scale);
    } else {
        return fail("talking_attention: unknown dtype code %d", dtype);
    }
    return check_launch("talking_attention_decode");
}

// q: [tokens, >= heads*head_dim] rows (row stride in elements); out: [tokens, >= heads*value_dim] rows.
// talk: float [heads, heads] or null; gate_in: [tokens, >= heads] rows of the storage type, or null.
MB_EXPORT int mb_talking_attention_rows(const void* q, int q_stride, void* out, int out_stride, int dtype, const void* k_pool,
                                        const void* v_pool, const int* block_table, int max_blocks, const int* cu_q,
                                        const int* kv_lens, int sequences, int max_q_len, const float* talk,
                                        const void* gate_in, int gate_stride, int heads, int kv_heads, int head_dim,
                                        int value_dim, int page_size, int window, int keep_first, float scale,
                                        float out_scale, cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0) return 0;
    if (heads <= 0 || kv_heads <= 0 || heads % kv_heads)
        return fail("talking_attention: %d heads are no multiple of %d kv heads", heads, kv_heads);
    if (head_dim <= 0 || value_dim <= 0) return fail("talking_attention: head sizes must be positive");
    if (page_size <= 0 || page_size % kChunk) return fail("talking_attention: page_size %d must be a multiple of %d", page_size, kChunk);
    if (window < 0 || keep_first < 0) return fail("talking_attention: window and keep_first must not be negative");
    if (sequences > 65535) return fail("talking_attention: %d sequences exceed the grid limit 65535", sequences);
    const int outputs = heads * value_dim;
    int threads = 128;
    while (threads < kMaxThreads && (threads * kMaxAcc < outputs || (threads < 32 * heads && threads < 256))) threads *= 2;
    if (threads * kMaxAcc < outputs)
        return fail("talking_attention: heads * value_dim = %d exceeds %d", outputs, kMaxThreads * kMaxAcc);
    const size_t smem = sizeof(float) * ((size_t)heads * head_dim + 2 * (size_t)heads * kChunk + 2 * heads + (size_t)heads * heads);
    if (smem > 200 * 1024) return fail("talking_attention: %d heads of %d do not fit a block's shared memory", heads, head_dim);
    const dim3 grid(max_q_len, sequences);
    cudaError_t status;
    if (dtype == MB_F32) {
        auto kernel = talking_attention_rows_kernel<float>;
        if (smem > 48 * 1024) {
            status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (status != cudaSuccess) return fail("talking_attention: %s", cudaGetErrorString(status));
        }
        MB_LAUNCH("talking_attention", kernel, dim3(grid), dim3(threads), smem, stream, true, (const float*)q,
                  q_stride, (float*)out, out_stride, (const float*)k_pool, (const float*)v_pool, block_table,
                  max_blocks, cu_q, kv_lens, talk, (const float*)gate_in, gate_stride, heads, kv_heads, head_dim,
                  value_dim, page_size, window, keep_first, scale, out_scale);
    } else if (dtype == MB_BF16) {
        auto kernel = talking_attention_rows_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) {
            status = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (status != cudaSuccess) return fail("talking_attention: %s", cudaGetErrorString(status));
        }
        MB_LAUNCH("talking_attention", kernel, dim3(grid), dim3(threads), smem, stream, true, (const __nv_bfloat16*)q,
                  q_stride, (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)k_pool,
                  (const __nv_bfloat16*)v_pool, block_table, max_blocks, cu_q, kv_lens, talk,
                  (const __nv_bfloat16*)gate_in, gate_stride, heads, kv_heads, head_dim, value_dim, page_size, window,
                  keep_first, scale, out_scale);
    } else {
        return fail("talking_attention: unknown dtype code %d", dtype);
    }
    return check_launch("talking_attention");
}
