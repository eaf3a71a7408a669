// Tensor-core form of the attention of csrc/talking_attention.cu for steps that bring many tokens
// (prompts): bfloat16 storage, m16n8k16 products, compiled for one head count and one pair of key and
// value sizes: -DMB_HEADS=<1..16> -DMB_KEY_DIM=<multiple of 16> -DMB_VALUE_DIM=<multiple of 16>.
//
// A block owns 16 consecutive query tokens of one sequence with ALL their heads, one warp per head,
// because the weights of a key are mixed across heads after the softmax: w'_h(i, j) = sum_g talk[h, g]
// w_g(i, j) needs every head's normalised weight.  The visible keys are walked twice in chunks of 32:
//   walk 1: S_g = Q_g K_c^T per warp, running maximum and sum of every row;
//   walk 2: S_g again, w_g = exp(S_g - max_g) / sum_g in float, put side by side with the other heads' in shared
//           memory; the mixing is itself a product, talk [heads x heads] times weights [heads x 512 elements of the
//           chunk], shared out over the warps with both factors as two bfloat16 numbers each (hi + lo, about 16
//           bits of the float value; float accumulation); each warp then takes its own head's mixed weights back,
//           splits them the same way and adds hi . V_c + lo . V_c into its output accumulator.
// Keys and values of a chunk are copied to shared memory once per block for all key/value heads, the next
// chunk's (cp.async, two stages) while the current one is worked on.
// Scores, weights, the mixing and every sum are float; only the operands of the products are bfloat16.
#include "common.cuh"

#include <math_constants.h>

#if !defined(MB_HEADS) || !defined(MB_KEY_DIM) || !defined(MB_VALUE_DIM)
#error "compile with -DMB_HEADS, -DMB_KEY_DIM and -DMB_VALUE_DIM"
#endif

MB_DEFINE_LAST_ERROR()

namespace mb {

constexpr int H = MB_HEADS, D = MB_KEY_DIM, DV = MB_VALUE_DIM;
static_assert(H >= 1 && H <= 16, "one warp per head, at most 16");
static_assert(D % 16 == 0 && D >= 16 && D <= 256, "key size must be a multiple of 16 in 16..256");
static_assert(DV % 16 == 0 && DV >= 16 && DV <= 256, "value size must be a multiple of 16 in 16..256");
constexpr int kRows = 16;                // query tokens per block
constexpr int kKeys = 32;                // keys per chunk
constexpr int kKRow = D * 2 + 16;        // padded shared-memory rows: ldmatrix reads without bank conflicts
constexpr int kVRow = DV * 2 + 16;
constexpr int kThreads = 32 * H;
constexpr int kWeightFloats = 16 * 32;   // one head's weights of a chunk: [register][lane]
constexpr int kWeightRow = kWeightFloats + 4;  // padded: four heads' values of one element lie in four different banks

using bf16 = __nv_bfloat16;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, bool real) {
    const int bytes = real ? 16 : 0;  // 0: sixteen zero bytes are written and nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

// 32 positions of one page, every key/value head, asked for into padded rows [head][32][row bytes].  Rows of
// positions beyond `last_pos` become zeros when `zero_beyond` (values: a weight of zero must meet a finite number).
template <int kDim, int kRowBytes>
__device__ __forceinline__ void load_chunk(uint32_t dst, const bf16* __restrict__ pool, size_t page, int kv_heads,
                                           int page_size, int offset, int first_key, int last_pos, bool zero_beyond) {
    constexpr int kPieces = kDim / 8;
    for (int i = threadIdx.x; i < kv_heads * kKeys * kPieces; i += kThreads) {
        const int piece = i % kPieces, row = (i / kPieces) % kKeys, head = i / (kPieces * kKeys);
        cp_async16(dst + (head * kKeys + row) * kRowBytes + piece * 16,
                   pool + ((page * kv_heads + head) * page_size + offset + row) * (size_t)kDim + piece * 8,
                   !zero_beyond || first_key + row <= last_pos);
    }
}

// The chunks of 32 positions a tile of queries walks: those of the kept first positions [0, kept_end), then those
// from the first position the tile's first row sees in its window to the tile's last row.
struct TileChunks {
    int window_first, kept_end, last_pos, kept_chunks, total;
    __device__ __forceinline__ TileChunks(int pos0, int last, int window, int keep_first) {
        last_pos = last;
        window_first = (window > 0 && pos0 - window + 1 > 0) ? pos0 - window + 1 : 0;
        kept_end = keep_first < window_first ? keep_first : window_first;
        kept_chunks = (kept_end + kKeys - 1) / kKeys;
        total = kept_chunks + last_pos / kKeys - window_first / kKeys + 1;
    }
    __device__ __forceinline__ void chunk(int index, int& first, int& begin, int& end) const {
        if (index < kept_chunks) {
            first = index * kKeys, begin = 0, end = kept_end;
        } else {
            first = (window_first / kKeys + index - kept_chunks) * kKeys, begin = window_first, end = last_pos + 1;
        }
    }
};

// S[16 x 32 keys] of one warp's head: four accumulators of 8 keys.
__device__ __forceinline__ void chunk_scores(float (&s)[4][4], uint32_t q_rows, uint32_t k_rows) {
    const int lane = threadIdx.x & 31;
    const int q_row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int k_row = (lane & 7) + ((lane >> 4) & 1) * 8;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.0f;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t a[4], b[4];
        ldmatrix_x4(a, q_rows + q_row * kKRow + (ks * 2 + (lane >> 4)) * 16);
#pragma unroll
        for (int part = 0; part < 2; ++part) {
            ldmatrix_x4(b, k_rows + (part * 16 + k_row) * kKRow + (ks * 2 + ((lane >> 3) & 1)) * 16);
            mma_bf16(s[2 * part], a, b[0], b[1]);
            mma_bf16(s[2 * part + 1], a, b[2], b[3]);
        }
    }
}

// grid (tiles of 16 query tokens, sequences); block 32 * H.
__global__ void __launch_bounds__(kThreads)
talking_attention_tc_kernel(const bf16* __restrict__ q, int q_stride, bf16* __restrict__ out, int out_stride,
                            const bf16* __restrict__ k_pool, const bf16* __restrict__ v_pool, const int* __restrict__ block_table,
                            int max_blocks, const int* __restrict__ cu_q, const int* __restrict__ kv_lens,
                            const float* __restrict__ talk, const bf16* __restrict__ gate_in, int gate_stride, int kv_heads,
                            int page_size, int window, int keep_first, float scale, float out_scale) {
    grid_launch_dependents();
    grid_dependency_wait();
    extern __shared__ __align__(16) unsigned char smem[];
    const int seq = blockIdx.y;
    const int q_begin = cu_q[seq];
    const int q_len = cu_q[seq + 1] - q_begin;
    const int tile = gridDim.x - 1 - blockIdx.x;  // the tiles with the most keys start first
    const int t0 = tile * kRows;
    if (t0 >= q_len) return;
    const int valid = min(kRows, q_len - t0);
    const int pos0 = kv_lens[seq] - q_len + t0, last_pos = pos0 + valid - 1;
    const int head = threadIdx.x >> 5, lane = threadIdx.x & 31, group_id = lane >> 2, tid4 = lane & 3;
    const int kv_head = head / (H / kv_heads);

    unsigned char* q_smem = smem;                                            // [H][16][kKRow]
    unsigned char* k_smem = q_smem + (size_t)H * kRows * kKRow;             // two stages of [kv_heads][32][kKRow]
    unsigned char* v_smem = k_smem + 2 * (size_t)kv_heads * kKeys * kKRow;  // two stages of [kv_heads][32][kVRow]
    float* w_smem = reinterpret_cast<float*>(v_smem + 2 * (size_t)kv_heads * kKeys * kVRow);  // [16][kWeightRow]: the weights
    float* m_smem = w_smem + 16 * kWeightRow;                               // [16][kWeightRow]: the mixed weights
    float* talk_smem = m_smem + 16 * kWeightRow;                            // [H][H]

    // queries: a row beyond the step's tokens repeats the last one (it is computed and not stored)
    for (int i = threadIdx.x; i < H * kRows * (D / 8); i += kThreads) {
        const int piece = i % (D / 8), row = (i / (D / 8)) % kRows, h = i / ((D / 8) * kRows);
        const int source = row < valid ? row : valid - 1;
        *reinterpret_cast<uint4*>(q_smem + (size_t)(h * kRows + row) * kKRow + piece * 16) =
            *reinterpret_cast<const uint4*>(q + (size_t)(q_begin + t0 + source) * q_stride + h * D + piece * 8);
    }
    if (talk != nullptr) {
        for (int i = threadIdx.x; i < H * H; i += kThreads) talk_smem[i] = talk[i];
        for (int i = threadIdx.x + H * kWeightRow; i < 16 * kWeightRow; i += kThreads) w_smem[i] = 0.0f;  // heads that are not there
    }
    __syncthreads();
    // the mixing matrix as the 16 x 16 left operand of a product (rows and columns beyond the heads are zero), hi + lo
    uint32_t talk_hi[4] = {0u, 0u, 0u, 0u}, talk_lo[4] = {0u, 0u, 0u, 0u};
    if (talk != nullptr) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = group_id + 8 * (j & 1), column = 2 * tid4 + 8 * (j >> 1);
            const float a = (row < H && column < H) ? talk_smem[row * H + column] : 0.0f;
            const float b = (row < H && column + 1 < H) ? talk_smem[row * H + column + 1] : 0.0f;
            const __nv_bfloat162 top = __floats2bfloat162_rn(a, b);
            const __nv_bfloat162 rest = __floats2bfloat162_rn(a - __low2float(top), b - __high2float(top));
            talk_hi[j] = *reinterpret_cast<const uint32_t*>(&top);
            talk_lo[j] = *reinterpret_cast<const uint32_t*>(&rest);
        }
    }

    int row_pos[2], row_first[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = group_id + 8 * r;
        row_pos[r] = pos0 + (row < valid ? row : valid - 1);
        row_first[r] = (window > 0 && row_pos[r] - window + 1 > 0) ? row_pos[r] - window + 1 : 0;
    }
    const TileChunks chunks(pos0, last_pos, window, keep_first);
    const int k_stage = kv_heads * kKeys * kKRow, v_stage = kv_heads * kKeys * kVRow;
    const float scale_log2 = scale * 1.4426950408889634f;
    const int* table = block_table + (size_t)seq * max_blocks;
    const uint32_t q_rows = smem_u32(q_smem) + head * kRows * kKRow;
    const uint32_t k_base = smem_u32(k_smem), v_base = smem_u32(v_smem);

    // walk 1: maximum and sum of every row of every head
    float run_max[2] = {-CUDART_INF_F, -CUDART_INF_F}, run_sum[2] = {0.0f, 0.0f};
    {
        int first, begin, end;
        chunks.chunk(0, first, begin, end);
        load_chunk<D, kKRow>(k_base, k_pool, table[first / page_size], kv_heads, page_size, first % page_size, first, last_pos, false);
        cp_async_commit();
    }
    for (int index = 0; index < chunks.total; ++index) {
        {
            int chunk, begin, end;
            cp_async_wait<0>();
            __syncthreads();  // this chunk's keys are there, and every warp is done with the chunk before it
            if (index + 1 < chunks.total) {  // the next chunk's keys are under way while this one's scores are taken
                chunks.chunk(index + 1, chunk, begin, end);
                load_chunk<D, kKRow>(k_base + ((index + 1) & 1) * k_stage, k_pool, table[chunk / page_size], kv_heads, page_size,
                                     chunk % page_size, chunk, last_pos, false);
                cp_async_commit();
            }
            chunks.chunk(index, chunk, begin, end);
            const uint32_t k_rows = k_base + (index & 1) * k_stage + kv_head * kKeys * kKRow;
            float s[4][4];
            chunk_scores(s, q_rows, k_rows);
            float part_max[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = chunk + nt * 8 + tid4 * 2 + (i & 1), r = i >> 1;
                    const bool seen = key >= begin && key < end && key <= row_pos[r] && (key >= row_first[r] || key < keep_first);
                    s[nt][i] = seen ? s[nt][i] * scale_log2 : -CUDART_INF_F;
                    part_max[r] = fmaxf(part_max[r], s[nt][i]);
                }
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                const float new_max = fmaxf(run_max[r], quad_max(part_max[r]));
                const float safe = new_max == -CUDART_INF_F ? 0.0f : new_max;  // a row that has seen nothing yet
                float local = 0.0f;
#pragma unroll
                for (int nt = 0; nt < 4; ++nt) local += exp2f(s[nt][2 * r] - safe) + exp2f(s[nt][2 * r + 1] - safe);
                run_sum[r] = run_sum[r] * exp2f(run_max[r] - safe) + local;
                run_max[r] = new_max;
            }
        }
    }
    __syncthreads();  // the second walk copies over the last chunks of the first
    float inv_sum[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) inv_sum[r] = 1.0f / quad_sum(run_sum[r]);  // every row sees its own position

    // walk 2: normalised weights, mixed across heads, applied to the values
    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    {
        int first, begin, end;
        chunks.chunk(0, first, begin, end);
        const size_t page = table[first / page_size];
        load_chunk<D, kKRow>(k_base, k_pool, page, kv_heads, page_size, first % page_size, first, last_pos, false);
        load_chunk<DV, kVRow>(v_base, v_pool, page, kv_heads, page_size, first % page_size, first, last_pos, true);
        cp_async_commit();
    }
    for (int index = 0; index < chunks.total; ++index) {
        {
            int chunk, begin, end;
            cp_async_wait<0>();
            __syncthreads();  // this chunk is there; every warp is done with the chunk before it, its weights included
            if (index + 1 < chunks.total) {
                chunks.chunk(index + 1, chunk, begin, end);
                const size_t page = table[chunk / page_size];
                const int stage = (index + 1) & 1;
                load_chunk<D, kKRow>(k_base + stage * k_stage, k_pool, page, kv_heads, page_size, chunk % page_size, chunk, last_pos, false);
                load_chunk<DV, kVRow>(v_base + stage * v_stage, v_pool, page, kv_heads, page_size, chunk % page_size, chunk, last_pos, true);
                cp_async_commit();
            }
            chunks.chunk(index, chunk, begin, end);
            const uint32_t k_rows = k_base + (index & 1) * k_stage + kv_head * kKeys * kKRow;
            const uint32_t v_rows = v_base + (index & 1) * v_stage + kv_head * kKeys * kVRow;
            float s[4][4];
            chunk_scores(s, q_rows, k_rows);
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int key = chunk + nt * 8 + tid4 * 2 + (i & 1), r = i >> 1;
                    const bool seen = key >= begin && key < end && key <= row_pos[r] && (key >= row_first[r] || key < keep_first);
                    s[nt][i] = seen ? exp2f(s[nt][i] * scale_log2 - run_max[r]) * inv_sum[r] : 0.0f;
                }
            if (talk != nullptr) {
                // every head's weights of the chunk side by side: w_smem[head][element], element = (accumulator, lane)
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) w_smem[head * kWeightRow + (nt * 4 + i) * 32 + lane] = s[nt][i];
                __syncthreads();
                // mixed[h][element] = sum_g talk[h][g] w[g][element] as products of 16 x 16 by 16 x 8 elements, the
                // elements shared out over the warps; talk and the weights each as hi + lo (lo x lo is left out)
                for (int tile = head; tile < kWeightFloats / 8; tile += H) {
                    const float* column = w_smem + tile * 8 + group_id;
                    const float x0 = column[(2 * tid4) * kWeightRow], x1 = column[(2 * tid4 + 1) * kWeightRow];
                    const float x2 = column[(2 * tid4 + 8) * kWeightRow], x3 = column[(2 * tid4 + 9) * kWeightRow];
                    const __nv_bfloat162 top0 = __floats2bfloat162_rn(x0, x1), top1 = __floats2bfloat162_rn(x2, x3);
                    const __nv_bfloat162 rest0 = __floats2bfloat162_rn(x0 - __low2float(top0), x1 - __high2float(top0));
                    const __nv_bfloat162 rest1 = __floats2bfloat162_rn(x2 - __low2float(top1), x3 - __high2float(top1));
                    const uint32_t b_hi0 = *reinterpret_cast<const uint32_t*>(&top0), b_hi1 = *reinterpret_cast<const uint32_t*>(&top1);
                    const uint32_t b_lo0 = *reinterpret_cast<const uint32_t*>(&rest0), b_lo1 = *reinterpret_cast<const uint32_t*>(&rest1);
                    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    mma_bf16(c, talk_lo, b_hi0, b_hi1);
                    mma_bf16(c, talk_hi, b_lo0, b_lo1);
                    mma_bf16(c, talk_hi, b_hi0, b_hi1);
                    float* mixed = m_smem + tile * 8 + 2 * tid4;
                    if (group_id < H) *reinterpret_cast<float2*>(mixed + group_id * kWeightRow) = make_float2(c[0], c[1]);
                    if (group_id + 8 < H) *reinterpret_cast<float2*>(mixed + (group_id + 8) * kWeightRow) = make_float2(c[2], c[3]);
                }
                __syncthreads();
#pragma unroll
                for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                    for (int i = 0; i < 4; ++i) s[nt][i] = m_smem[head * kWeightRow + (nt * 4 + i) * 32 + lane];
            }
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                uint32_t hi[4], lo[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {  // accumulators (2 part + j / 2), elements 2 (j % 2) and 2 (j % 2) + 1
                    const float a = s[2 * part + (j >> 1)][2 * (j & 1)], b = s[2 * part + (j >> 1)][2 * (j & 1) + 1];
                    const __nv_bfloat162 top = __floats2bfloat162_rn(a, b);
                    const __nv_bfloat162 rest = __floats2bfloat162_rn(a - __low2float(top), b - __high2float(top));
                    hi[j] = *reinterpret_cast<const uint32_t*>(&top);
                    lo[j] = *reinterpret_cast<const uint32_t*>(&rest);
                }
                const int v_row = part * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
                for (int dp = 0; dp < DV / 16; ++dp) {
                    uint32_t b[4];
                    ldmatrix_x4_trans(b, v_rows + v_row * kVRow + (dp * 2 + (lane >> 4)) * 16);
                    mma_bf16(o[2 * dp], hi, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], hi, b[2], b[3]);
                    mma_bf16(o[2 * dp], lo, b[0], b[1]);
                    mma_bf16(o[2 * dp + 1], lo, b[2], b[3]);
                }
            }
        }
    }

#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = group_id + 8 * r;
        if (row >= valid) continue;
        float factor = out_scale;
        if (gate_in != nullptr) {
            const float z = __bfloat162float(gate_in[(size_t)(q_begin + t0 + row) * gate_stride + head]);
            factor *= 1.0f / (1.0f + expf(-z));
        }
        bf16* dst = out + (size_t)(q_begin + t0 + row) * out_stride + (size_t)head * DV;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            const __nv_bfloat162 pair = __floats2bfloat162_rn(o[i][2 * r] * factor, o[i][2 * r + 1] * factor);
            *reinterpret_cast<uint32_t*>(dst + i * 8 + tid4 * 2) = *reinterpret_cast<const uint32_t*>(&pair);
        }
    }
}

}  // namespace mb

using namespace mb;

static size_t block_bytes(int kv_heads) {
    return (size_t)H * kRows * kKRow + 2 * (size_t)kv_heads * kKeys * (kKRow + kVRow) + sizeof(float) * (2 * 16 * (size_t)kWeightRow + H * H);
}

MB_EXPORT size_t mb_talking_attention_tc_block_bytes(int kv_heads) { return block_bytes(kv_heads); }

// As mb_talking_attention_rows (csrc/talking_attention.cu), for bfloat16 and the compiled sizes.
MB_EXPORT int mb_talking_attention_tc(const void* q, int q_stride, void* out, int out_stride, const void* k_pool,
                                      const void* v_pool, const int* block_table, int max_blocks, const int* cu_q,
                                      const int* kv_lens, int sequences, int max_q_len, const float* talk, const void* gate_in,
                                      int gate_stride, int kv_heads, int page_size, int window, int keep_first, float scale,
                                      float out_scale, cudaStream_t stream) {
    if (sequences <= 0 || max_q_len <= 0) return 0;
    if (kv_heads <= 0 || H % kv_heads) return fail("talking_attention_tc: %d heads are no multiple of %d kv heads", H, kv_heads);
    if (page_size <= 0 || page_size % kKeys) return fail("talking_attention_tc: page_size %d must be a multiple of %d", page_size, kKeys);
    if (window < 0 || keep_first < 0) return fail("talking_attention_tc: window and keep_first must not be negative");
    if (q_stride % 8 || out_stride % 2 || ((uintptr_t)q & 15) || ((uintptr_t)out & 3) || ((uintptr_t)k_pool & 15) || ((uintptr_t)v_pool & 15))
        return fail("talking_attention_tc: q rows must start on 16 bytes, out rows on 4, the pools on 16");
    if (sequences > 65535) return fail("talking_attention_tc: %d sequences exceed the grid limit 65535", sequences);
    const size_t smem = block_bytes(kv_heads);
    if (smem > 227 * 1024) return fail("talking_attention_tc: a block would need %zu bytes of shared memory", smem);
    static bool configured[64] = {false};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 64 && !configured[device]) {
        cudaError_t status = cudaFuncSetAttribute(talking_attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
        if (status != cudaSuccess) return fail("talking_attention_tc: cannot reserve shared memory: %s", cudaGetErrorString(status));
        configured[device] = true;
    }
    const dim3 grid((max_q_len + kRows - 1) / kRows, sequences);
    MB_LAUNCH("talking_attention_tc", talking_attention_tc_kernel, dim3(grid), dim3(kThreads), smem, stream, true,
                  (const bf16*)q, q_stride, (bf16*)out, out_stride, (const bf16*)k_pool, (const bf16*)v_pool,
                  block_table, max_blocks, cu_q, kv_lens, talk, (const bf16*)gate_in, gate_stride, kv_heads, page_size,
                  window, keep_first, scale, out_scale);
    return check_launch("talking_attention_tc");
}
