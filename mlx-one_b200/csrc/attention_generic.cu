// Paged grouped-query attention for any batch: the general kernel.
//
// One warp per (token, query head). The query at position p reads the keys of its request at
// positions max(0, p - window + 1) .. p from the request's pages (this step's own keys have
// been written there before). Keys are taken 32 at a time, in blocks aligned to absolute
// positions, one key per lane; softmax statistics and the output are kept in 32-bit and
// updated block by block (online softmax). The order of operations for a query depends only
// on its position, never on how the tokens were cut into steps or batched.
//
// This kernel serves the 32-bit engine and every shape that the faster kernels refuse.
#include "common.cuh"

namespace {

constexpr int WARPS = 4;
constexpr int MAX_HEAD_DIM = 512;
constexpr int MAX_ACC = MAX_HEAD_DIM / 32;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ kv,
                         const int* __restrict__ block_table, int table_width, int page_size,
                         long long kv_half, const int* __restrict__ positions,
                         const int* __restrict__ token_request, T* __restrict__ out, int tokens,
                         int heads, int kv_heads, int head_dim, float scale, int window,
                         int* __restrict__ error_flag) {
    extern __shared__ float shared[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads);
    const int head = (int)(item % heads);
    const int kv_head = head / (heads / kv_heads);
    const int r = token_request[t];
    const int position = positions[t];
    const int* table = block_table + (size_t)r * table_width;

    float* query = shared + warp * head_dim;
    const T* q_row = q + ((size_t)t * heads + head) * head_dim;
    for (int e = lane; e < head_dim; e += 32) query[e] = to_float<T>(q_row[e]) * scale;
    __syncwarp();

    const int lowest = window > 0 ? max(position - window + 1, 0) : 0;
    float running_max = -INFINITY, running_sum = 0.f;
    float acc[MAX_ACC];
#pragma unroll
    for (int i = 0; i < MAX_ACC; ++i) acc[i] = 0.f;
    const int pieces = (head_dim + 31) / 32;

    for (int base = (lowest / 32) * 32; base <= position; base += 32) {
        const int key = base + lane;
        const bool live = key >= lowest && key <= position;
        float score = -INFINITY;
        const T* key_row = nullptr;
        if (live) {
            const int block = key / page_size;
            const int page = block < table_width ? table[block] : -1;
            if (page < 0) {
                atomicExch(error_flag, 3);
            } else {
                key_row = kv + (((size_t)page * kv_heads + kv_head) * page_size +
                                key % page_size) * head_dim;
                float dot = 0.f;
                for (int e = 0; e < head_dim; ++e) dot = fmaf(query[e], to_float<T>(key_row[e]), dot);
                score = dot;
            }
        }
        const float block_max = warp_max(score);
        const float new_max = fmaxf(running_max, block_max);
        if (new_max == -INFINITY) continue;           // nothing live in this block
        const float weight = key_row != nullptr ? expf(score - new_max) : 0.f;
        const float correction = expf(running_max - new_max);   // 0 when running_max = -inf
        running_sum = running_sum * correction + warp_sum(weight);
        running_max = new_max;
#pragma unroll
        for (int i = 0; i < MAX_ACC; ++i)
            if (i < pieces) acc[i] *= correction;
        for (int j = 0; j < 32; ++j) {
            const float w = __shfl_sync(0xffffffffu, weight, j);
            // every lane follows lane j's value row; rows of dead keys carry weight 0
            const unsigned long long row_bits =
                __shfl_sync(0xffffffffu, (unsigned long long)(uintptr_t)key_row, j);
            if (row_bits == 0ull) continue;
            const T* value_row = reinterpret_cast<const T*>((uintptr_t)row_bits) + kv_half;
#pragma unroll
            for (int i = 0; i < MAX_ACC; ++i) {
                const int e = lane + 32 * i;
                if (i < pieces && e < head_dim) acc[i] = fmaf(w, to_float<T>(value_row[e]), acc[i]);
            }
        }
    }
    T* out_row = out + ((size_t)t * heads + head) * head_dim;
    const float inv = running_sum > 0.f ? 1.f / running_sum : 0.f;
#pragma unroll
    for (int i = 0; i < MAX_ACC; ++i) {
        const int e = lane + 32 * i;
        if (i < pieces && e < head_dim) out_row[e] = from_float<T>(acc[i] * inv);
    }
}

}  // namespace

MLXONE_API int mlxone_attention_generic(const void* q, const void* kv, const int* block_table,
                                        int table_width, int page_size, int pages,
                                        const int* positions, const int* token_request, void* out,
                                        int tokens, int heads, int kv_heads, int head_dim,
                                        float scale, int window, int dtype, int* error_flag,
                                        cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                   "attention: %d heads cannot share %d key heads", heads, kv_heads);
    MLXONE_REQUIRE(head_dim >= 1 && head_dim <= MAX_HEAD_DIM,
                   "attention: head size %d is not in 1..%d", head_dim, MAX_HEAD_DIM);
    MLXONE_REQUIRE(page_size > 0 && pages > 0 && table_width > 0, "attention: bad page geometry");
    const long long items = (long long)tokens * heads;
    const int blocks = ceil_div_host(items, WARPS);
    const size_t shared = (size_t)WARPS * head_dim * sizeof(float);
    const long long kv_half = (long long)pages * kv_heads * page_size * head_dim;
    if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        attention_generic_kernel<T><<<blocks, WARPS * 32, shared, stream>>>(
            (const T*)q, (const T*)kv, block_table, table_width, page_size, kv_half, positions,
            token_request, (T*)out, tokens, heads, kv_heads, head_dim, scale, window, error_flag);
    } else {
        using T = float;
        attention_generic_kernel<T><<<blocks, WARPS * 32, shared, stream>>>(
            (const T*)q, (const T*)kv, block_table, table_width, page_size, kv_half, positions,
            token_request, (T*)out, tokens, heads, kv_heads, head_dim, scale, window, error_flag);
    }
    MLXONE_LAUNCH_CHECK("attention_generic");
    return 0;
}
