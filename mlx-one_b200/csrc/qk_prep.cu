// Per-head RMSNorm of queries and keys, rotary position encoding, and the write of keys and
// values into the request's pages.
//
// qkv[t] = [q heads | k heads | v heads], each head of head_dim values. One warp handles one
// (token, head): it norms q or k over head_dim in 32-bit (if a norm weight is given), rotates
// the first rotary_dim dimensions by position * inv_freq (pairs j and j + rotary_dim/2, the
// non-interleaved form; angles in 32-bit), writes q to q_out[t, head, :] and k, v to
// kv[0 or 1, page, kv_head, position % page_size, :] with page = block_table[request,
// position / page_size].
#include "common.cuh"

namespace {

constexpr int WARPS = 8;
constexpr int MAX_HEAD_DIM = 512;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
qk_prep_kernel(const T* __restrict__ qkv, const float* __restrict__ q_weight,
               const float* __restrict__ k_weight, float eps, const float* __restrict__ inv_freq,
               int rotary_dim, const int* __restrict__ positions,
               const int* __restrict__ token_request, T* __restrict__ q_out,
               T* __restrict__ kv, const int* __restrict__ block_table, int table_width,
               int page_size, long long kv_half, int tokens, int heads, int kv_heads,
               int head_dim, int write_kv, int* __restrict__ error_flag) {
    extern __shared__ float shared[];
    griddep_launch();
    griddep_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots_per_token = heads + 2 * kv_heads;
    const long long item = (long long)blockIdx.x * WARPS + warp;
    if (item >= (long long)tokens * slots_per_token) return;
    const int t = (int)(item / slots_per_token);
    const int slot = (int)(item % slots_per_token);
    float* values = shared + warp * head_dim;

    const T* src = qkv + (size_t)t * slots_per_token * head_dim + (size_t)slot * head_dim;
    const bool is_q = slot < heads;
    const bool is_k = !is_q && slot < heads + kv_heads;
    if (!is_q && !write_kv) return;

    float sum = 0.f;
    for (int e = lane; e < head_dim; e += 32) {
        const float v = to_float<T>(src[e]);
        values[e] = v;
        sum += v * v;
    }
    const int position = positions[t];
    if (is_q || is_k) {
        const float* weight = is_q ? q_weight : k_weight;
        if (weight != nullptr) {
            sum = warp_sum(sum);
            const float inv = rsqrtf(sum / (float)head_dim + eps);
            for (int e = lane; e < head_dim; e += 32) values[e] = values[e] * inv * weight[e];
        }
        __syncwarp();
        if (inv_freq != nullptr) {
            const int half = rotary_dim / 2;
            for (int j = lane; j < half; j += 32) {
                const float angle = (float)position * inv_freq[j];
                float sine, cosine;
                sincosf(angle, &sine, &cosine);
                const float a = values[j], b = values[j + half];
                values[j] = a * cosine - b * sine;
                values[j + half] = b * cosine + a * sine;
            }
        }
    }
    __syncwarp();

    T* dst;
    if (is_q) {
        dst = q_out + ((size_t)t * heads + slot) * head_dim;
    } else {
        const int kv_head = is_k ? slot - heads : slot - heads - kv_heads;
        const int r = token_request[t];
        const int block = position / page_size;
        const int page = block < table_width ? block_table[(size_t)r * table_width + block] : -1;
        if (page < 0) {
            if (lane == 0) atomicExch(error_flag, 2);
            return;
        }
        dst = kv + (is_k ? 0 : kv_half) +
              (((size_t)page * kv_heads + kv_head) * page_size + position % page_size) * head_dim;
    }
    for (int e = lane; e < head_dim; e += 32) dst[e] = from_float<T>(values[e]);
}

// bfloat16 with a head size of 32, 64, 128 or 256 that is rotated as a whole (or not at all):
// a lane keeps HD/32 neighbouring values of the head in registers, its rotation partner sits 16
// lanes away, and the angles are computed once per token, not once per head. One block per
// token; its warps take the token's heads in turn.
template <int HD>
__global__ void __launch_bounds__(WARPS * 32)
qk_prep_wide_kernel(const __nv_bfloat16* __restrict__ qkv, const float* __restrict__ q_weight,
                    const float* __restrict__ k_weight, float eps,
                    const float* __restrict__ inv_freq, const int* __restrict__ positions,
                    const int* __restrict__ token_request, __nv_bfloat16* __restrict__ q_out,
                    __nv_bfloat16* __restrict__ kv, const int* __restrict__ block_table,
                    int table_width, int page_size, long long kv_half, int heads, int kv_heads,
                    int write_kv, int* __restrict__ error_flag) {
    using T = __nv_bfloat16;
    constexpr int E = HD / 32;
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int slots = heads + 2 * kv_heads;
    const int e0 = E * lane;
    // AHEAD of the warp's heads at a time: their loads are issued together, the first ones
    // before anything that waits for the token's position or page
    constexpr int AHEAD = 6;
    const T* row = qkv + (size_t)t * slots * HD;
    float held[AHEAD][E];
    auto load_heads = [&](int base) {
#pragma unroll
        for (int a = 0; a < AHEAD; ++a) {
            const int slot = base + a * WARPS;
            if (slot >= slots) continue;
            const T* src = row + (size_t)slot * HD + e0;
            if (E == 1) {
                held[a][0] = __bfloat162float(src[0]);
            } else {
#pragma unroll
                for (int i = 0; i < E; i += 2) {
                    const __nv_bfloat162 pair = *reinterpret_cast<const __nv_bfloat162*>(src + i);
                    held[a][i] = __low2float(pair);
                    held[a][i + 1] = __high2float(pair);
                }
            }
        }
    };
    load_heads(warp);
    const int position = positions[t];
    float cosine[E], sine[E], q_scale[E], k_scale[E];
#pragma unroll
    for (int i = 0; i < E; ++i) {
        cosine[i] = 1.f;
        sine[i] = 0.f;
        if (inv_freq != nullptr) {
            const float angle = (float)position * inv_freq[(e0 + i) % (HD / 2)];
            sincosf(angle, &sine[i], &cosine[i]);
            if (lane < 16) sine[i] = -sine[i];       // first half: a cos - b sin
        }
        q_scale[i] = q_weight ? q_weight[e0 + i] : 1.f;
        k_scale[i] = k_weight ? k_weight[e0 + i] : 1.f;
    }
    // where this token's keys and values go
    T* page_base = nullptr;
    if (write_kv) {
        const int r = token_request[t];
        const int block = position / page_size;
        const int page = block < table_width ? block_table[(size_t)r * table_width + block] : -1;
        if (page < 0) {
            if (threadIdx.x == 0) atomicExch(error_flag, 2);
        } else {
            page_base = kv + ((size_t)page * kv_heads * page_size + position % page_size) * HD;
        }
    }
    for (int base = warp; base < slots; base += AHEAD * WARPS) {
        if (base != warp) load_heads(base);
#pragma unroll
        for (int a = 0; a < AHEAD; ++a) {
            const int slot = base + a * WARPS;
            if (slot >= slots) continue;
            const bool is_q = slot < heads;
            const bool is_k = !is_q && slot < heads + kv_heads;
            if (!is_q && page_base == nullptr) continue;
            float (&v)[E] = held[a];
            if (is_q || is_k) {
                const float* scale = is_q ? q_scale : k_scale;
                if ((is_q ? q_weight : k_weight) != nullptr) {
                    float sum = 0.f;
#pragma unroll
                    for (int i = 0; i < E; ++i) sum += v[i] * v[i];
                    sum = warp_sum(sum);
                    const float inv = rsqrtf(sum / (float)HD + eps);
#pragma unroll
                    for (int i = 0; i < E; ++i) v[i] = v[i] * inv * scale[i];
                }
                if (inv_freq != nullptr) {
#pragma unroll
                    for (int i = 0; i < E; ++i) {
                        const float partner = __shfl_xor_sync(0xffffffffu, v[i], 16);
                        v[i] = v[i] * cosine[i] + partner * sine[i];
                    }
                }
            }
            T* dst;
            if (is_q) {
                dst = q_out + ((size_t)t * heads + slot) * HD + e0;
            } else {
                const int kv_head = is_k ? slot - heads : slot - heads - kv_heads;
                dst = page_base + (is_k ? 0 : kv_half) + (size_t)kv_head * page_size * HD + e0;
            }
            if (E == 1) {
                dst[0] = __float2bfloat16_rn(v[0]);
            } else {
#pragma unroll
                for (int i = 0; i < E; i += 2)
                    *reinterpret_cast<__nv_bfloat162*>(dst + i) = __floats2bfloat162_rn(v[i], v[i + 1]);
            }
        }
    }
}

template <int HD>
static void launch_qk_prep_wide(const void* qkv, const float* q_weight, const float* k_weight,
                                float eps, const float* inv_freq, const int* positions,
                                const int* token_request, void* q_out, void* kv,
                                const int* block_table, int table_width, int page_size,
                                long long kv_half, int tokens, int heads, int kv_heads,
                                int write_kv, int* error_flag, cudaStream_t stream) {
    using T = __nv_bfloat16;
    launch_kernel(qk_prep_wide_kernel<HD>, dim3(tokens), dim3(WARPS * 32), 0, stream, true,
                  (const T*)qkv, q_weight, k_weight, eps, inv_freq, positions, token_request,
                  (T*)q_out, (T*)kv, block_table, table_width, page_size, kv_half, heads, kv_heads,
                  write_kv, error_flag);
}

}  // namespace

MLXONE_API int mlxone_qk_prep(const void* qkv, const float* q_weight, const float* k_weight,
                              float eps, const float* inv_freq, int rotary_dim,
                              const int* positions, const int* token_request, void* q_out,
                              void* kv, const int* block_table, int table_width, int page_size,
                              int pages, int tokens, int heads, int kv_heads, int head_dim,
                              int write_kv, int dtype, int* error_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && heads > 0 && kv_heads > 0, "qk_prep: bad sizes");
    MLXONE_REQUIRE(head_dim >= 2 && head_dim <= MAX_HEAD_DIM,
                   "qk_prep: head size %d is not in 2..%d", head_dim, MAX_HEAD_DIM);
    MLXONE_REQUIRE(inv_freq == nullptr ||
                       (rotary_dim > 0 && rotary_dim % 2 == 0 && rotary_dim <= head_dim),
                   "qk_prep: rotary size %d must be even and at most the head size %d", rotary_dim,
                   head_dim);
    MLXONE_REQUIRE(page_size > 0 && pages > 0 && table_width > 0, "qk_prep: bad page geometry");
    const long long items = (long long)tokens * (heads + 2 * kv_heads);
    const int blocks = ceil_div_host(items, WARPS);
    const size_t shared = (size_t)WARPS * head_dim * sizeof(float);
    const long long kv_half = (long long)pages * kv_heads * page_size * head_dim;
    const bool whole = inv_freq == nullptr || rotary_dim == head_dim;
    if (dtype == MLXONE_BF16 && whole &&
        (head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256)) {
#define WIDE(HD)                                                                                 \
    launch_qk_prep_wide<HD>(qkv, q_weight, k_weight, eps, inv_freq, positions, token_request,   \
                            q_out, kv, block_table, table_width, page_size, kv_half, tokens,    \
                            heads, kv_heads, write_kv, error_flag, stream)
        if (head_dim == 32) WIDE(32);
        else if (head_dim == 64) WIDE(64);
        else if (head_dim == 128) WIDE(128);
        else WIDE(256);
#undef WIDE
    } else if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        launch_kernel(qk_prep_kernel<T>, dim3(blocks), dim3(WARPS * 32), shared, stream, true, (const T*)qkv, q_weight, k_weight, eps, inv_freq, rotary_dim, positions,
            token_request, (T*)q_out, (T*)kv, block_table, table_width, page_size, kv_half,
            tokens, heads, kv_heads, head_dim, write_kv, error_flag);
    } else {
        using T = float;
        launch_kernel(qk_prep_kernel<T>, dim3(blocks), dim3(WARPS * 32), shared, stream, true, (const T*)qkv, q_weight, k_weight, eps, inv_freq, rotary_dim, positions,
            token_request, (T*)q_out, (T*)kv, block_table, table_width, page_size, kv_half,
            tokens, heads, kv_heads, head_dim, write_kv, error_flag);
    }
    MLXONE_LAUNCH_CHECK("qk_prep");
    return 0;
}
