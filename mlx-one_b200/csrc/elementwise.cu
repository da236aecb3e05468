// Embedding lookup, residual add + RMSNorm, row gather, SwiGLU gate, bias add.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// out[t, :] = float(table[ids[t], :]). The residual stream is 32-bit.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab,
                                 int* __restrict__ error_flag) {
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        id = 0;
    }
    const T* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)t * hidden;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_float<T>(row[c]);
}

MLXONE_API int mlxone_embedding(const int* ids, const void* table, float* out, int tokens,
                                int hidden, int vocab, int dtype, int* error_flag,
                                cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16)
        embedding_kernel<__nv_bfloat16><<<tokens, threads, 0, stream>>>(
            ids, (const __nv_bfloat16*)table, out, hidden, vocab, error_flag);
    else
        embedding_kernel<float><<<tokens, threads, 0, stream>>>(ids, (const float*)table, out,
                                                               hidden, vocab, error_flag);
    MLXONE_LAUNCH_CHECK("embedding");
    return 0;
}

// ------------------------------------------------------------------ add + RMSNorm
// residual[t, :] += delta[t, :] (if delta); out[t, :] = residual * rsqrt(mean(residual^2)
// + eps) * weight. One block per row; sums in 32-bit in an order fixed by the row length.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                   const float* __restrict__ weight, T* __restrict__ out,
                                   int hidden, float eps) {
    __shared__ float scratch[33];
    const size_t base = (size_t)blockIdx.x * hidden;
    float sum = 0.f;
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        float v = residual[base + c];
        if (delta != nullptr) {
            v += to_float<T>(delta[base + c]);
            residual[base + c] = v;
        }
        sum += v * v;
    }
    const float total = block_sum(sum, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x)
        out[base + c] = from_float<T>(residual[base + c] * inv * weight[c]);
}

MLXONE_API int mlxone_add_rmsnorm(float* residual, const void* delta, const float* weight,
                                  void* out, int rows, int hidden, float eps, int dtype,
                                  cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && hidden > 0, "add_rmsnorm: bad sizes");
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    if (dtype == MLXONE_BF16)
        add_rmsnorm_kernel<__nv_bfloat16><<<rows, threads, 0, stream>>>(
            residual, (const __nv_bfloat16*)delta, weight, (__nv_bfloat16*)out, hidden, eps);
    else
        add_rmsnorm_kernel<float><<<rows, threads, 0, stream>>>(
            residual, (const float*)delta, weight, (float*)out, hidden, eps);
    MLXONE_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

// ------------------------------------------------------------------ row gather
// picked[i, :] = residual[rows[i], :]; picked_delta[i, :] = delta[rows[i], :] (if delta).
template <typename T>
__global__ void gather_rows_kernel(const float* __restrict__ residual, const T* __restrict__ delta,
                                   const int* __restrict__ rows, float* __restrict__ picked,
                                   T* __restrict__ picked_delta, int hidden, int tokens) {
    int src = rows[blockIdx.x];
    src = min(max(src, 0), tokens - 1);
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        picked[(size_t)blockIdx.x * hidden + c] = residual[(size_t)src * hidden + c];
        if (delta != nullptr)
            picked_delta[(size_t)blockIdx.x * hidden + c] = delta[(size_t)src * hidden + c];
    }
}

MLXONE_API int mlxone_gather_rows(const float* residual, const void* delta, const int* rows,
                                  float* picked, void* picked_delta, int count, int hidden,
                                  int tokens, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    MLXONE_REQUIRE(count > 0 && hidden > 0 && tokens > 0, "gather_rows: bad sizes");
    if (dtype == MLXONE_BF16)
        gather_rows_kernel<__nv_bfloat16><<<count, 256, 0, stream>>>(
            residual, (const __nv_bfloat16*)delta, rows, picked, (__nv_bfloat16*)picked_delta,
            hidden, tokens);
    else
        gather_rows_kernel<float><<<count, 256, 0, stream>>>(
            residual, (const float*)delta, rows, picked, (float*)picked_delta, hidden, tokens);
    MLXONE_LAUNCH_CHECK("gather_rows");
    return 0;
}

// ------------------------------------------------------------------ SwiGLU gate
// out[t, f] = silu(gate_up[t, f]) * gate_up[t, width + f], in 32-bit.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int width,
                              long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / width;
    const int f = (int)(i - t * width);
    const float gate = to_float<T>(gate_up[t * 2 * width + f]);
    const float up = to_float<T>(gate_up[t * 2 * width + width + f]);
    out[i] = from_float<T>(gate / (1.f + expf(-gate)) * up);
}

MLXONE_API int mlxone_swiglu(const void* gate_up, void* out, int rows, int width, int dtype,
                             cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && width > 0, "swiglu: bad sizes");
    const long long total = (long long)rows * width;
    const int blocks = ceil_div_host(total, 256);
    if (dtype == MLXONE_BF16)
        swiglu_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>(
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, width, total);
    else
        swiglu_kernel<float><<<blocks, 256, 0, stream>>>((const float*)gate_up, (float*)out,
                                                        width, total);
    MLXONE_LAUNCH_CHECK("swiglu");
    return 0;
}

// ------------------------------------------------------------------ bias add
template <typename T>
__global__ void add_bias_kernel(T* __restrict__ x, const float* __restrict__ bias, int width,
                                long long total) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    x[i] = from_float<T>(to_float<T>(x[i]) + bias[i % width]);
}

MLXONE_API int mlxone_add_bias(void* x, const float* bias, int rows, int width, int dtype,
                               cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && width > 0, "add_bias: bad sizes");
    const long long total = (long long)rows * width;
    const int blocks = ceil_div_host(total, 256);
    if (dtype == MLXONE_BF16)
        add_bias_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)x, bias, width,
                                                                  total);
    else
        add_bias_kernel<float><<<blocks, 256, 0, stream>>>((float*)x, bias, width, total);
    MLXONE_LAUNCH_CHECK("add_bias");
    return 0;
}
