// Embedding lookup, residual add + RMSNorm, row gather, SwiGLU gate, bias add.
#include "common.cuh"

// ------------------------------------------------------------------ embedding
// out[t, :] = float(table[ids[t], :]). The residual stream is 32-bit.
template <typename T>
__global__ void embedding_kernel(const int* __restrict__ ids, const T* __restrict__ table,
                                 float* __restrict__ out, int hidden, int vocab,
                                 int* __restrict__ error_flag) {
    griddep_launch();
    griddep_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 || id >= vocab) {
        if (threadIdx.x == 0) atomicExch(error_flag, 1);
        id = 0;
    }
    const T* row = table + (size_t)id * hidden;
    float* dst = out + (size_t)t * hidden;
    if (sizeof(T) == 2 && hidden % 8 == 0 && (reinterpret_cast<uintptr_t>(table) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
        // eight values a load: the whole row is asked for at once (it comes from DRAM, and a
        // decode step begins with this kernel)
        for (int c = threadIdx.x * 8; c < hidden; c += blockDim.x * 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(row + c);
            const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&raw);
            float4 lo, hi;
            lo.x = __low2float(pairs[0]); lo.y = __high2float(pairs[0]);
            lo.z = __low2float(pairs[1]); lo.w = __high2float(pairs[1]);
            hi.x = __low2float(pairs[2]); hi.y = __high2float(pairs[2]);
            hi.z = __low2float(pairs[3]); hi.w = __high2float(pairs[3]);
            *reinterpret_cast<float4*>(dst + c) = lo;
            *reinterpret_cast<float4*>(dst + c + 4) = hi;
        }
        return;
    }
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) dst[c] = to_float<T>(row[c]);
}

MLXONE_API int mlxone_embedding(const int* ids, const void* table, float* out, int tokens,
                                int hidden, int vocab, int dtype, int* error_flag,
                                cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && hidden > 0 && vocab > 0, "embedding: bad sizes");
    const int threads = hidden >= 1024 ? 256 : 128;
    if (dtype == MLXONE_BF16)
        launch_kernel(embedding_kernel<__nv_bfloat16>, dim3(tokens), dim3(threads), 0, stream, true,
                      ids, (const __nv_bfloat16*)table, out, hidden, vocab, error_flag);
    else
        launch_kernel(embedding_kernel<float>, dim3(tokens), dim3(threads), 0, stream, true, ids,
                      (const float*)table, out, hidden, vocab, error_flag);
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
    griddep_launch();
    griddep_wait();
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

// The same for rows of up to 4 * blockDim.x * PASSES values with hidden % 4 == 0: every value
// stays in a register between the sum and the scaling, so the row is read once.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[4]) {
        const uint2 x = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&x.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&x.y);
        v[0] = __low2float(lo); v[1] = __high2float(lo);
        v[2] = __low2float(hi); v[3] = __high2float(hi);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&v)[4]) {
        const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]);
        const __nv_bfloat162 hi = __floats2bfloat162_rn(v[2], v[3]);
        uint2 x;
        x.x = *reinterpret_cast<const uint32_t*>(&lo);
        x.y = *reinterpret_cast<const uint32_t*>(&hi);
        *reinterpret_cast<uint2*>(p) = x;
    }
};

template <typename T, int PASSES>
__global__ void add_rmsnorm_rows_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                                        const float* __restrict__ weight, T* __restrict__ out,
                                        int hidden, float eps) {
    __shared__ float scratch[33];
    griddep_launch();
    // the norm's weights do not depend on the kernel before this one: they are on their way
    // while it finishes, and the row's values are the only round trip after it
    float scale[PASSES][4];
#pragma unroll
    for (int pass = 0; pass < PASSES; ++pass) {
        const int c = (pass * blockDim.x + threadIdx.x) * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) scale[pass][i] = 0.f;
        if (c < hidden) Vec4<float>::load(weight + c, scale[pass]);
    }
    griddep_wait();
    const size_t base = (size_t)blockIdx.x * hidden;
    float values[PASSES][4];
    float sum = 0.f;
#pragma unroll
    for (int pass = 0; pass < PASSES; ++pass) {
        const int c = (pass * blockDim.x + threadIdx.x) * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) values[pass][i] = 0.f;
        if (c < hidden) {
            Vec4<float>::load(residual + base + c, values[pass]);
            if (delta != nullptr) {
                float more[4];
                Vec4<T>::load(delta + base + c, more);
#pragma unroll
                for (int i = 0; i < 4; ++i) values[pass][i] += more[i];
                Vec4<float>::store(residual + base + c, values[pass]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) sum += values[pass][i] * values[pass][i];
        }
    }
    const float total = block_sum(sum, scratch);
    const float inv = rsqrtf(total / (float)hidden + eps);
#pragma unroll
    for (int pass = 0; pass < PASSES; ++pass) {
        const int c = (pass * blockDim.x + threadIdx.x) * 4;
        if (c < hidden) {
            float result[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) result[i] = values[pass][i] * inv * scale[pass][i];
            Vec4<T>::store(out + base + c, result);
        }
    }
}

// Many rows (prefill): one warp per row, the whole row in registers (hidden <= 128 * VEC * ... ),
// all of a lane's loads in flight together and no block-wide barrier.
template <typename T, int VEC>
__global__ void __launch_bounds__(256)
add_rmsnorm_warp_kernel(float* __restrict__ residual, const T* __restrict__ delta,
                        const float* __restrict__ weight, T* __restrict__ out, int rows,
                        int hidden, float eps) {
    griddep_launch();
    griddep_wait();
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (row >= rows) return;
    const size_t base = (size_t)row * hidden;
    float values[VEC][4];
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const int c = (j * 32 + lane) * 4;
#pragma unroll
        for (int i = 0; i < 4; ++i) values[j][i] = 0.f;
        if (c < hidden) Vec4<float>::load(residual + base + c, values[j]);
    }
    if (delta != nullptr) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const int c = (j * 32 + lane) * 4;
            if (c < hidden) {
                float more[4];
                Vec4<T>::load(delta + base + c, more);
#pragma unroll
                for (int i = 0; i < 4; ++i) values[j][i] += more[i];
                Vec4<float>::store(residual + base + c, values[j]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < VEC; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) sum += values[j][i] * values[j][i];
    sum = warp_sum(sum);
    const float inv = rsqrtf(sum / (float)hidden + eps);
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const int c = (j * 32 + lane) * 4;
        if (c < hidden) {
            float scale[4], result[4];
            Vec4<float>::load(weight + c, scale);
#pragma unroll
            for (int i = 0; i < 4; ++i) result[i] = values[j][i] * inv * scale[i];
            Vec4<T>::store(out + base + c, result);
        }
    }
}

template <typename T>
static cudaError_t launch_add_rmsnorm(float* residual, const void* delta, const float* weight,
                                      void* out, int rows, int hidden, float eps,
                                      cudaStream_t stream) {
    const bool aligned = hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(residual) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(weight) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(out) & 7) == 0 &&
                         (reinterpret_cast<uintptr_t>(delta) & 7) == 0;
    // measured at 2048 columns: a block per row is faster up to about a thousand rows (64 rows:
    // 1.7 us against 2.6 us), a warp per row beyond (2048 rows: 3.5 us against 5.6 us)
    if (aligned && rows >= 1536 && hidden <= 2048) {
        const dim3 grid((rows + 7) / 8);
        if (hidden <= 512)
            return launch_kernel(add_rmsnorm_warp_kernel<T, 4>, grid, dim3(256), 0, stream, true,
                                 residual, (const T*)delta, weight, (T*)out, rows, hidden, eps);
        if (hidden <= 1024)
            return launch_kernel(add_rmsnorm_warp_kernel<T, 8>, grid, dim3(256), 0, stream, true,
                                 residual, (const T*)delta, weight, (T*)out, rows, hidden, eps);
        return launch_kernel(add_rmsnorm_warp_kernel<T, 16>, grid, dim3(256), 0, stream, true,
                             residual, (const T*)delta, weight, (T*)out, rows, hidden, eps);
    }
    if (aligned && hidden <= 8192) {
        const int quads = hidden / 4;
        const int passes = quads <= 1024 ? 1 : 2;
        int threads = ((quads + passes - 1) / passes + 31) / 32 * 32;
        if (passes == 1)
            return launch_kernel(add_rmsnorm_rows_kernel<T, 1>, dim3(rows), dim3(threads), 0, stream,
                                 true, residual, (const T*)delta, weight, (T*)out, hidden, eps);
        return launch_kernel(add_rmsnorm_rows_kernel<T, 2>, dim3(rows), dim3(threads), 0, stream,
                             true, residual, (const T*)delta, weight, (T*)out, hidden, eps);
    }
    const int threads = hidden >= 2048 ? 512 : (hidden >= 512 ? 256 : 128);
    return launch_kernel(add_rmsnorm_kernel<T>, dim3(rows), dim3(threads), 0, stream, true, residual,
                         (const T*)delta, weight, (T*)out, hidden, eps);
}

MLXONE_API int mlxone_add_rmsnorm(float* residual, const void* delta, const float* weight,
                                  void* out, int rows, int hidden, float eps, int dtype,
                                  cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && hidden > 0, "add_rmsnorm: bad sizes");
    if (dtype == MLXONE_BF16)
        launch_add_rmsnorm<__nv_bfloat16>(residual, delta, weight, out, rows, hidden, eps, stream);
    else
        launch_add_rmsnorm<float>(residual, delta, weight, out, rows, hidden, eps, stream);
    MLXONE_LAUNCH_CHECK("add_rmsnorm");
    return 0;
}

// ------------------------------------------------------------------ row gather
// picked[i, :] = residual[rows[i], :]; picked_delta[i, :] = delta[rows[i], :] (if delta).
template <typename T>
__global__ void gather_rows_kernel(const float* __restrict__ residual, const T* __restrict__ delta,
                                   const int* __restrict__ rows, float* __restrict__ picked,
                                   T* __restrict__ picked_delta, int hidden, int tokens) {
    griddep_launch();
    griddep_wait();
    int src = rows[blockIdx.x];
    src = min(max(src, 0), tokens - 1);
    const float* from = residual + (size_t)src * hidden;
    float* to = picked + (size_t)blockIdx.x * hidden;
    if (hidden % 4 == 0 && (reinterpret_cast<uintptr_t>(residual) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(picked) & 15) == 0) {
        // 16 bytes a load, so that a row's loads are on their way together
        for (int c = threadIdx.x * 4; c < hidden; c += blockDim.x * 4)
            *reinterpret_cast<float4*>(to + c) = *reinterpret_cast<const float4*>(from + c);
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) to[c] = from[c];
    }
    if (delta != nullptr)
        for (int c = threadIdx.x; c < hidden; c += blockDim.x)
            picked_delta[(size_t)blockIdx.x * hidden + c] = delta[(size_t)src * hidden + c];
}

MLXONE_API int mlxone_gather_rows(const float* residual, const void* delta, const int* rows,
                                  float* picked, void* picked_delta, int count, int hidden,
                                  int tokens, int dtype, cudaStream_t stream) {
    if (count == 0) return 0;
    MLXONE_REQUIRE(count > 0 && hidden > 0 && tokens > 0, "gather_rows: bad sizes");
    if (dtype == MLXONE_BF16)
        launch_kernel(gather_rows_kernel<__nv_bfloat16>, dim3(count), dim3(256), 0, stream, true,
                      residual, (const __nv_bfloat16*)delta, rows, picked,
                      (__nv_bfloat16*)picked_delta, hidden, tokens);
    else
        launch_kernel(gather_rows_kernel<float>, dim3(count), dim3(256), 0, stream, true, residual,
                      (const float*)delta, rows, picked, (float*)picked_delta, hidden, tokens);
    MLXONE_LAUNCH_CHECK("gather_rows");
    return 0;
}

// ------------------------------------------------------------------ SwiGLU gate
// out[t, f] = silu(gate_up[t, f]) * gate_up[t, width + f], in 32-bit.
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int width,
                              long long total) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const long long t = i / width;
    const int f = (int)(i - t * width);
    const float gate = to_float<T>(gate_up[t * 2 * width + f]);
    const float up = to_float<T>(gate_up[t * 2 * width + width + f]);
    out[i] = from_float<T>(gate / (1.f + expf(-gate)) * up);
}

// The same for bfloat16 with width % 8 == 0: eight neighbouring values a thread, 16-byte loads.
__global__ void swiglu_wide_kernel(const __nv_bfloat16* __restrict__ gate_up,
                                   __nv_bfloat16* __restrict__ out, int width, long long groups) {
    griddep_launch();
    griddep_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= groups) return;
    const int per_row = width / 8;
    const long long t = i / per_row;
    const int f = (int)(i - t * per_row) * 8;
    const uint4 g = *reinterpret_cast<const uint4*>(gate_up + t * 2 * width + f);
    const uint4 u = *reinterpret_cast<const uint4*>(gate_up + t * 2 * width + width + f);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 packed;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float g0 = __low2float(gp[k]), g1 = __high2float(gp[k]);
        q[k] = __floats2bfloat162_rn(g0 / (1.f + expf(-g0)) * __low2float(up[k]),
                                     g1 / (1.f + expf(-g1)) * __high2float(up[k]));
    }
    *reinterpret_cast<uint4*>(out + t * width + f) = packed;
}

MLXONE_API int mlxone_swiglu(const void* gate_up, void* out, int rows, int width, int dtype,
                             cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && width > 0, "swiglu: bad sizes");
    const long long total = (long long)rows * width;
    const int blocks = ceil_div_host(total, 256);
    if (dtype == MLXONE_BF16 && width % 8 == 0 && (reinterpret_cast<uintptr_t>(gate_up) & 15) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 15) == 0)
        launch_kernel(swiglu_wide_kernel, dim3(ceil_div_host(total / 8, 256)), dim3(256), 0, stream,
                      true, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, width, total / 8);
    else if (dtype == MLXONE_BF16)
        launch_kernel(swiglu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true,
                      (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, width, total);
    else
        launch_kernel(swiglu_kernel<float>, dim3(blocks), dim3(256), 0, stream, true,
                      (const float*)gate_up, (float*)out, width, total);
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
