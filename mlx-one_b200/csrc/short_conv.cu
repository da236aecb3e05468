// Gated short convolution over a ragged batch, with per-request state in slots.
//
// bcx[t, 0:H] = B, bcx[t, H:2H] = C, bcx[t, 2H:3H] = x.  g = round(B * x).
// y[t, d] = bias[d] + sum_k kernel[d, k] * g_at(position(t) - (taps-1) + k), where g_at reads
// this step's rows for positions inside the request's portion, the request's state for the
// taps-1 positions before it, and zero before position 0.  out[t, d] = C * y.
// State row s of a request holds g at position history - (taps-1) + s.
//
// g is rounded to the storage type before it is used, so that a value taken from this
// step's rows equals the value that a later step reads from the state.
#include "common.cuh"

namespace {

template <typename T>
__global__ void short_conv_kernel(const T* __restrict__ bcx, const float* __restrict__ kernel,
                                  const float* __restrict__ bias, const T* __restrict__ state,
                                  const int* __restrict__ slots,
                                  const int* __restrict__ token_request,
                                  const int* __restrict__ request_start,
                                  const int* __restrict__ history, T* __restrict__ out,
                                  int tokens, int hidden, int taps) {
    griddep_launch();
    griddep_wait();
    const int d = blockIdx.y * blockDim.x + threadIdx.x;
    const int t = blockIdx.x;
    if (d >= hidden) return;
    const int r = token_request[t];
    const int first = request_start[r];
    const int index = t - first;                      // place inside the portion
    const int position = history[r] + index;
    const size_t row = (size_t)3 * hidden;
    float y = bias ? bias[d] : 0.f;
    for (int k = 0; k < taps; ++k) {
        const int back = taps - 1 - k;                // how many positions before t
        float g = 0.f;
        if (index - back >= 0) {
            const T* src = bcx + (size_t)(t - back) * row;
            g = round_to<T>(to_float<T>(src[d]) * to_float<T>(src[2 * hidden + d]));
        } else if (position - back >= 0) {
            const int s = taps - 1 + (index - back);  // state row, 0 .. taps-2
            g = to_float<T>(state[((size_t)slots[r] * (taps - 1) + s) * hidden + d]);
        }
        y = fmaf(kernel[(size_t)d * taps + k], g, y);
    }
    out[(size_t)t * hidden + d] = from_float<T>(to_float<T>(bcx[(size_t)t * row + hidden + d]) * y);
}

// The same for bfloat16 with hidden % 8 == 0: a thread takes 8 neighbouring channels of one token
// with 16-byte loads.
template <int TAPS>
__global__ void short_conv_wide_kernel(const __nv_bfloat16* __restrict__ bcx,
                                       const float* __restrict__ kernel,
                                       const float* __restrict__ bias,
                                       const __nv_bfloat16* __restrict__ state,
                                       const int* __restrict__ slots,
                                       const int* __restrict__ token_request,
                                       const int* __restrict__ request_start,
                                       const int* __restrict__ history,
                                       __nv_bfloat16* __restrict__ out, int tokens, int hidden) {
    using T = __nv_bfloat16;
    constexpr int taps = TAPS;
    griddep_launch();
    griddep_wait();
    const int groups = hidden / 8;
    const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (item >= (long long)tokens * groups) return;
    const int t = (int)(item / groups);
    const int d = (int)(item % groups) * 8;
    const int r = token_request[t];
    const int index = t - request_start[r];
    const int position = history[r] + index;
    const size_t row = (size_t)3 * hidden;
    auto unpack = [](const uint4& v, float (&f)[8]) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(p[i]); f[2 * i + 1] = __high2float(p[i]); }
    };
    float y[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) y[i] = bias ? bias[d + i] : 0.f;
    // this thread's 8 * taps kernel weights lie together in memory
    float weights[8 * TAPS];
    {
        const float4* src = reinterpret_cast<const float4*>(kernel + (size_t)d * taps);
#pragma unroll
        for (int j = 0; j < 2 * TAPS; ++j) {
            const float4 v = src[j];
            weights[4 * j] = v.x; weights[4 * j + 1] = v.y;
            weights[4 * j + 2] = v.z; weights[4 * j + 3] = v.w;
        }
    }
#pragma unroll
    for (int k = 0; k < TAPS; ++k) {
        const int back = taps - 1 - k;
        float g[8];
        if (index - back >= 0) {
            const T* src = bcx + (size_t)(t - back) * row;
            float b[8], x[8];
            unpack(*reinterpret_cast<const uint4*>(src + d), b);
            unpack(*reinterpret_cast<const uint4*>(src + 2 * hidden + d), x);
#pragma unroll
            for (int i = 0; i < 8; ++i) g[i] = round_to<T>(b[i] * x[i]);
        } else if (position - back >= 0) {
            const int s = taps - 1 + (index - back);
            unpack(*reinterpret_cast<const uint4*>(
                       state + ((size_t)slots[r] * (taps - 1) + s) * hidden + d), g);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) g[i] = 0.f;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) y[i] = fmaf(weights[i * taps + k], g[i], y[i]);
    }
    float c[8];
    unpack(*reinterpret_cast<const uint4*>(bcx + (size_t)t * row + hidden + d), c);
    uint4 packed;
    __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
    for (int i = 0; i < 4; ++i) q[i] = __floats2bfloat162_rn(c[2 * i] * y[2 * i], c[2 * i + 1] * y[2 * i + 1]);
    *reinterpret_cast<uint4*>(out + (size_t)t * hidden + d) = packed;
}

// Many tokens (prefill): a thread takes 8 neighbouring channels of RUN consecutive tokens. The
// rows of the run are loaded first (they do not wait for one another), and g of the taps - 1
// positions before a token stays in registers from token to token, so that a row is read once
// for the run and not once per tap. A request that begins inside the run starts afresh.
template <int TAPS, int RUN>
__global__ void __launch_bounds__(256)
short_conv_run_kernel(const __nv_bfloat16* __restrict__ bcx, const float* __restrict__ kernel,
                      const float* __restrict__ bias, const __nv_bfloat16* __restrict__ state,
                      const int* __restrict__ slots, const int* __restrict__ token_request,
                      const int* __restrict__ request_start, const int* __restrict__ history,
                      __nv_bfloat16* __restrict__ out, int tokens, int hidden) {
    using T = __nv_bfloat16;
    griddep_launch();
    griddep_wait();
    const int groups = hidden / 8;
    const long long item = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const int t0 = (int)(item / groups) * RUN;
    if (t0 >= tokens) return;
    const int d = (int)(item % groups) * 8;
    const size_t row = (size_t)3 * hidden;
    auto unpack = [](const uint4& v, float (&f)[8]) {
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) { f[2 * i] = __low2float(p[i]); f[2 * i + 1] = __high2float(p[i]); }
    };
    uint4 raw_b[RUN], raw_c[RUN], raw_x[RUN];
#pragma unroll
    for (int i = 0; i < RUN; ++i) {
        const int t = min(t0 + i, tokens - 1);
        const T* src = bcx + (size_t)t * row + d;
        raw_b[i] = *reinterpret_cast<const uint4*>(src);
        raw_c[i] = *reinterpret_cast<const uint4*>(src + hidden);
        raw_x[i] = *reinterpret_cast<const uint4*>(src + 2 * hidden);
    }
    // this thread's 8 * taps kernel weights lie together in memory
    float weights[8 * TAPS], offset[8];
    {
        const float4* src = reinterpret_cast<const float4*>(kernel + (size_t)d * TAPS);
#pragma unroll
        for (int j = 0; j < 2 * TAPS; ++j) {
            const float4 v = src[j];
            weights[4 * j] = v.x; weights[4 * j + 1] = v.y;
            weights[4 * j + 2] = v.z; weights[4 * j + 3] = v.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) offset[i] = bias ? bias[d + i] : 0.f;
    }
    float past[TAPS > 1 ? TAPS - 1 : 1][8];      // g of the positions before the token, oldest first
    int end = -1;                                 // where the current request's tokens end
#pragma unroll
    for (int i = 0; i < RUN; ++i) {
        const int t = t0 + i;
        if (t >= tokens) break;
        if (t >= end) {
            // the run's first token, or a request begins here: g of the positions before it
            // comes from this step's rows, from the request's state, or is zero
            const int r = token_request[t];
            const int first = request_start[r];
            end = request_start[r + 1];
            const int index = t - first, position = history[r] + index;
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) {
                const int back = TAPS - 1 - k;
                if (index - back >= 0) {
                    const T* src = bcx + (size_t)(t - back) * row + d;
                    float b[8], x[8];
                    unpack(*reinterpret_cast<const uint4*>(src), b);
                    unpack(*reinterpret_cast<const uint4*>(src + 2 * hidden), x);
#pragma unroll
                    for (int c = 0; c < 8; ++c) past[k][c] = round_to<T>(b[c] * x[c]);
                } else if (position - back >= 0) {
                    const int s = TAPS - 1 + (index - back);
                    unpack(*reinterpret_cast<const uint4*>(
                               state + ((size_t)slots[r] * (TAPS - 1) + s) * hidden + d), past[k]);
                } else {
#pragma unroll
                    for (int c = 0; c < 8; ++c) past[k][c] = 0.f;
                }
            }
        }
        float b[8], gate[8], x[8], y[8];
        unpack(raw_b[i], b);
        unpack(raw_c[i], gate);
        unpack(raw_x[i], x);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            const float g = round_to<T>(b[c] * x[c]);
            float sum = offset[c];
#pragma unroll
            for (int k = 0; k < TAPS - 1; ++k) sum = fmaf(weights[c * TAPS + k], past[k][c], sum);
            y[c] = fmaf(weights[c * TAPS + TAPS - 1], g, sum);
#pragma unroll
            for (int k = 0; k + 1 < TAPS - 1; ++k) past[k][c] = past[k + 1][c];
            if (TAPS > 1) past[TAPS - 2][c] = g;
        }
        uint4 packed;
        __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
        for (int c = 0; c < 4; ++c)
            q[c] = __floats2bfloat162_rn(gate[2 * c] * y[2 * c], gate[2 * c + 1] * y[2 * c + 1]);
        *reinterpret_cast<uint4*>(out + (size_t)t * hidden + d) = packed;
    }
}

// New state after the step: row s holds g at position (history + n) - (taps-1) + s.
template <typename T>
__global__ void short_conv_state_kernel(const T* __restrict__ bcx, T* __restrict__ state,
                                        const int* __restrict__ slots,
                                        const int* __restrict__ request_start,
                                        const int* __restrict__ history, int hidden, int taps) {
    griddep_launch();
    griddep_wait();
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (d >= hidden) return;
    const int first = request_start[r];
    const int n = request_start[r + 1] - first;
    if (n <= 0) return;
    const int before = history[r];
    T* rows = state + (size_t)slots[r] * (taps - 1) * hidden;
    constexpr int MAX_ROWS = 16;
    float kept[MAX_ROWS];
    for (int s = 0; s < taps - 1; ++s) {
        const int index = n - (taps - 1) + s;          // place inside the portion, may be < 0
        float g = 0.f;
        if (index >= 0) {
            const T* src = bcx + (size_t)(first + index) * 3 * hidden;
            g = round_to<T>(to_float<T>(src[d]) * to_float<T>(src[2 * hidden + d]));
        } else if (before + index >= 0) {
            g = to_float<T>(rows[(size_t)(taps - 1 + index) * hidden + d]);
        }
        kept[s] = g;
    }
    for (int s = 0; s < taps - 1; ++s) rows[(size_t)s * hidden + d] = from_float<T>(kept[s]);
}

// One token per request (decode): output and new state in one pass. A thread owns one channel
// of one request, so it reads the old state before it writes the new one.
template <typename T>
__global__ void short_conv_decode_kernel(const T* __restrict__ bcx, const float* __restrict__ kernel,
                                         const float* __restrict__ bias, T* __restrict__ state,
                                         const int* __restrict__ slots,
                                         const int* __restrict__ history, T* __restrict__ out,
                                         int hidden, int taps, int write_state) {
    griddep_launch();
    griddep_wait();
    const int d = blockIdx.x * blockDim.x + threadIdx.x;
    const int r = blockIdx.y;
    if (d >= hidden) return;
    const int position = history[r];
    const T* row = bcx + (size_t)r * 3 * hidden;
    T* rows = state + (size_t)slots[r] * (taps - 1) * hidden;
    constexpr int MAX_ROWS = 16;
    float kept[MAX_ROWS];
    float y = bias ? bias[d] : 0.f;
    for (int s = 0; s < taps - 1; ++s) {
        // state row s holds position - (taps-1) + s; zero before the sequence began
        const float g = position - (taps - 1) + s >= 0 ? to_float<T>(rows[(size_t)s * hidden + d]) : 0.f;
        kept[s] = g;
        y = fmaf(kernel[(size_t)d * taps + s], g, y);
    }
    const float g_now = round_to<T>(to_float<T>(row[d]) * to_float<T>(row[2 * hidden + d]));
    y = fmaf(kernel[(size_t)d * taps + taps - 1], g_now, y);
    out[(size_t)r * hidden + d] = from_float<T>(to_float<T>(row[hidden + d]) * y);
    if (write_state) {
        for (int s = 0; s + 1 < taps - 1; ++s) rows[(size_t)s * hidden + d] = from_float<T>(kept[s + 1]);
        if (taps > 1) rows[(size_t)(taps - 2) * hidden + d] = from_float<T>(g_now);
    }
}

}  // namespace

MLXONE_API int mlxone_short_conv_decode(const void* bcx, const float* kernel, const float* bias,
                                        void* state, const int* slots, const int* history,
                                        void* out, int requests, int hidden, int taps,
                                        int write_state, int dtype, cudaStream_t stream) {
    if (requests == 0) return 0;
    MLXONE_REQUIRE(requests > 0 && requests <= 65535 && hidden > 0, "short_conv_decode: bad sizes");
    MLXONE_REQUIRE(taps >= 1 && taps <= 17, "short_conv: kernel width %d is not in 1..17", taps);
    const int threads = 128;
    const dim3 grid(ceil_div_host(hidden, threads), requests);
    if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        launch_kernel(short_conv_decode_kernel<T>, grid, dim3(threads), 0, stream, true,
                      (const T*)bcx, kernel, bias, (T*)state, slots, history, (T*)out, hidden, taps,
                      write_state);
    } else {
        using T = float;
        launch_kernel(short_conv_decode_kernel<T>, grid, dim3(threads), 0, stream, true,
                      (const T*)bcx, kernel, bias, (T*)state, slots, history, (T*)out, hidden, taps,
                      write_state);
    }
    MLXONE_LAUNCH_CHECK("short_conv_decode");
    return 0;
}

MLXONE_API int mlxone_short_conv(const void* bcx, const float* kernel, const float* bias,
                                 void* state, const int* slots, const int* token_request,
                                 const int* request_start, const int* history, void* out,
                                 int tokens, int requests, int hidden, int taps, int write_state,
                                 int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && requests > 0 && hidden > 0, "short_conv: bad sizes");
    MLXONE_REQUIRE(taps >= 1 && taps <= 17, "short_conv: kernel width %d is not in 1..17", taps);
    const int threads = 128;
    const dim3 grid(tokens, ceil_div_host(hidden, threads));
    const dim3 state_grid(ceil_div_host(hidden, threads), requests);
    MLXONE_REQUIRE(requests <= 65535, "short_conv: at most 65535 requests a step");
    if (dtype == MLXONE_BF16) {
        using T = __nv_bfloat16;
        const bool wide = hidden % 8 == 0 && taps <= 4 &&
                          (reinterpret_cast<uintptr_t>(kernel) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(bcx) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(state) & 15) == 0 &&
                          (reinterpret_cast<uintptr_t>(out) & 15) == 0;
        if (wide && tokens >= 256) {
            constexpr int RUN = 4;
            const long long items = (long long)ceil_div_host(tokens, RUN) * (hidden / 8);
#define RUNS(TAPS)                                                                                 \
    launch_kernel(short_conv_run_kernel<TAPS, RUN>, dim3(ceil_div_host(items, 256)), dim3(256), 0, \
                  stream, true, (const T*)bcx, kernel, bias, (const T*)state, slots,              \
                  token_request, request_start, history, (T*)out, tokens, hidden)
            if (taps == 1) RUNS(1);
            else if (taps == 2) RUNS(2);
            else if (taps == 3) RUNS(3);
            else RUNS(4);
#undef RUNS
        } else if (wide) {
            const long long items = (long long)tokens * (hidden / 8);
#define WIDE(TAPS)                                                                              \
    launch_kernel(short_conv_wide_kernel<TAPS>, dim3(ceil_div_host(items, 256)), dim3(256), 0,  \
                  stream, true, (const T*)bcx, kernel, bias, (const T*)state, slots,            \
                  token_request, request_start, history, (T*)out, tokens, hidden)
            if (taps == 1) WIDE(1);
            else if (taps == 2) WIDE(2);
            else if (taps == 3) WIDE(3);
            else WIDE(4);
#undef WIDE
        } else
        launch_kernel(short_conv_kernel<T>, grid, dim3(threads), 0, stream, true, (const T*)bcx, kernel, bias, (const T*)state, slots, token_request, request_start,
            history, (T*)out, tokens, hidden, taps);
        MLXONE_LAUNCH_CHECK("short_conv");
        if (write_state && taps > 1) {
            launch_kernel(short_conv_state_kernel<T>, state_grid, dim3(threads), 0, stream, true, (const T*)bcx, (T*)state, slots, request_start, history, hidden, taps);
            MLXONE_LAUNCH_CHECK("short_conv_state");
        }
    } else {
        using T = float;
        launch_kernel(short_conv_kernel<T>, grid, dim3(threads), 0, stream, true, (const T*)bcx, kernel, bias, (const T*)state, slots, token_request, request_start,
            history, (T*)out, tokens, hidden, taps);
        MLXONE_LAUNCH_CHECK("short_conv");
        if (write_state && taps > 1) {
            launch_kernel(short_conv_state_kernel<T>, state_grid, dim3(threads), 0, stream, true, (const T*)bcx, (T*)state, slots, request_start, history, hidden, taps);
            MLXONE_LAUNCH_CHECK("short_conv_state");
        }
    }
    return 0;
}
