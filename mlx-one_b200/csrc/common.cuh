// Shared helpers of the sm_100a kernels: dtype conversion, reductions, error reporting.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>

#define MLXONE_API extern "C" __attribute__((visibility("default")))

// dtype codes of the C interface
enum : int { MLXONE_F32 = 0, MLXONE_BF16 = 1 };

// Error text of the last failed call of this thread (see mlxone_last_error).
void mlxone_set_error(const char* format, ...);

#define MLXONE_REQUIRE(cond, ...)          \
    do {                                   \
        if (!(cond)) {                     \
            mlxone_set_error(__VA_ARGS__); \
            return 1;                      \
        }                                  \
    } while (0)

#define MLXONE_LAUNCH_CHECK(name)                                                \
    do {                                                                         \
        cudaError_t err__ = cudaGetLastError();                                  \
        if (err__ != cudaSuccess) {                                              \
            mlxone_set_error("%s: launch failed: %s", name, cudaGetErrorString(err__)); \
            return 2;                                                            \
        }                                                                        \
    } while (0)

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) {
    return __bfloat162float(v);
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Rounds a 32-bit value to the storage type and back: what a value looks like after
// it has been stored, so that a value used at once equals the value read back later.
template <typename T>
__device__ __forceinline__ float round_to(float v) { return to_float<T>(from_float<T>(v)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1)
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds
// 33 floats of shared memory. The order of additions is fixed by the block size.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// ------------------------------------------------------------------ dependent launches
// A kernel launched with the programmatic-serialization attribute may start while its
// predecessor in the stream still runs. It must call griddep_wait() before it reads anything
// the predecessor wrote (what it does before that, such as fetching weights, overlaps with the
// predecessor's tail). griddep_launch() lets the successor start early in the same way. Both
// do nothing in a kernel launched the ordinary way.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Whether launches of the decode path ask for programmatic serialization (mlxone_set_pdl).
bool mlxone_pdl_enabled();

template <typename... KernelArgs, typename... Args>
static inline cudaError_t launch_kernel(void (*kernel)(KernelArgs...), dim3 grid, dim3 block,
                                        size_t shared, cudaStream_t stream, bool dependent,
                                        Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = dependent && mlxone_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
}

static inline int ceil_div_host(long long a, long long b) { return (int)((a + b - 1) / b); }
