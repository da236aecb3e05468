// bfloat16 matrix product for many rows (prefill) on the fifth-generation tensor cores:
// out[M, N] = a[M, K] * w[N, K]^T with the accumulator in tensor memory.
//
// Persistent blocks, one per SM; each computes 128 x BN tiles of the output (BN = 128 or 256),
// one after the other, with two accumulators in tensor memory so that the epilogue of a tile
// runs under the products of the next. The warps have roles:
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor) of a 128 x 64 tile of `a` and
//            a BN x 64 tile of `w` per stage into shared memory (128-byte swizzle), through a
//            ring of stages guarded by mbarriers;
//   warp 1   allocates tensor memory and one thread issues tcgen05.mma (M = 128, N = BN,
//            K = 16, four per stage), releasing each stage with tcgen05.commit;
//   warps 2-5  the epilogue: each reads its quarter of the accumulator's 128 lanes with
//            tcgen05.ld, 32 columns at a time, and writes the result.
// Both operands are K-major, so no transposition is needed anywhere.
//
// Epilogues: store bfloat16 (+ bias); SwiGLU (the w tile is 128 gate rows followed by the 128
// matching up rows, the block writes silu(gate) * up); add into the 32-bit residual stream;
// store float32.
//
// Every wait on an mbarrier gives up after a bounded number of polls, raises the error flag
// and lets the block run to its end, where tensor memory is given back.
#include <cuda.h>

#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int WIDE_STAGES = 4;         // 128 x 256 tiles: 4 x 48 KB
constexpr int NARROW_STAGES = 6;       // 128 x 128 tiles: 6 x 32 KB
constexpr int THREADS = 192;           // producer warp, mma warp, four epilogue warps
constexpr int WAIT_LIMIT = 1 << 24;    // polls before a wait gives up
constexpr int ERROR_WAIT = 9;

enum : int { STORE_BF16 = 0, SWIGLU = 1, ADD_RESIDUAL = 2, STORE_F32 = 3 };

__device__ __forceinline__ uint32_t shared_address(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ------------------------------------------------------------------ mbarriers
__device__ __forceinline__ void barrier_init(uint32_t bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void barrier_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool barrier_test(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Waits for the phase with the given parity; false (and the error flag set) after WAIT_LIMIT polls.
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity, int* error_flag) {
    for (int i = 0; i < WAIT_LIMIT; ++i)
        if (barrier_test(bar, parity)) return true;
    atomicExch(error_flag, ERROR_WAIT);
    return false;
}

// ------------------------------------------------------------------ TMA
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

// ------------------------------------------------------------------ tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t dst_shared, int columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_shared),
                 "r"(columns));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
}
__device__ __forceinline__ void tmem_free(uint32_t address, int columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns));
}
__device__ __forceinline__ void fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Makes the barrier arrive once all tcgen05.mma issued so far by this thread have finished.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                         uint32_t idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// 32 consecutive 32-bit columns of this thread's lane of tensor memory.
__device__ __forceinline__ void tmem_load_32(uint32_t address, float (&v)[32]) {
    uint32_t r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(address));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory operand descriptor: K-major tile whose rows are 128 bytes (64 bf16), swizzled
// in atoms of 8 rows x 128 bytes; start address, stride between atoms (1024 bytes), version 1,
// swizzle mode 2 (128 bytes). The leading offset is not used by this layout.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t address) {
    uint64_t d = (uint64_t)((address & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor: float32 accumulator, bfloat16 operands, both K-major, N and M.
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

template <int BN, int EPILOGUE, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_w, const float* __restrict__ bias,
                    void* out, int ldo, int m, int n, int k, int up_offset, int tiles_m,
                    int total_tiles, int* __restrict__ error_flag) {
    constexpr int A_BYTES = BM * BK * 2, W_BYTES = BN * BK * 2;
    constexpr int OUT_COLUMNS = EPILOGUE == SWIGLU ? BN / 2 : BN;
    extern __shared__ unsigned char shared_raw[];
    // full[s], empty[s] per stage; ready[b], drained[b] per accumulator buffer
    __shared__ __align__(8) unsigned long long barriers[2 * STAGES + 4];
    __shared__ uint32_t tmem_base_slot;
    // operand tiles must start on 1024-byte boundaries (the swizzle works on address bits)
    const uint32_t tiles = (shared_address(shared_raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = (k + BK - 1) / BK;
    auto full = [&](int s) { return shared_address(&barriers[s]); };
    auto empty = [&](int s) { return shared_address(&barriers[STAGES + s]); };
    auto ready = [&](int b) { return shared_address(&barriers[2 * STAGES + b]); };
    auto drained = [&](int b) { return shared_address(&barriers[2 * STAGES + 2 + b]); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            barrier_init(full(s), 1);
            barrier_init(empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            barrier_init(ready(b), 1);
            barrier_init(drained(b), 4);               // the four epilogue warps
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(shared_address(&tmem_base_slot), 2 * BN);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    // Persistent: this block takes tiles blockIdx.x, + gridDim.x, ... Tiles that follow one
    // another in this order share their rows of w (the same columns of the output), so blocks
    // that run at the same time read the same w tile from L2.
    if (warp == 0) {
        if (lane == 0) {
            int step = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
                const int tile_m = (tile % tiles_m) * BM;
                const int tile_n = (tile / tiles_m) * OUT_COLUMNS;
                for (int kt = 0; kt < k_tiles; ++kt, ++step) {
                    const int s = step % STAGES;
                    ok = barrier_wait(empty(s), ((step / STAGES) & 1) ^ 1, error_flag);
                    if (!ok) break;
                    barrier_expect(full(s), A_BYTES + W_BYTES);
                    const uint32_t a_tile = tiles + s * (A_BYTES + W_BYTES);
                    tma_load_2d(a_tile, &map_a, kt * BK, tile_m, full(s));
                    tma_load_2d(a_tile + A_BYTES, &map_w, kt * BK, tile_n, full(s));
                    if (EPILOGUE == SWIGLU)
                        tma_load_2d(a_tile + A_BYTES + W_BYTES / 2, &map_w, kt * BK,
                                    up_offset + tile_n, full(s));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instruction_descriptor(BM, BN);
            int step = 0, round = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++round) {
                const int buffer = round & 1;
                // the epilogue must have read this buffer's previous tile
                ok = barrier_wait(drained(buffer), ((round >> 1) & 1) ^ 1, error_flag);
                if (!ok) break;
                fence_after_sync();
                const uint32_t accumulator = tmem_base + buffer * BN;
                for (int kt = 0; kt < k_tiles; ++kt, ++step) {
                    const int s = step % STAGES;
                    ok = barrier_wait(full(s), (step / STAGES) & 1, error_flag);
                    if (!ok) break;
                    fence_after_sync();
                    const uint32_t a_tile = tiles + s * (A_BYTES + W_BYTES);
                    const uint64_t a_desc = operand_descriptor(a_tile);
                    const uint64_t w_desc = operand_descriptor(a_tile + A_BYTES);
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk)   // 16 bf16 = 32 bytes = 2 address units
                        mma_bf16(accumulator, a_desc + 2 * kk, w_desc + 2 * kk, idesc,
                                 kt > 0 || kk > 0);
                    mma_commit(empty(s));                  // the stage is free once these finish
                }
                if (ok) mma_commit(ready(buffer));
            }
        }
    } else {
        // epilogue warps 2..5 read the lane quarters 2, 3, 0, 1 (a warp may only touch its own).
        // A thread gets 32 columns of one row from tensor memory and writes them itself.
        const int quarter = warp & 3;
        float* turn = reinterpret_cast<float*>(shared_raw + (tiles - shared_address(shared_raw)) +
                                               STAGES * (A_BYTES + W_BYTES)) + (warp - 2) * 32 * 33;
        const int limit = EPILOGUE == SWIGLU ? up_offset : n;
        // whether every row of the output starts on a 16-byte boundary
        const bool whole_rows =
            (EPILOGUE == STORE_BF16 || EPILOGUE == SWIGLU)
                ? (ldo % 8 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0)
                : (ldo % 4 == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0);
        int round = 0;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++round) {
            const int buffer = round & 1;
            const int tile_m = (tile % tiles_m) * BM;
            const int tile_n = (tile / tiles_m) * OUT_COLUMNS;
            if (!barrier_wait(ready(buffer), (round >> 1) & 1, error_flag)) break;
            fence_after_sync();
            const uint32_t accumulator = tmem_base + buffer * BN + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < OUT_COLUMNS; c0 += 32) {
                float value[32];
                tmem_load_32(accumulator + c0, value);
                if (EPILOGUE == SWIGLU) {
                    float up[32];
                    tmem_load_32(accumulator + BN / 2 + c0, up);
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        float gate = value[i], other = up[i];
                        if (bias != nullptr && tile_n + c0 + i < up_offset) {
                            gate += bias[tile_n + c0 + i];
                            other += bias[up_offset + tile_n + c0 + i];
                        }
                        // the result is rounded to bfloat16; the fast exponential is exact enough
                        value[i] = __fdividef(gate, 1.f + __expf(-gate)) * other;
                    }
                } else if (bias != nullptr) {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (tile_n + c0 + i < n) value[i] += bias[tile_n + c0 + i];
                }
                if (c0 + 32 >= OUT_COLUMNS) {
                    // the last piece has left tensor memory: the buffer may be overwritten
                    fence_before_sync();
                    __syncwarp();
                    if (lane == 0)
                        asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(drained(buffer))
                                     : "memory");
                }
                const int row = tile_m + quarter * 32 + lane;
                const int column0 = tile_n + c0;
                if (whole_rows && column0 + 32 <= limit) {
                    // This thread's 32 columns of its own row, 16 bytes at a time: the lanes
                    // touch 32 rows, but every access fills whole sectors and there are a
                    // quarter as many of them as with one value per access.
                    if (row < m) {
                        const size_t at = (size_t)row * ldo + column0;
                        if (EPILOGUE == STORE_BF16 || EPILOGUE == SWIGLU) {
                            uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(out) + at);
#pragma unroll
                            for (int piece = 0; piece < 4; ++piece) {
                                uint4 packed;
                                __nv_bfloat162* pairs = reinterpret_cast<__nv_bfloat162*>(&packed);
#pragma unroll
                                for (int i = 0; i < 4; ++i)
                                    pairs[i] = __floats2bfloat162_rn(value[piece * 8 + 2 * i],
                                                                     value[piece * 8 + 2 * i + 1]);
                                dst[piece] = packed;
                            }
                        } else if (EPILOGUE == ADD_RESIDUAL) {
                            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + at);
                            float4 old[8];
#pragma unroll
                            for (int piece = 0; piece < 8; ++piece) old[piece] = dst[piece];
#pragma unroll
                            for (int piece = 0; piece < 8; ++piece)
                                dst[piece] = make_float4(old[piece].x + value[piece * 4],
                                                         old[piece].y + value[piece * 4 + 1],
                                                         old[piece].z + value[piece * 4 + 2],
                                                         old[piece].w + value[piece * 4 + 3]);
                        } else {
                            float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + at);
#pragma unroll
                            for (int piece = 0; piece < 8; ++piece)
                                dst[piece] = make_float4(value[piece * 4], value[piece * 4 + 1],
                                                         value[piece * 4 + 2], value[piece * 4 + 3]);
                        }
                    }
                    continue;
                }
                // rows that 16-byte accesses cannot take, or the ragged last columns: the warp
                // turns its 32 x 32 piece around in shared memory and writes a row at a time
                __syncwarp();
#pragma unroll
                for (int i = 0; i < 32; ++i) turn[lane * 33 + i] = value[i];
                __syncwarp();
                const int column = tile_n + c0 + lane;
                const int row0 = tile_m + quarter * 32;
                const int rows = min(32, m - row0);
                if (column < limit && rows > 0) {
                    const size_t at = (size_t)row0 * ldo + column;
                    if (EPILOGUE == STORE_BF16 || EPILOGUE == SWIGLU) {
                        bf16* dst = reinterpret_cast<bf16*>(out) + at;
#pragma unroll 8
                        for (int r = 0; r < rows; ++r)
                            dst[(size_t)r * ldo] = __float2bfloat16_rn(turn[r * 33 + lane]);
                    } else if (EPILOGUE == ADD_RESIDUAL) {
                        float* dst = reinterpret_cast<float*>(out) + at;
                        // all loads first: they do not wait for one another
                        float old[32];
#pragma unroll
                        for (int r = 0; r < 32; ++r) old[r] = r < rows ? dst[(size_t)r * ldo] : 0.f;
#pragma unroll
                        for (int r = 0; r < 32; ++r)
                            if (r < rows) dst[(size_t)r * ldo] = old[r] + turn[r * 33 + lane];
                    } else {
                        float* dst = reinterpret_cast<float*>(out) + at;
#pragma unroll 8
                        for (int r = 0; r < rows; ++r) dst[(size_t)r * ldo] = turn[r * 33 + lane];
                    }
                }
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        fence_after_sync();
        if (*reinterpret_cast<volatile int*>(error_flag) == ERROR_WAIT) {
            // a wait gave up: leave time for copies that may still be landing in this block's
            // shared memory before the block ends
            for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        }
        tmem_free(tmem_base, 2 * BN);
    }
}

// ------------------------------------------------------------------ host side

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled g_encode = nullptr;
int g_tile_choice = 0;
int g_sm_count = 0;

bool find_encoder() {
    if (g_encode != nullptr) return true;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult status;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &status) !=
            cudaSuccess || status != cudaDriverEntryPointSuccess || fn == nullptr)
        return false;
    g_encode = reinterpret_cast<EncodeTiled>(fn);
    return true;
}

// A map of a row-major [rows, columns] bfloat16 matrix with boxes of `box_rows` x 64 elements.
bool make_map(CUtensorMap* map, const void* base, long long rows, long long columns, long long ld,
              int box_rows) {
    const cuuint64_t dims[2] = {(cuuint64_t)columns, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {BK, (cuuint32_t)box_rows};
    const cuuint32_t element_strides[2] = {1, 1};
    return g_encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides,
                    box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int BN, int EPILOGUE, int STAGES>
int launch(const void* a, int lda, const void* w, const float* bias, void* out, int ldo, int m,
           int n, int k, int up_offset, int* error_flag, cudaStream_t stream) {
    CUtensorMap map_a, map_w;
    const int w_box = EPILOGUE == SWIGLU ? BN / 2 : BN;
    if (!make_map(&map_a, a, m, k, lda, BM) || !make_map(&map_w, w, n, k, k, w_box)) {
        mlxone_set_error("gemm_tcgen05: cannot encode a tensor map");
        return 2;
    }
    const int out_columns = EPILOGUE == SWIGLU ? BN / 2 : BN;
    const int columns = EPILOGUE == SWIGLU ? up_offset : n;
    const int tiles_m = (m + BM - 1) / BM;
    const int total_tiles = tiles_m * ((columns + out_columns - 1) / out_columns);
    if (g_sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, device);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    const dim3 grid(total_tiles < g_sm_count ? total_tiles : g_sm_count);
    const size_t shared = (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 1024 + 4 * 32 * 33 * 4;
    auto kernel = gemm_tcgen05_kernel<BN, EPILOGUE, STAGES>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)shared);
    if (err != cudaSuccess) {
        mlxone_set_error("gemm_tcgen05: %s", cudaGetErrorString(err));
        return 2;
    }
    kernel<<<grid, THREADS, shared, stream>>>(map_a, map_w, bias, out, ldo, m, n, k, up_offset,
                                              tiles_m, total_tiles, error_flag);
    return 0;
}

}  // namespace

// Tile width for measurements: 0 = the rule, 1 = 128 x 128 tiles, 2 = 128 x 256 tiles.
MLXONE_API void mlxone_gemm_tcgen05_tiles(int choice) { g_tile_choice = choice; }

// 1 if this build and driver can run the tcgen05 product (the tensor-map encoder was found).
MLXONE_API int mlxone_gemm_tcgen05_available() { return find_encoder() ? 1 : 0; }

// epilogue as for mlxone_gemm_skinny. a: [m, k] with row stride lda; w: [n, k] dense.
MLXONE_API int mlxone_gemm_tcgen05(const void* a, int lda, const void* w, const float* bias,
                                   void* out, int ldo, int m, int n, int k, int epilogue,
                                   int* error_flag, cudaStream_t stream) {
    if (m == 0 || n == 0) return 0;
    MLXONE_REQUIRE(find_encoder(), "gemm_tcgen05: the driver has no cuTensorMapEncodeTiled");
    MLXONE_REQUIRE(m > 0 && n > 0 && k > 0 && k % 8 == 0 && lda % 8 == 0,
                   "gemm_tcgen05: K (%d) and the row stride of a (%d) must be multiples of 8", k, lda);
    MLXONE_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                   "gemm_tcgen05: operands must be 16-byte aligned");
    MLXONE_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_tcgen05: unknown epilogue %d", epilogue);
    MLXONE_REQUIRE(epilogue != SWIGLU || n % 2 == 0, "gemm_tcgen05: SwiGLU needs an even n");
    int code;
    // 128 x 256 tiles unless the output is narrower: a 128 x 128 product reads its operands
    // from shared memory twice as often per flop and is bound by that
    const bool wide = g_tile_choice == 0 ? n > 128 : g_tile_choice == 2;
    switch (epilogue) {
        case STORE_BF16:
            code = wide ? launch<256, STORE_BF16, WIDE_STAGES>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream)
                        : launch<128, STORE_BF16, NARROW_STAGES>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream);
            break;
        case SWIGLU:
            code = launch<256, SWIGLU, WIDE_STAGES>(a, lda, w, bias, out, ldo, m, n, k, n / 2, error_flag, stream);
            break;
        case ADD_RESIDUAL:
            code = wide ? launch<256, ADD_RESIDUAL, WIDE_STAGES>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream)
                        : launch<128, ADD_RESIDUAL, NARROW_STAGES>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream);
            break;
        default:
            code = wide ? launch<256, STORE_F32, WIDE_STAGES>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream)
                        : launch<128, STORE_F32, NARROW_STAGES>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream);
            break;
    }
    if (code != 0) return code;
    MLXONE_LAUNCH_CHECK("gemm_tcgen05");
    return 0;
}
