// bfloat16 matrix product for 33 to 128 rows (decode steps of many requests, short portions) on
// the fifth-generation tensor cores, with the operands swapped: out[M, N] = a[M, K] * w[N, K]^T is
// computed as its transpose, 128 rows of w being the 128-row operand of tcgen05.mma and the M
// rows of a (padded to 64 or 128) the other one. Such a product is bound by reading w once, so
// the work is cut for streaming: a block owns 128 rows of w (for SwiGLU 64 gate rows and the 64
// matching up rows) and a range of K; where w has too few rows to give every SM a block, K is
// split over the 2 to 8 blocks of a thread-block cluster, which add their partial sums through
// distributed shared memory in the order of their ranks (no scratch buffer, no atomics, the same
// sum whatever the timing).
//
// The warps of a block have roles:
//   warp 0   one thread issues TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of 128 x 64
//            tiles of w and Mpad x 64 tiles of a into a ring of stages; the first tiles of w are
//            requested before griddepcontrol.wait, so that weights stream while the kernel
//            before this one finishes;
//   warp 1   allocates tensor memory; one thread issues tcgen05.mma (M = 128, N = Mpad, K = 16);
//   warps 2-5  read the accumulator (lane = row of w, column = row of a) with tcgen05.ld and leave
//            it in shared memory as [row of a][row of w]; after a barrier over the cluster, block
//            r adds the partial sums of the rows r, r + S, ... of a from all blocks and writes
//            them (bias; SwiGLU; residual add; float32), 128 neighbouring outputs at a time.
//
// Every wait on an mbarrier gives up after a bounded number of polls and raises the error flag
// (code 9); a block that gave up still takes part in the cluster's barriers.
#include <cuda.h>

#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int ROWS = 128;              // rows of w per block
constexpr int BK = 64;                 // 64 bf16 = 128 bytes: one swizzle row
constexpr int THREADS = 192;
constexpr int WAIT_LIMIT = 1 << 24;
constexpr int ERROR_WAIT = 9;
constexpr int W_BYTES = ROWS * BK * 2;

enum : int { STORE_BF16 = 0, SWIGLU = 1, ADD_RESIDUAL = 2, STORE_F32 = 3 };

__device__ __forceinline__ uint32_t shared_address(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
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
__device__ __forceinline__ bool barrier_wait(uint32_t bar, uint32_t parity, int* error_flag) {
    for (int i = 0; i < WAIT_LIMIT; ++i)
        if (barrier_test(bar, parity)) return true;
    atomicExch(error_flag, ERROR_WAIT);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
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
__device__ __forceinline__ void cluster_barrier() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// K-major operand tile with rows of 128 bytes, swizzled in atoms of 8 rows x 128 bytes.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t address) {
    uint64_t d = (uint64_t)((address & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// MPAD: rows of a, padded (64 or 128). STAGES: ring depth.
template <int MPAD, int EPILOGUE, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_swapped_kernel(const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_a, const float* __restrict__ bias,
                    void* out, int ldo, int m, int n, int k, int up_offset, int splits,
                    int* __restrict__ error_flag) {
    constexpr int A_BYTES = MPAD * BK * 2;
    constexpr int STAGE_BYTES = W_BYTES + A_BYTES;
    constexpr int PARTIAL_BYTES = MPAD * ROWS * 4;       // [row of a][row of w] float
    static_assert(PARTIAL_BYTES <= STAGES * STAGE_BYTES, "the partial sums reuse the ring");
    extern __shared__ unsigned char shared_raw[];
    __shared__ __align__(8) unsigned long long barriers[2 * STAGES + 1];
    __shared__ uint32_t tmem_base_slot;
    const uint32_t tiles = (shared_address(shared_raw) + 1023u) & ~1023u;
    float* partial = reinterpret_cast<float*>(shared_raw + (tiles - shared_address(shared_raw)));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int split = blockIdx.x;                        // rank in the cluster
    const int tile = blockIdx.y;
    const int columns = EPILOGUE == SWIGLU ? up_offset : n;      // outputs
    const int tile_rows = EPILOGUE == SWIGLU ? ROWS / 2 : ROWS;  // outputs of a tile
    const int k_tiles = (k + BK - 1) / BK;
    const int kt_begin = (int)((long long)k_tiles * split / splits);
    const int kt_end = (int)((long long)k_tiles * (split + 1) / splits);
    const int mine = kt_end - kt_begin;
    // Blocks walk their K range from different starting points (and around): at any moment they
    // ask L2 for different tiles of a, not all for the same one. The order of a block's sum
    // depends on its place only, so results do not depend on timing.
    const int rotate = mine > 0 ? (tile * 5 + split * 3) % mine : 0;
    auto full = [&](int s) { return shared_address(&barriers[s]); };
    auto empty = [&](int s) { return shared_address(&barriers[STAGES + s]); };
    const uint32_t ready = shared_address(&barriers[2 * STAGES]);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            barrier_init(full(s), 1);
            barrier_init(empty(s), 1);
        }
        barrier_init(ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(shared_address(&tmem_base_slot), MPAD);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;
    griddep_launch();

    if (warp == 0) {
        if (lane == 0) {
            auto load_w = [&](int i) {
                const uint32_t at = tiles + (i % STAGES) * STAGE_BYTES;
                const int x = (kt_begin + (i + rotate) % mine) * BK;
                if (EPILOGUE == SWIGLU) {
                    tma_load_2d(at, &map_w, x, tile * tile_rows, full(i % STAGES));
                    tma_load_2d(at + W_BYTES / 2, &map_w, x, up_offset + tile * tile_rows,
                                full(i % STAGES));
                } else {
                    tma_load_2d(at, &map_w, x, tile * ROWS, full(i % STAGES));
                }
            };
            auto load_a = [&](int i) {
                tma_load_2d(tiles + (i % STAGES) * STAGE_BYTES + W_BYTES, &map_a,
                            (kt_begin + (i + rotate) % mine) * BK, 0, full(i % STAGES));
            };
            // the first stages' weights do not depend on the kernel before this one
            const int early = mine < STAGES ? mine : STAGES;
            for (int i = 0; i < early; ++i) {
                barrier_expect(full(i), STAGE_BYTES);
                load_w(i);
            }
            griddep_wait();            // a is what the kernel before this one wrote
            for (int i = 0; i < early; ++i) load_a(i);
            bool ok = true;
            for (int i = early; i < mine && ok; ++i) {
                const int s = i % STAGES;
                ok = barrier_wait(empty(s), ((i / STAGES) & 1) ^ 1, error_flag);
                if (!ok) break;
                barrier_expect(full(s), STAGE_BYTES);
                load_w(i);
                load_a(i);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instruction_descriptor(ROWS, MPAD);
            bool ok = true;
            for (int i = 0; i < mine && ok; ++i) {
                const int s = i % STAGES;
                ok = barrier_wait(full(s), (i / STAGES) & 1, error_flag);
                if (!ok) break;
                fence_after_sync();
                const uint32_t w_tile = tiles + s * STAGE_BYTES;
                const uint64_t w_desc = operand_descriptor(w_tile);
                const uint64_t a_desc = operand_descriptor(w_tile + W_BYTES);
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk)
                    mma_bf16(tmem_base, w_desc + 2 * kk, a_desc + 2 * kk, idesc, i > 0 || kk > 0);
                mma_commit(empty(s));
            }
            if (ok) mma_commit(ready);
        }
    } else {
        // warps 2..5 read the lane quarters 2, 3, 0, 1 (a warp may only touch its own)
        const int quarter = warp & 3;
        const int row = quarter * 32 + lane;                    // row of w within the tile
        griddep_wait();            // `out` may be the stream that the kernel before this one updated
        bool ok = mine == 0 || barrier_wait(ready, 0, error_flag);
        fence_after_sync();
        // all products have finished, so the ring is free: the partial sums go there
#pragma unroll 1
        for (int c0 = 0; c0 < MPAD; c0 += 32) {
            float value[32];
            if (ok && mine > 0) {
                tmem_load_32(tmem_base + ((uint32_t)(quarter * 32) << 16) + c0, value);
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) value[i] = 0.f;
            }
#pragma unroll
            for (int i = 0; i < 32; ++i) partial[(c0 + i) * ROWS + row] = value[i];
        }
    }
    // every block of the cluster has left its partial sums
    fence_before_sync();
    __syncthreads();
    cluster_barrier();
    if (warp >= 2) {
        // Block `split` finishes the rows split, split + splits, ... of a. A warp takes one such
        // row at a time: lane l adds outputs 4 l .. 4 l + 3 of the tile over the blocks of the
        // cluster, in the order of their ranks; the loads of two rows of a are in flight together.
        const int sub = warp - 2;
        const uint32_t own = shared_address(partial) + (uint32_t)lane * 16;
        uint32_t remote[8];
#pragma unroll
        for (int s = 0; s < 8; ++s)
            asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n"
                         : "=r"(remote[s]) : "r"(own), "r"(s < splits ? s : 0));
        const int count = m > split ? (m - split + splits - 1) / splits : 0;   // rows of a for this block
        for (int j0 = sub; j0 < count; j0 += 8) {
            float4 parts[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int token = split + splits * (j0 + 4 * u);
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < splits && j0 + 4 * u < count) {
                        if (s == split)          // this block's own sums: an ordinary load
                            parts[u][s] = *reinterpret_cast<const float4*>(
                                partial + (size_t)token * ROWS + 4 * lane);
                        else
                            asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                                         : "=f"(parts[u][s].x), "=f"(parts[u][s].y),
                                           "=f"(parts[u][s].z), "=f"(parts[u][s].w)
                                         : "r"(remote[s] + (uint32_t)(token * ROWS) * 4));
                    }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                if (j0 + 4 * u >= count) continue;
                const int token = split + splits * (j0 + 4 * u);
                float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int s = 0; s < 8; ++s)
                    if (s < splits) {
                        sum[0] += parts[u][s].x; sum[1] += parts[u][s].y;
                        sum[2] += parts[u][s].z; sum[3] += parts[u][s].w;
                    }
                float up[4];
                if (EPILOGUE == SWIGLU) {
                    // lanes 16..31 hold the up rows that match the gate rows of lanes 0..15
#pragma unroll
                    for (int i = 0; i < 4; ++i) up[i] = __shfl_down_sync(0xffffffffu, sum[i], 16);
                    if (lane >= 16) continue;
                }
                const int column = tile * tile_rows + 4 * lane;
                float result[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float value = sum[i];
                    if (bias != nullptr && column + i < columns) {
                        value += bias[column + i];
                        if (EPILOGUE == SWIGLU) up[i] += bias[up_offset + column + i];
                    }
                    result[i] = EPILOGUE == SWIGLU
                        ? __fdividef(value, 1.f + __expf(-value)) * up[i] : value;
                }
                const size_t at = (size_t)token * ldo + column;
                const bool whole = column + 4 <= columns && ldo % 4 == 0;
                if (EPILOGUE == STORE_BF16 || EPILOGUE == SWIGLU) {
                    bf16* dst = reinterpret_cast<bf16*>(out) + at;
                    if (whole && (reinterpret_cast<uintptr_t>(out) & 7) == 0) {
                        uint2 packed;
                        __nv_bfloat162 lo = __floats2bfloat162_rn(result[0], result[1]);
                        __nv_bfloat162 hi = __floats2bfloat162_rn(result[2], result[3]);
                        packed.x = *reinterpret_cast<uint32_t*>(&lo);
                        packed.y = *reinterpret_cast<uint32_t*>(&hi);
                        *reinterpret_cast<uint2*>(dst) = packed;
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (column + i < columns) dst[i] = __float2bfloat16_rn(result[i]);
                    }
                } else {
                    float* dst = reinterpret_cast<float*>(out) + at;
                    if (whole && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
                        float4 old = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (EPILOGUE == ADD_RESIDUAL) old = *reinterpret_cast<float4*>(dst);
                        *reinterpret_cast<float4*>(dst) = make_float4(
                            old.x + result[0], old.y + result[1], old.z + result[2], old.w + result[3]);
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (column + i < columns)
                                dst[i] = (EPILOGUE == ADD_RESIDUAL ? dst[i] : 0.f) + result[i];
                    }
                }
            }
        }
    }
    // no block may leave while another still reads its shared memory
    cluster_barrier();
    if (warp == 1) {
        fence_after_sync();
        if (*reinterpret_cast<volatile int*>(error_flag) == ERROR_WAIT) {
            // a wait gave up: leave time for copies that may still be landing in this block's
            // shared memory before the block ends
            for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        }
        tmem_free(tmem_base, MPAD);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled g_encode = nullptr;
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

template <int MPAD, int EPILOGUE>
int launch(const void* a, int lda, const void* w, const float* bias, void* out, int ldo, int m,
           int n, int k, int up_offset, int* error_flag, cudaStream_t stream) {
    constexpr int STAGES = MPAD == 64 ? 4 : 3;           // 4 x 24 KB, 3 x 32 KB: two blocks an SM
    constexpr int STAGE_BYTES = W_BYTES + MPAD * BK * 2;
    CUtensorMap map_w, map_a;
    const int w_box = EPILOGUE == SWIGLU ? ROWS / 2 : ROWS;
    if (!make_map(&map_w, w, n, k, k, w_box) || !make_map(&map_a, a, m, k, lda, MPAD)) {
        mlxone_set_error("gemm_tcgen05_swapped: cannot encode a tensor map");
        return 2;
    }
    if (g_sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, device);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    const int columns = EPILOGUE == SWIGLU ? up_offset : n;
    const int tile_rows = EPILOGUE == SWIGLU ? ROWS / 2 : ROWS;
    const int row_tiles = (columns + tile_rows - 1) / tile_rows;
    // K is split over a cluster where w has too few rows to give every SM a block: as many
    // blocks as SMs, at most 8 a cluster, at least two stages of K each
    const int k_tiles = (k + BK - 1) / BK;
    int splits = g_sm_count / row_tiles;
    if (splits > 8) splits = 8;
    if (splits > k_tiles / 2) splits = k_tiles / 2;
    if (splits < 1) splits = 1;
    const size_t shared = (size_t)STAGES * STAGE_BYTES + 1024;
    auto kernel = gemm_swapped_kernel<MPAD, EPILOGUE, STAGES>;
    cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           (int)shared);
    if (err != cudaSuccess) {
        mlxone_set_error("gemm_tcgen05_swapped: %s", cudaGetErrorString(err));
        return 2;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(splits, row_tiles);
    config.blockDim = dim3(THREADS);
    config.dynamicSmemBytes = shared;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    attributes[0].id = cudaLaunchAttributeClusterDimension;
    attributes[0].val.clusterDim.x = splits;
    attributes[0].val.clusterDim.y = 1;
    attributes[0].val.clusterDim.z = 1;
    attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attributes[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attributes;
    config.numAttrs = mlxone_pdl_enabled() ? 2 : 1;
    err = cudaLaunchKernelEx(&config, kernel, map_w, map_a, bias, out, ldo, m, n, k, up_offset,
                             splits, error_flag);
    if (err != cudaSuccess) {
        mlxone_set_error("gemm_tcgen05_swapped: launch failed: %s", cudaGetErrorString(err));
        return 2;
    }
    return 0;
}

template <int MPAD>
int launch_epilogue(int epilogue, const void* a, int lda, const void* w, const float* bias,
                    void* out, int ldo, int m, int n, int k, int* error_flag, cudaStream_t stream) {
    switch (epilogue) {
        case STORE_BF16:
            return launch<MPAD, STORE_BF16>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream);
        case SWIGLU:
            return launch<MPAD, SWIGLU>(a, lda, w, bias, out, ldo, m, n, k, n / 2, error_flag, stream);
        case ADD_RESIDUAL:
            return launch<MPAD, ADD_RESIDUAL>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream);
        default:
            return launch<MPAD, STORE_F32>(a, lda, w, bias, out, ldo, m, n, k, 0, error_flag, stream);
    }
}

}  // namespace

// Most rows (of a) that the swapped product takes.
MLXONE_API int mlxone_gemm_tcgen05_swapped_max_rows() { return 128; }

// epilogue as for mlxone_gemm_skinny. a: [m, k] with row stride lda, m <= 128; w: [n, k] dense.
MLXONE_API int mlxone_gemm_tcgen05_swapped(const void* a, int lda, const void* w, const float* bias,
                                           void* out, int ldo, int m, int n, int k, int epilogue,
                                           int* error_flag, cudaStream_t stream) {
    if (m == 0 || n == 0) return 0;
    MLXONE_REQUIRE(find_encoder(), "gemm_tcgen05_swapped: the driver has no cuTensorMapEncodeTiled");
    MLXONE_REQUIRE(m > 0 && m <= 128, "gemm_tcgen05_swapped: %d rows, at most 128", m);
    MLXONE_REQUIRE(n > 0 && k > 0 && k % 8 == 0 && lda % 8 == 0,
                   "gemm_tcgen05_swapped: K (%d) and the row stride of a (%d) must be multiples of 8",
                   k, lda);
    MLXONE_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                   "gemm_tcgen05_swapped: operands must be 16-byte aligned");
    MLXONE_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_tcgen05_swapped: unknown epilogue %d", epilogue);
    MLXONE_REQUIRE(epilogue != SWIGLU || n % 2 == 0, "gemm_tcgen05_swapped: SwiGLU needs an even n");
    const int code = m <= 64
        ? launch_epilogue<64>(epilogue, a, lda, w, bias, out, ldo, m, n, k, error_flag, stream)
        : launch_epilogue<128>(epilogue, a, lda, w, bias, out, ldo, m, n, k, error_flag, stream);
    if (code != 0) return code;
    MLXONE_LAUNCH_CHECK("gemm_tcgen05_swapped");
    return 0;
}
