// Prefill attention over the paged cache on the fifth-generation tensor cores, for bfloat16 and
// a head size of 64: both products of a tile (scores = Q K^T, out += P V) are tcgen05.mma with
// accumulators in tensor memory, keys and values arrive by TMA (cp.async.bulk.tensor, 128-byte
// swizzle) straight from the cache's pages, and only the softmax runs on ordinary threads.
//
// One block = up to 128 query rows that share a key head: 128 / group tokens of one request times
// the group's query heads (row = token * group + head), so that a key tile is fetched once for
// the whole group and short portions waste few rows. It walks the request's keys in tiles of 128.
// The warps have roles:
//   warps 0-7  softmax: two threads share query row r (lane r of tensor memory), one for keys
//              0-63 of a tile and output dimensions 0-31, one for the other halves. Per tile a
//              thread reads its scores with tcgen05.ld, the two agree on the maximum, it writes
//              exp2(score - max) as bfloat16 into shared memory in the operand layout of the
//              second product, and then adds the previous tile's P V (read from tensor memory)
//              into its 32 output registers, scaled as the running maximum moved;
//   warp 8     the TMA loads: the query tile once (a 3-D box: head size x group x tokens),
//              then per key tile lane b looks up page b and copies its K and V into a ring of
//              three stages;
//   warp 9     allocates tensor memory; one thread issues the products: scores of tile j + 1
//              are computed while the softmax warps work on tile j (two score buffers), P V
//              of tile j runs while they work on tile j + 1 (two buffers for it as well).
// V is used as it lies in the cache ([key, head size], head size contiguous): the second
// product takes it as an MN-major operand.
//
// Masking (causal, window, rows beyond the portion's end) is applied to the scores of tiles that
// need it. Keys that no query row may see contribute exp2(-inf) = 0 times their value, so the
// rows of a page that were never written must hold finite numbers (the cache is zeroed when it is
// made); stages of shared memory are zeroed before their first use for the same reason.
//
// Every wait on an mbarrier gives up after a bounded number of polls, raises the error flag
// (code 9) and lets the block run to its end, where tensor memory is given back.
#include <cuda.h>

#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int HD = 64;
constexpr int ROWS = 128;              // query rows per block
constexpr int KEYS = 128;              // keys per tile
constexpr int STAGES = 3;              // ring of key/value tiles
constexpr int THREADS = 320;            // eight softmax warps, the copy warp, the product warp
constexpr int COPY_WARP = 8, MMA_WARP = 9;
constexpr int WAIT_LIMIT = 1 << 24;
constexpr int ERROR_WAIT = 9;
constexpr int Q_BYTES = ROWS * HD * 2;
constexpr int K_BYTES = KEYS * HD * 2;
constexpr int STAGE_BYTES = 2 * K_BYTES;
constexpr int P_BYTES = ROWS * KEYS * 2;
constexpr int SHARED_BYTES = Q_BYTES + STAGES * STAGE_BYTES + 2 * P_BYTES + 1024;
constexpr int TMEM_COLUMNS = 512;      // scores 2 x 128, P V 2 x 64: 384, rounded to a power of two

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
__device__ __forceinline__ void barrier_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y,
                                            int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, "
        "{%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z)
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
__device__ __forceinline__ void fence_async_shared() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
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
// 64 columns: two loads in flight, one wait.
__device__ __forceinline__ void tmem_load_64(uint32_t address, float (&v)[64]) {
    uint32_t r[64];
#pragma unroll
    for (int h = 0; h < 2; ++h)
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
            "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
            "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
            : "=r"(r[h * 32 + 0]), "=r"(r[h * 32 + 1]), "=r"(r[h * 32 + 2]), "=r"(r[h * 32 + 3]),
              "=r"(r[h * 32 + 4]), "=r"(r[h * 32 + 5]), "=r"(r[h * 32 + 6]), "=r"(r[h * 32 + 7]),
              "=r"(r[h * 32 + 8]), "=r"(r[h * 32 + 9]), "=r"(r[h * 32 + 10]), "=r"(r[h * 32 + 11]),
              "=r"(r[h * 32 + 12]), "=r"(r[h * 32 + 13]), "=r"(r[h * 32 + 14]), "=r"(r[h * 32 + 15]),
              "=r"(r[h * 32 + 16]), "=r"(r[h * 32 + 17]), "=r"(r[h * 32 + 18]), "=r"(r[h * 32 + 19]),
              "=r"(r[h * 32 + 20]), "=r"(r[h * 32 + 21]), "=r"(r[h * 32 + 22]), "=r"(r[h * 32 + 23]),
              "=r"(r[h * 32 + 24]), "=r"(r[h * 32 + 25]), "=r"(r[h * 32 + 26]), "=r"(r[h * 32 + 27]),
              "=r"(r[h * 32 + 28]), "=r"(r[h * 32 + 29]), "=r"(r[h * 32 + 30]), "=r"(r[h * 32 + 31])
            : "r"(address + h * 32));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Shared-memory operand descriptor for tiles whose rows are 128 bytes, swizzled in atoms of 8
// rows x 128 bytes that follow one another every 1024 bytes: start address, stride between
// atoms, version 1, swizzle mode 2 (128 bytes). It serves K-major operands (rows = M or N, 64
// elements of K per row) and the MN-major V (rows = keys, 64 elements of N per row) alike; which
// of the two it is says the instruction descriptor.
__device__ __forceinline__ uint64_t operand_descriptor(uint32_t address) {
    uint64_t d = (uint64_t)((address & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// float32 accumulator, bfloat16 operands, A K-major; B K-major or MN-major; N and M.
__host__ __device__ constexpr uint32_t instruction_descriptor(int m, int n, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__global__ void __launch_bounds__(THREADS)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                         const __grid_constant__ CUtensorMap map_kv, long long value_rows,
                         const int* __restrict__ block_table, int table_width, int page_size,
                         int box_keys, const int* __restrict__ request_start,
                         const int* __restrict__ history, bf16* __restrict__ out, int requests,
                         int heads, int kv_heads, float scale_log2, int window,
                         int* __restrict__ error_flag) {
    extern __shared__ unsigned char shared_raw[];
    // q_full; kv_full[s], kv_empty[s]; s_ready[b], p_ready[b], o_ready[b]
    __shared__ __align__(8) unsigned long long barriers[1 + 2 * STAGES + 6];
    __shared__ uint32_t tmem_base_slot;
    __shared__ int found[2];
    __shared__ float maxima[2 * 2 * ROWS];          // [tile parity][half][row]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = heads / kv_heads;
    const int tile_tokens = ROWS / group;

    // which request and which tokens of it this block serves (the last tiles of a causal
    // prompt walk the most keys: they go first)
    if (threadIdx.x == 0) {
        int left = gridDim.x - 1 - blockIdx.x, request = -1, start = 0;
        for (int r = 0; r < requests; ++r) {
            const int tiles = (request_start[r + 1] - request_start[r] + tile_tokens - 1) / tile_tokens;
            if (left < tiles) { request = r; start = left * tile_tokens; break; }
            left -= tiles;
        }
        found[0] = request;
        found[1] = start;
    }
    __syncthreads();
    const int request = found[0];
    if (request < 0) return;
    const int token_start = found[1];                 // within the portion
    const int kv_head = blockIdx.y;
    const int first_token = request_start[request];
    const int count = request_start[request + 1] - first_token;
    const int tokens_here = min(tile_tokens, count - token_start);
    const int first_position = history[request] + token_start;
    const int last_position = first_position + tokens_here - 1;
    const int lowest = window > 0 ? max(first_position - window + 1, 0) : 0;
    const int tile_first = lowest / KEYS, tile_last = last_position / KEYS;
    const int tile_count = tile_last - tile_first + 1;

    const uint32_t base = (shared_address(shared_raw) + 1023u) & ~1023u;
    const uint32_t q_tile = base;
    const uint32_t stages = base + Q_BYTES;
    const uint32_t p_tiles = stages + STAGES * STAGE_BYTES;
    unsigned char* generic_base = shared_raw + (base - shared_address(shared_raw));
    auto q_full = [&]() { return shared_address(&barriers[0]); };
    auto kv_full = [&](int s) { return shared_address(&barriers[1 + s]); };
    auto kv_empty = [&](int s) { return shared_address(&barriers[1 + STAGES + s]); };
    auto s_ready = [&](int b) { return shared_address(&barriers[1 + 2 * STAGES + b]); };
    auto p_ready = [&](int b) { return shared_address(&barriers[1 + 2 * STAGES + 2 + b]); };
    auto o_ready = [&](int b) { return shared_address(&barriers[1 + 2 * STAGES + 4 + b]); };

    if (threadIdx.x == 0) {
        barrier_init(q_full(), 1);
        for (int s = 0; s < STAGES; ++s) {
            barrier_init(kv_full(s), 1);
            barrier_init(kv_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            barrier_init(s_ready(b), 1);
            barrier_init(p_ready(b), 8);               // the eight softmax warps
            barrier_init(o_ready(b), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // stages start as zeros: a page that is skipped must not show what shared memory held
    {
        uint4* stage_words = reinterpret_cast<uint4*>(generic_base + Q_BYTES);
        for (int i = threadIdx.x; i < STAGES * STAGE_BYTES / 16; i += THREADS)
            stage_words[i] = make_uint4(0u, 0u, 0u, 0u);
        fence_async_shared();
    }
    if (warp == MMA_WARP) tmem_alloc(shared_address(&tmem_base_slot), TMEM_COLUMNS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == COPY_WARP) {
        // Lane b brings box b of every key tile (one page, or a page's part): it looks up the
        // page and issues the two copies itself, so that neither the look-ups nor the copies of
        // a tile wait for one another. Lane 0 announces the bytes first.
        if (lane == 0) {
            barrier_expect(q_full(), Q_BYTES);
            tma_load_3d(q_tile, &map_q, 0, kv_head * group, first_token + token_start, q_full());
        }
        const int* table = block_table + (size_t)request * table_width;
        const int boxes = KEYS / box_keys;
        bool ok = true;
        for (int j = 0; j < tile_count && ok; ++j) {
            const int s = j % STAGES;
            // this box's rows in the cache, if some query row may see its keys
            long long row = -1;
            const int key = (tile_first + j) * KEYS + lane * box_keys;
            if (lane < boxes && key <= last_position && key + box_keys - 1 >= lowest) {
                const int block = key / page_size;
                const int page = block < table_width ? table[block] : -1;
                if (page >= 0)
                    row = ((long long)page * kv_heads + kv_head) * page_size + key % page_size;
            }
            const int live = __popc(__ballot_sync(0xffffffffu, row >= 0));
            if (lane == 0) {
                ok = barrier_wait(kv_empty(s), ((j / STAGES) & 1) ^ 1, error_flag);
                if (ok) barrier_expect(kv_full(s), (uint32_t)live * 2u * (uint32_t)box_keys * HD * 2u);
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (ok && row >= 0) {
                const uint32_t at = stages + s * STAGE_BYTES + (uint32_t)(lane * box_keys) * HD * 2;
                tma_load_2d(at, &map_kv, 0, (int)row, kv_full(s));
                tma_load_2d(at + K_BYTES, &map_kv, 0, (int)(row + value_rows), kv_full(s));
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc_scores = instruction_descriptor(ROWS, KEYS, false);
            constexpr uint32_t idesc_out = instruction_descriptor(ROWS, HD, true);
            bool ok = barrier_wait(q_full(), 0, error_flag);
            const uint64_t q_desc = operand_descriptor(q_tile);
            auto scores = [&](int j) {
                const int s = j % STAGES;
                if (!barrier_wait(kv_full(s), (j / STAGES) & 1, error_flag)) return false;
                fence_after_sync();
                const uint64_t k_desc = operand_descriptor(stages + s * STAGE_BYTES);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    mma_bf16(tmem_base + (j & 1) * KEYS, q_desc + 2 * kk, k_desc + 2 * kk,
                             idesc_scores, kk > 0);
                mma_commit(s_ready(j & 1));
                return true;
            };
            if (ok) ok = scores(0);
            for (int j = 0; j < tile_count && ok; ++j) {
                // the next tile's scores run while the softmax warps work on this one; their
                // buffer was read to its end before p_ready of tile j - 1 arrived
                if (j + 1 < tile_count) {
                    ok = scores(j + 1);
                    if (!ok) break;
                }
                ok = barrier_wait(p_ready(j & 1), (j >> 1) & 1, error_flag);
                if (!ok) break;
                fence_after_sync();
                const int s = j % STAGES;
                const uint32_t p_tile = p_tiles + (j & 1) * P_BYTES;
                const uint32_t v_tile = stages + s * STAGE_BYTES + K_BYTES;
#pragma unroll
                for (int kk = 0; kk < KEYS / 16; ++kk) {
                    // P: two blocks of 64 keys, 16 keys = 32 bytes within a block's rows;
                    // V: 16 keys = 16 rows of 128 bytes = two swizzle atoms
                    const uint64_t p_desc =
                        operand_descriptor(p_tile + (kk / 4) * (ROWS * 128)) + 2 * (kk % 4);
                    const uint64_t v_desc = operand_descriptor(v_tile + kk * 2048);
                    mma_bf16(tmem_base + 2 * KEYS + (j & 1) * HD, p_desc, v_desc, idesc_out, kk > 0);
                }
                mma_commit(kv_empty(s));                 // K and V of this tile are done with
                mma_commit(o_ready(j & 1));
            }
        }
    } else {
        // Softmax warps. Row r of the block is lane r of tensor memory, and a warp may only touch
        // lanes 32 (w % 4) .. + 31; warps w and w + 4 share their rows: the first takes keys
        // 0-63 of every tile and output dimensions 0-31, the second the other halves. They
        // agree on the row's maximum through shared memory once per tile; their sums are added
        // at the end.
        const int half = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const int token = row / group;
        const bool valid = token < tokens_here;
        const int position = first_position + token;
        const int limit_hi = valid ? position : -1;
        const int limit_lo = window > 0 ? max(position - window + 1, 0) : 0;
        // keys that every row of the block sees: from the last row's lower limit to the first
        // row's position; a block with rows beyond the portion's end always masks
        const bool whole = tokens_here == tile_tokens;
        const int open_lo = window > 0 ? max(last_position - window + 1, 0) : 0;
        const uint32_t lanes = (uint32_t)((warp & 3) * 32) << 16;
        // this thread's 128 bytes of P: block `half` of 64 keys, row `row`
        unsigned char* p_row = generic_base + Q_BYTES + STAGES * STAGE_BYTES + half * (ROWS * 128) +
                               (row >> 3) * 1024 + (row & 7) * 128;
        const int pair_barrier = 1 + (warp & 3);           // named barrier of the two warps
        float m = -INFINITY, l = 0.f, correction = 1.f;
        float o[HD / 2];
#pragma unroll
        for (int d = 0; d < HD / 2; ++d) o[d] = 0.f;
        bool ok = true;
        auto add_out = [&](int j) {
            // o = o * (how far the maximum moved when tile j was seen) + P_j V_j
            if (!barrier_wait(o_ready(j & 1), (j >> 1) & 1, error_flag)) return false;
            fence_after_sync();
            float part[32];
            tmem_load_32(tmem_base + lanes + 2 * KEYS + (j & 1) * HD + half * 32, part);
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = fmaf(o[i], correction, part[i]);
            return true;
        };
        for (int j = 0; j < tile_count && ok; ++j) {
            const int key0 = (tile_first + j) * KEYS + half * 64;
            ok = barrier_wait(s_ready(j & 1), (j >> 1) & 1, error_flag);
            if (!ok) break;
            fence_after_sync();
            float v[64];
            tmem_load_64(tmem_base + lanes + (j & 1) * KEYS + half * 64, v);
            const bool open = whole && (tile_first + j) * KEYS >= open_lo &&
                              (tile_first + j) * KEYS + KEYS - 1 <= first_position;
            if (!open) {
#pragma unroll
                for (int i = 0; i < 64; ++i)
                    if (!(key0 + i >= limit_lo && key0 + i <= limit_hi)) v[i] = -INFINITY;
            }
            float tops[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
            for (int i = 0; i < 64; ++i) tops[i & 3] = fmaxf(tops[i & 3], v[i]);
            const float mine = fmaxf(fmaxf(tops[0], tops[1]), fmaxf(tops[2], tops[3]));
            maxima[((j & 1) * 2 + half) * ROWS + row] = mine;
            asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
            const float top = fmaxf(mine, maxima[((j & 1) * 2 + (half ^ 1)) * ROWS + row]);
            const float new_m = fmaxf(m, top * scale_log2);
            const float previous = correction;
            const float moved = new_m == -INFINITY ? 1.f : fast_exp2(m - new_m);
            const float shift = new_m == -INFINITY ? 0.f : new_m;
            float sums[4] = {0.f, 0.f, 0.f, 0.f};
            unsigned char* p_tile_row = p_row + (j & 1) * P_BYTES;
#pragma unroll
            for (int chunk = 0; chunk < 8; ++chunk) {
                float p[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    p[i] = fast_exp2(fmaf(v[chunk * 8 + i], scale_log2, -shift));   // exp2(-inf) = 0
                    sums[i & 3] += p[i];
                }
                uint4 packed;
                packed.x = pack_bf16(p[0], p[1]);
                packed.y = pack_bf16(p[2], p[3]);
                packed.z = pack_bf16(p[4], p[5]);
                packed.w = pack_bf16(p[6], p[7]);
                *reinterpret_cast<uint4*>(p_tile_row + ((chunk ^ (row & 7)) << 4)) = packed;
            }
            l = l * moved + (sums[0] + sums[1]) + (sums[2] + sums[3]);
            m = new_m;
            // P is written and the scores are read: tell the product warp
            fence_async_shared();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) barrier_arrive(p_ready(j & 1));
            // the previous tile's P V, scaled by how far the maximum had moved then
            correction = previous;
            if (j > 0) ok = add_out(j - 1);
            correction = moved;
        }
        if (ok && tile_count > 0) ok = add_out(tile_count - 1);
        // the row's sum: both halves used the same maxima, so their sums add
        maxima[half * ROWS + row] = l;
        asm volatile("bar.sync %0, 64;" ::"r"(pair_barrier) : "memory");
        l += maxima[(half ^ 1) * ROWS + row];
        if (ok && valid) {
            const float inv = l > 0.f ? 1.f / l : 0.f;
            const int head = kv_head * group + row % group;
            bf16* dst = out + ((size_t)(first_token + token_start + token) * heads + head) * HD +
                        half * 32;
#pragma unroll
            for (int piece = 0; piece < 4; ++piece) {
                uint4 packed;
                packed.x = pack_bf16(o[piece * 8 + 0] * inv, o[piece * 8 + 1] * inv);
                packed.y = pack_bf16(o[piece * 8 + 2] * inv, o[piece * 8 + 3] * inv);
                packed.z = pack_bf16(o[piece * 8 + 4] * inv, o[piece * 8 + 5] * inv);
                packed.w = pack_bf16(o[piece * 8 + 6] * inv, o[piece * 8 + 7] * inv);
                *reinterpret_cast<uint4*>(dst + piece * 8) = packed;
            }
        }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == MMA_WARP) {
        fence_after_sync();
        if (*reinterpret_cast<volatile int*>(error_flag) == ERROR_WAIT) {
            // a wait gave up: leave time for copies that may still be landing in this block's
            // shared memory before the block ends
            for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        }
        tmem_free(tmem_base, TMEM_COLUMNS);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiled g_encode = nullptr;

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

bool supported(int head_dim, int heads, int kv_heads, int page_size) {
    if (head_dim != HD || kv_heads <= 0 || heads % kv_heads != 0) return false;
    const int group = heads / kv_heads;
    if (group > ROWS || ROWS % group != 0) return false;
    if (page_size < 8 || page_size % 8 != 0) return false;
    return page_size <= KEYS ? KEYS % page_size == 0 : page_size % KEYS == 0;
}

}  // namespace

// 1 if the tcgen05 prefill kernel takes this geometry (bfloat16 is implied) and the driver has
// the tensor-map encoder.
MLXONE_API int mlxone_attention_tcgen05_supports(int head_dim, int heads, int kv_heads,
                                                 int page_size) {
    return supported(head_dim, heads, kv_heads, page_size) && find_encoder() ? 1 : 0;
}

// q: [tokens, heads, 64] bfloat16; kv: [2, pages, kv_heads, page_size, 64]; out: [tokens, heads * 64].
MLXONE_API int mlxone_attention_prefill_tcgen05(const void* q, const void* kv, const int* block_table,
                                                int table_width, int page_size, int pages,
                                                const int* request_start, const int* history,
                                                void* out, int tokens, int requests, int heads,
                                                int kv_heads, int head_dim, float scale, int window,
                                                int* error_flag, cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && requests > 0, "attention_prefill_tcgen05: bad sizes");
    MLXONE_REQUIRE(supported(head_dim, heads, kv_heads, page_size),
                   "attention_prefill_tcgen05: head size %d, %d heads over %d key heads and pages of "
                   "%d keys are not supported", head_dim, heads, kv_heads, page_size);
    MLXONE_REQUIRE(find_encoder(), "attention_prefill_tcgen05: the driver has no cuTensorMapEncodeTiled");
    MLXONE_REQUIRE((reinterpret_cast<uintptr_t>(q) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(kv) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(out) & 15) == 0,
                   "attention_prefill_tcgen05: operands must be 16-byte aligned");
    MLXONE_REQUIRE(table_width > 0 && pages > 0, "attention_prefill_tcgen05: bad page geometry");
    const int group = heads / kv_heads;
    const int tile_tokens = ROWS / group;
    const int box_keys = page_size < KEYS ? page_size : KEYS;
    const long long value_rows = (long long)pages * kv_heads * page_size;
    MLXONE_REQUIRE(2 * value_rows < (1LL << 31), "attention_prefill_tcgen05: the cache has too many rows");
    CUtensorMap map_q, map_kv;
    {
        const cuuint64_t dims[3] = {HD, (cuuint64_t)heads, (cuuint64_t)tokens};
        const cuuint64_t strides[2] = {HD * 2, (cuuint64_t)heads * HD * 2};
        const cuuint32_t box[3] = {HD, (cuuint32_t)group, (cuuint32_t)tile_tokens};
        const cuuint32_t element_strides[3] = {1, 1, 1};
        const CUresult r = g_encode(&map_q, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q),
                                    dims, strides, box, element_strides,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        MLXONE_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tcgen05: cannot encode the query map (%d)", (int)r);
    }
    {
        const cuuint64_t dims[2] = {HD, (cuuint64_t)(2 * value_rows)};
        const cuuint64_t strides[1] = {HD * 2};
        const cuuint32_t box[2] = {HD, (cuuint32_t)box_keys};
        const cuuint32_t element_strides[2] = {1, 1};
        const CUresult r = g_encode(&map_kv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(kv),
                                    dims, strides, box, element_strides,
                                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        MLXONE_REQUIRE(r == CUDA_SUCCESS, "attention_prefill_tcgen05: cannot encode the cache map (%d)", (int)r);
    }
    cudaError_t err = cudaFuncSetAttribute(attention_tcgen05_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SHARED_BYTES);
    if (err != cudaSuccess) {
        mlxone_set_error("attention_prefill_tcgen05: %s", cudaGetErrorString(err));
        return 2;
    }
    const dim3 grid((tokens + tile_tokens - 1) / tile_tokens + requests, kv_heads);
    attention_tcgen05_kernel<<<grid, THREADS, SHARED_BYTES, stream>>>(
        map_q, map_kv, value_rows, block_table, table_width, page_size, box_keys, request_start,
        history, static_cast<bf16*>(out), requests, heads, kv_heads, scale * 1.4426950408889634f,
        window, error_flag);
    MLXONE_LAUNCH_CHECK("attention_prefill_tcgen05");
    return 0;
}
