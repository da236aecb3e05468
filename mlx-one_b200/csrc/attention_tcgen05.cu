// Prefill attention over the paged cache on the fifth-generation tensor cores, for bfloat16 and
// a head size of 64: both products of a tile (scores = Q K^T, out += P V) are tcgen05.mma with
// accumulators in tensor memory, keys and values arrive by TMA (cp.async.bulk.tensor, 128-byte
// swizzle) straight from the cache's pages, and only the softmax runs on ordinary threads.
//
// One item of work = up to 128 query rows that share a key head: 128 / group tokens of one request
// times the group's query heads (row = token * group + head), so that a key tile is fetched once
// for the whole group and short portions waste few rows; the request's keys are walked in tiles
// of 128 or of 64 (two shapes of the kernel, see Shape below). Blocks are persistent, as many as
// the GPU holds at once: a block lists its items once and its rings of buffers run on from one
// item into the next, so that the first loads and products of an item overlap the end of the
// one before. The warps have roles:
//   softmax warps (4 x PARTS): PARTS threads share query row r (lane r of tensor memory), each
//              for its share of a tile's keys and of the output dimensions. Per tile a thread
//              reads its scores with tcgen05.ld, the row's threads agree on the maximum, and
//              it writes exp2(score - m) as bfloat16 into shared memory in the operand layout
//              of the second product. The output is summed over the item's tiles by the
//              product warp in tensor memory; m follows the row's running maximum only when
//              that has moved by more than 2^8, and only then do the row's threads rescale the
//              output in tensor memory (tcgen05.ld, multiply, tcgen05.st) before they hand P
//              over, so most tiles cost no pass over the output. At the item's end they read
//              the output once, divide by the row's sum and store it;
//   copy warp  the TMA loads: the query tile once (a 3-D box: head size x group x tokens),
//              then per key tile lane b looks up page b and copies its K and V into a ring of
//              three stages;
//   product warp  allocates tensor memory; one thread issues the products: scores of tile j + 1
//              are computed while the softmax warps work on tile j (two score buffers), P V
//              of tile j, added to the item's output, runs while they work on tile j + 1.
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
constexpr int STAGES = 3;              // ring of key/value tiles
// PARTS (a parameter of the kernel): threads that share a query row, each for its share of a
// tile's keys and of the output dimensions. One: a thread owns its row's scores of a tile and
// all of its output, and the softmax warps exchange nothing, which is the faster form when an SM
// has several items to overlap (8192 tokens: 603 against 556 TFLOP/s). Two: a tile's softmax
// takes half as long, which is what counts when a block has one item and nothing beside it, the
// portion of a prompt in a step of decodes (see the launch).
constexpr int WAIT_LIMIT = 1 << 24;
constexpr int ERROR_WAIT = 9;
constexpr int Q_BYTES = ROWS * HD * 2;

// Two shapes of the kernel. With 128 keys a tile a block fills an SM (tensor memory: scores
// 2 x 128 columns, output 64); with 64 keys a tile two blocks share an SM, and while one waits
// for a product or a barrier the other computes: faster when there are items for all of them,
// slower when there are not, since a block then walks its keys in more, smaller steps.
template <int KEYS_>
struct Shape {
    static constexpr int KEYS = KEYS_;
    static constexpr int BLOCKS_PER_SM = KEYS == 64 ? 2 : 1;
    static constexpr int Q_BUFFERS = KEYS == 64 ? 1 : 2;           // query tiles in shared memory
    static constexpr int K_BYTES = KEYS * HD * 2;
    static constexpr int STAGE_BYTES = 2 * K_BYTES;
    static constexpr int P_BYTES = ROWS * KEYS * 2;
    static constexpr int SHARED_BYTES = Q_BUFFERS * Q_BYTES + STAGES * STAGE_BYTES + 2 * P_BYTES + 1024;
    static constexpr int TMEM_COLUMNS = KEYS == 64 ? 256 : 512;    // scores 2 x KEYS, output 64 (a power of two is allocated)
};
constexpr int MAX_ITEMS = 128;         // (token tile, key head) pairs one block may be given

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
// N consecutive 32-bit columns (16, 32 or 64) of this thread's lane of tensor memory; all loads
// are in flight before the one wait.
__device__ __forceinline__ void tmem_issue_16(uint32_t address, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(address));
}
template <int N>
__device__ __forceinline__ void tmem_load(uint32_t address, float (&v)[N]) {
    static_assert(N % 16 == 0, "whole loads of 16 columns");
    uint32_t r[N];
#pragma unroll
    for (int c = 0; c < N / 16; ++c) tmem_issue_16(address + c * 16, r + c * 16);
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = __uint_as_float(r[i]);
}
// Writes 16 consecutive 32-bit columns of this thread's lane of tensor memory.
__device__ __forceinline__ void tmem_store_16(uint32_t address, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(address), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}
template <int N>
__device__ __forceinline__ void tmem_store(uint32_t address, const float (&v)[N]) {
    static_assert(N % 16 == 0, "whole stores of 16 columns");
    uint32_t r[N];
#pragma unroll
    for (int i = 0; i < N; ++i) r[i] = __float_as_uint(v[i]);
#pragma unroll
    for (int c = 0; c < N / 16; ++c) tmem_store_16(address + c * 16, r + c * 16);
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// Two 32-bit floats in one instruction (fma.rn.f32x2, add.rn.f32x2) and a maximum of three: the
// softmax warps issue about one instruction less per score for each of them, and their issue
// slots are what a tile's softmax costs beside its exponentials.
__device__ __forceinline__ unsigned long long pair_of(float lo, float hi) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void unpair(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_pair(unsigned long long a, unsigned long long b,
                                                       unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add_pair(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max_of_three(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
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

// What a block does for one (request, tokens, key head): filled in once, read by every role.
struct Item {
    int request;            // -1: nothing to do (the grid is sized by an upper bound)
    int kv_head;
    int q_token;            // first token of the tile among all tokens of the step
    int tokens_here;        // tokens of the tile that belong to the portion
    int first_position;     // position of the first token in its request
    int tile_first;         // first key tile (of this item's split)
    int tile_count;         // 0: a split without keys (it only reports that it saw none)
    int split;
};

template <int KEYS, int PARTS>
__global__ void __launch_bounds__((4 * PARTS + 2) * 32, Shape<KEYS>::BLOCKS_PER_SM)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q,
                         const __grid_constant__ CUtensorMap map_kv, long long value_rows,
                         const int* __restrict__ block_table, int table_width, int page_size,
                         int box_keys, const int* __restrict__ request_start,
                         const int* __restrict__ history, bf16* __restrict__ out, int requests,
                         int heads, int kv_heads, float scale_log2, int window, int token_tiles,
                         int splits, float* __restrict__ partial, int* __restrict__ error_flag) {
    using S = Shape<KEYS>;
    constexpr int COPY_WARP = 4 * PARTS, MMA_WARP = 4 * PARTS + 1;
    constexpr int THREADS = (4 * PARTS + 2) * 32;     // softmax warps, the copy warp, the product warp
    constexpr int Q_BUFFERS = S::Q_BUFFERS, K_BYTES = S::K_BYTES, STAGE_BYTES = S::STAGE_BYTES;
    constexpr int P_BYTES = S::P_BYTES, TMEM_COLUMNS = S::TMEM_COLUMNS;
    extern __shared__ unsigned char shared_raw[];
    // q_full[2], q_empty[2]; kv_full[s], kv_empty[s]; s_ready[b], p_ready[b], o_ready[b]
    __shared__ __align__(8) unsigned long long barriers[4 + 2 * STAGES + 6];
    __shared__ uint32_t tmem_base_slot;
    __shared__ Item items[MAX_ITEMS];
    __shared__ float maxima[2 * PARTS * ROWS];      // [tile parity][part][row]
    __shared__ float sums[PARTS * ROWS];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = heads / kv_heads;
    const int tile_tokens = ROWS / group;

    // This block's items among all (token tile, key head) pairs, the token tiles counted from
    // the end (the last tiles of a causal prompt walk the most keys). They are dealt out in
    // rounds of gridDim.x, every other round in reverse, so that the block with the heaviest
    // item of one round gets the lightest of the next and all blocks walk about as many keys.
    // (With `splits` > 1 an item is cut further, by key tiles: split s of an item walks its share
    // of the item's key tiles and leaves an unnormalised output with its maximum and sum in
    // `partial`, [token, head, split][HD + 2], which a merge kernel adds up. That is for launches
    // with fewer items than SMs, whose blocks would otherwise walk long rows of tiles alone.)
    const int all_items = token_tiles * kv_heads * splits;
    const int rounds = all_items / (int)gridDim.x, rest = all_items % (int)gridDim.x;
    const int last_place = (rounds & 1) ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    const int mine = rounds + (last_place < rest ? 1 : 0);
    if (mine == 0) return;
    for (int k = threadIdx.x; k < mine; k += THREADS) {
        const int index = k * gridDim.x + ((k & 1) ? gridDim.x - 1 - blockIdx.x : blockIdx.x);
        Item item;
        item.request = -1;
        item.split = index % splits;
        item.kv_head = (index / splits) % kv_heads;
        int left = index / splits / kv_heads;
        for (int r = 0; r < requests; ++r) {
            const int first = request_start[r], count = request_start[r + 1] - first;
            const int tiles = (count + tile_tokens - 1) / tile_tokens;
            if (left < tiles) {
                const int token_start = (tiles - 1 - left) * tile_tokens;
                item.request = r;
                item.q_token = first + token_start;
                item.tokens_here = min(tile_tokens, count - token_start);
                item.first_position = history[r] + token_start;
                const int last_position = item.first_position + item.tokens_here - 1;
                const int lowest = window > 0 ? max(item.first_position - window + 1, 0) : 0;
                item.tile_first = lowest / KEYS;
                item.tile_count = last_position / KEYS - item.tile_first + 1;
                if (splits > 1) {
                    const int share = (item.tile_count + splits - 1) / splits;
                    const int end = item.tile_first + item.tile_count;
                    item.tile_first += item.split * share;
                    item.tile_count = max(min(share, end - item.tile_first), 0);
                }
                break;
            }
            left -= tiles;
        }
        items[k] = item;
    }

    const uint32_t base = (shared_address(shared_raw) + 1023u) & ~1023u;
    const uint32_t q_tiles = base;
    const uint32_t stages = base + Q_BUFFERS * Q_BYTES;
    const uint32_t p_tiles = stages + STAGES * STAGE_BYTES;
    unsigned char* generic_base = shared_raw + (base - shared_address(shared_raw));
    auto q_full = [&](int b) { return shared_address(&barriers[b]); };
    auto q_empty = [&](int b) { return shared_address(&barriers[2 + b]); };
    auto kv_full = [&](int s) { return shared_address(&barriers[4 + s]); };
    auto kv_empty = [&](int s) { return shared_address(&barriers[4 + STAGES + s]); };
    auto s_ready = [&](int b) { return shared_address(&barriers[4 + 2 * STAGES + b]); };
    auto p_ready = [&](int b) { return shared_address(&barriers[4 + 2 * STAGES + 2 + b]); };
    auto o_ready = [&](int b) { return shared_address(&barriers[4 + 2 * STAGES + 4 + b]); };

    if (threadIdx.x == 0) {
        for (int b = 0; b < 2; ++b) {
            barrier_init(q_full(b), 1);
            barrier_init(q_empty(b), 1);
            barrier_init(s_ready(b), 1);
            barrier_init(p_ready(b), 4 * PARTS);       // the softmax warps
            barrier_init(o_ready(b), 1);
        }
        for (int s = 0; s < STAGES; ++s) {
            barrier_init(kv_full(s), 1);
            barrier_init(kv_empty(s), 1);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // query buffers and stages start as zeros: a page that is skipped, and the query rows beyond
    // a group that does not divide ROWS, must not show what shared memory held
    {
        uint4* words = reinterpret_cast<uint4*>(generic_base);
        for (int i = threadIdx.x; i < (Q_BUFFERS * Q_BYTES + STAGES * STAGE_BYTES) / 16; i += THREADS)
            words[i] = make_uint4(0u, 0u, 0u, 0u);
        fence_async_shared();
    }
    if (warp == MMA_WARP) tmem_alloc(shared_address(&tmem_base_slot), TMEM_COLUMNS);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    // Every role walks the same items and key tiles in the same order and counts them the same
    // way: `taken` items with work (it picks the query buffer), `t` key tiles (it picks the
    // stage, the score, P and P V buffers). The rings run on from one item into the next, so an
    // item's first loads and products overlap the end of the item before it.
    if (warp == COPY_WARP) {
        // Lane b brings box b of every key tile (one page, or a page's part): it looks up the
        // page and issues the two copies itself, so that neither the look-ups nor the copies of
        // a tile wait for one another. Lane 0 announces the bytes first.
        const int boxes = KEYS / box_keys;
        bool ok = true;
        int taken = 0, t = 0;
        for (int n = 0; n < mine && ok; ++n) {
            const Item item = items[n];
            if (item.request < 0 || item.tile_count <= 0) continue;
            if (lane == 0) {
                const int qb = taken % Q_BUFFERS;
                ok = barrier_wait(q_empty(qb), ((taken / Q_BUFFERS) & 1) ^ 1, error_flag);
                if (ok) {
                    // the box holds tile_tokens x group rows: all ROWS, or a few less when the
                    // group does not divide them (those rows stay zero and are never stored)
                    barrier_expect(q_full(qb), (uint32_t)(tile_tokens * group) * HD * 2u);
                    tma_load_3d(q_tiles + qb * Q_BYTES, &map_q, 0, item.kv_head * group,
                                item.q_token, q_full(qb));
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            ++taken;
            const int* table = block_table + (size_t)item.request * table_width;
            const int last_position = item.first_position + item.tokens_here - 1;
            const int lowest = window > 0 ? max(item.first_position - window + 1, 0) : 0;
            // this lane's box of the item's tile j: its rows in the cache, if some query row
            // may see its keys
            auto box_row = [&](int j) {
                long long row = -1;
                const int key = (item.tile_first + j) * KEYS + lane * box_keys;
                if (lane < boxes && key <= last_position && key + box_keys - 1 >= lowest) {
                    const int block = key / page_size;
                    const int page = block < table_width ? table[block] : -1;
                    if (page >= 0)
                        row = ((long long)page * kv_heads + item.kv_head) * page_size + key % page_size;
                }
                return row;
            };
            for (int j = 0; j < item.tile_count && ok; ++j, ++t) {
                const int s = t % STAGES;
                const long long row = box_row(j);
                const int live = __popc(__ballot_sync(0xffffffffu, row >= 0));
                if (lane == 0) {
                    ok = barrier_wait(kv_empty(s), ((t / STAGES) & 1) ^ 1, error_flag);
                    if (ok) barrier_expect(kv_full(s), (uint32_t)live * 2u * (uint32_t)box_keys * HD * 2u);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (ok && row >= 0) {
                    const uint32_t at = stages + s * STAGE_BYTES + (uint32_t)(lane * box_keys) * HD * 2;
                    tma_load_2d(at, &map_kv, 0, (int)row, kv_full(s));
                    tma_load_2d(at + K_BYTES, &map_kv, 0, (int)(row + value_rows), kv_full(s));
                }
            }
        }
    } else if (warp == MMA_WARP) {
        if (lane == 0) {
            constexpr uint32_t idesc_scores = instruction_descriptor(ROWS, KEYS, false);
            constexpr uint32_t idesc_out = instruction_descriptor(ROWS, HD, true);
            // a place in the walk: item n, its tile j; `taken` and `t` as above
            struct Place { int n, j, taken, t; };
            auto settle = [&](Place& place) {          // skips items without work
                while (place.n < mine &&
                       (items[place.n].request < 0 || items[place.n].tile_count <= 0)) ++place.n;
            };
            auto step = [&](Place place) {
                if (place.j + 1 < items[place.n].tile_count) {
                    ++place.j;
                } else {
                    ++place.n; place.j = 0; ++place.taken;
                    settle(place);
                }
                ++place.t;
                return place;
            };
            // scores of the tile at `place` into score buffer t & 1
            auto scores = [&](const Place& place) {
                const int tile_count = items[place.n].tile_count;
                const int qb = place.taken % Q_BUFFERS, s = place.t % STAGES;
                if (place.j == 0 &&
                    !barrier_wait(q_full(qb), (place.taken / Q_BUFFERS) & 1, error_flag)) return false;
                if (!barrier_wait(kv_full(s), (place.t / STAGES) & 1, error_flag)) return false;
                fence_after_sync();
                const uint64_t q_desc = operand_descriptor(q_tiles + qb * Q_BYTES);
                const uint64_t k_desc = operand_descriptor(stages + s * STAGE_BYTES);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    mma_bf16(tmem_base + (place.t & 1) * KEYS, q_desc + 2 * kk, k_desc + 2 * kk,
                             idesc_scores, kk > 0);
                mma_commit(s_ready(place.t & 1));
                if (place.j == tile_count - 1) mma_commit(q_empty(qb));   // the query tile is done with
                return true;
            };
            Place now{0, 0, 0, 0};
            settle(now);
            bool ok = now.n < mine ? scores(now) : false;
            while (ok && now.n < mine) {
                // the next tile's scores run while the softmax warps work on this one; their
                // buffer was read to its end before p_ready of the tile before this one arrived
                const Place next = step(now);
                if (next.n < mine) {
                    ok = scores(next);
                    if (!ok) break;
                }
                ok = barrier_wait(p_ready(now.t & 1), (now.t >> 1) & 1, error_flag);
                if (!ok) break;
                fence_after_sync();
                const int s = now.t % STAGES;
                const uint32_t p_tile = p_tiles + (now.t & 1) * P_BYTES;
                const uint32_t v_tile = stages + s * STAGE_BYTES + K_BYTES;
#pragma unroll
                for (int kk = 0; kk < KEYS / 16; ++kk) {
                    // P: two blocks of 64 keys, 16 keys = 32 bytes within a block's rows;
                    // V: 16 keys = 16 rows of 128 bytes = two swizzle atoms
                    const uint64_t p_desc =
                        operand_descriptor(p_tile + (kk / 4) * (ROWS * 128)) + 2 * (kk % 4);
                    const uint64_t v_desc = operand_descriptor(v_tile + kk * 2048);
                    mma_bf16(tmem_base + 2 * KEYS, p_desc, v_desc, idesc_out, kk > 0 || now.j > 0);
                }
                mma_commit(kv_empty(s));                 // K and V of this tile are done with
                mma_commit(o_ready(now.t & 1));
                now = next;
            }
        }
    } else {
        // Softmax warps. Row r of the block is lane r of tensor memory, and a warp may only touch
        // lanes 32 (w % 4) .. + 31; the PARTS warps w, w + 4, ... share their rows: each takes
        // KEYS / PARTS keys of every tile and HD / PARTS output dimensions. They agree on the
        // row's maximum through shared memory once per tile; their sums are added at the end.
        constexpr int MY_KEYS = KEYS / PARTS, MY_DIMS = HD / PARTS;
        constexpr int PIECES = MY_KEYS / 8;
        const int part = warp >> 2;
        const int row = (warp & 3) * 32 + lane;
        const int token = row / group;
        const uint32_t lanes = (uint32_t)((warp & 3) * 32) << 16;
        // this thread's row of P in the first block of 64 keys; its keys may span several blocks
        unsigned char* p_row = generic_base + Q_BUFFERS * Q_BYTES + STAGES * STAGE_BYTES +
                               (row >> 3) * 1024 + (row & 7) * 128;
        const int row_barrier = 1 + (warp & 3);            // named barrier of the row's warps
        bool ok = true;
        int t = 0;
        for (int n = 0; n < mine && ok; ++n) {
            const Item item = items[n];
            if (item.request < 0) continue;
            const bool valid = token < item.tokens_here;
            // where this row's part of the split's result goes (splits > 1)
            float* split_row = partial == nullptr ? nullptr
                : partial + (((size_t)(item.q_token + token) * heads + item.kv_head * group +
                              row % group) * splits + item.split) * (HD + 2);
            if (item.tile_count <= 0) {
                // a split without keys: nothing was loaded or multiplied, the row reports zeros
                // with a maximum of minus infinity, which the merge gives no weight
                if (valid && split_row != nullptr) {
#pragma unroll
                    for (int d = 0; d < MY_DIMS; ++d) split_row[part * MY_DIMS + d] = 0.f;
                    if (part == 0) { split_row[HD] = -INFINITY; split_row[HD + 1] = 0.f; }
                }
                continue;
            }
            const int position = item.first_position + token;
            const int last_position = item.first_position + item.tokens_here - 1;
            const int limit_hi = valid ? position : -1;
            const int limit_lo = window > 0 ? max(position - window + 1, 0) : 0;
            // keys that every row of the block sees: from the last row's lower limit to the
            // first row's position; a block with rows beyond the portion's end always masks
            const bool whole = item.tokens_here == tile_tokens;
            const int open_lo = window > 0 ? max(last_position - window + 1, 0) : 0;
            // m: the maximum that the exponentials are taken against. It follows the running
            // maximum only when that has moved by more than LAZY (in powers of two), so that the
            // output so far, which the product warp accumulates in tensor memory over the item's
            // tiles, has to be rescaled there only then: P grows to 2^LAZY at most meanwhile.
            constexpr float LAZY = 8.f;
            float m = -INFINITY, l = 0.f;
            const uint32_t my_out = tmem_base + lanes + 2 * KEYS + part * MY_DIMS;
            auto out_ready = [&](int tile) {
                if (!barrier_wait(o_ready(tile & 1), (tile >> 1) & 1, error_flag)) return false;
                fence_after_sync();
                return true;
            };
            for (int j = 0; j < item.tile_count && ok; ++j, ++t) {
                const int tile_key = (item.tile_first + j) * KEYS;
                const int key0 = tile_key + part * MY_KEYS;
                ok = barrier_wait(s_ready(t & 1), (t >> 1) & 1, error_flag);
                if (!ok) break;
                fence_after_sync();
                float v[MY_KEYS];
                tmem_load<MY_KEYS>(tmem_base + lanes + (t & 1) * KEYS + part * MY_KEYS, v);
                const bool open = whole && tile_key >= open_lo &&
                                  tile_key + KEYS - 1 <= item.first_position;
                if (!open) {
#pragma unroll
                    for (int i = 0; i < MY_KEYS; ++i)
                        if (!(key0 + i >= limit_lo && key0 + i <= limit_hi)) v[i] = -INFINITY;
                }
                float tops[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < MY_KEYS; i += 2)
                    tops[(i >> 1) & 3] = max_of_three(tops[(i >> 1) & 3], v[i], v[i + 1]);
                float top = fmaxf(max_of_three(tops[0], tops[1], tops[2]), tops[3]);
                if (PARTS > 1) {
                    maxima[((t & 1) * PARTS + part) * ROWS + row] = top;
                    asm volatile("bar.sync %0, %1;" ::"r"(row_barrier), "n"(PARTS * 32) : "memory");
#pragma unroll
                    for (int other = 0; other < PARTS; ++other)
                        top = fmaxf(top, maxima[((t & 1) * PARTS + other) * ROWS + row]);
                }
                const float running = fmaxf(m, top * scale_log2);
                // both threads of a row see the same maxima and take the same decision
                const bool follow = running > m + LAZY || (m == -INFINITY && running > m);
                const float moved = !follow ? 1.f : m == -INFINITY ? 0.f : fast_exp2(m - running);
                // what the product warp has summed so far is against the old maximum: bring it
                // to the new one before the product of this tile is added (a row that has seen
                // no key yet has summed zeros). All lanes of a warp go together.
                const bool rescale = follow && m != -INFINITY && j > 0;
                if (__any_sync(0xffffffffu, rescale)) {
                    ok = out_ready(t - 1);
                    if (!ok) break;
                    float sofar[MY_DIMS];
                    tmem_load<MY_DIMS>(my_out, sofar);
                    const float factor = rescale ? moved : 1.f;
#pragma unroll
                    for (int i = 0; i < MY_DIMS; ++i) sofar[i] *= factor;
                    tmem_store<MY_DIMS>(my_out, sofar);
                }
                if (follow) m = running;
                const float shift = m == -INFINITY ? 0.f : m;
                unsigned long long partial[2] = {pair_of(0.f, 0.f), pair_of(0.f, 0.f)};
                const unsigned long long scale_pair = pair_of(scale_log2, scale_log2);
                const unsigned long long shift_pair = pair_of(-shift, -shift);
                unsigned char* p_tile_row = p_row + (t & 1) * P_BYTES;
#pragma unroll
                for (int piece = 0; piece < PIECES; ++piece) {
                    float p[8];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        float lo, hi;
                        unpair(fma_pair(pair_of(v[piece * 8 + i], v[piece * 8 + i + 1]), scale_pair,
                                        shift_pair), lo, hi);
                        p[i] = fast_exp2(lo);                     // exp2(-inf) = 0
                        p[i + 1] = fast_exp2(hi);
                        partial[(i >> 1) & 1] = add_pair(partial[(i >> 1) & 1], pair_of(p[i], p[i + 1]));
                    }
                    uint4 packed;
                    packed.x = pack_bf16(p[0], p[1]);
                    packed.y = pack_bf16(p[2], p[3]);
                    packed.z = pack_bf16(p[4], p[5]);
                    packed.w = pack_bf16(p[6], p[7]);
                    // 16-byte piece `at` of the row: block at / 8 of 64 keys, swizzled within it
                    const int at = (part * MY_KEYS) / 8 + piece;
                    *reinterpret_cast<uint4*>(p_tile_row + (at >> 3) * (ROWS * 128) +
                                              (((at & 7) ^ (row & 7)) << 4)) = packed;
                }
                {
                    float even, odd;
                    unpair(add_pair(partial[0], partial[1]), even, odd);
                    l = l * moved + (even + odd);
                }
                // P is written, the scores are read and the output is against m: tell the
                // product warp
                fence_async_shared();
                fence_before_sync();
                __syncwarp();
                if (lane == 0) barrier_arrive(p_ready(t & 1));
            }
            float o[MY_DIMS];
#pragma unroll
            for (int d = 0; d < MY_DIMS; ++d) o[d] = 0.f;
            if (ok) ok = out_ready(t - 1);
            if (ok) tmem_load<MY_DIMS>(my_out, o);
            // the next item's first product overwrites the output: it waits for this item's
            // reads, since it needs that item's P, which these warps write after this
            fence_before_sync();
            // the row's sum: all parts used the same maxima, so their sums add
            if (PARTS > 1) {
                sums[part * ROWS + row] = l;
                asm volatile("bar.sync %0, %1;" ::"r"(row_barrier), "n"(PARTS * 32) : "memory");
                l = 0.f;
#pragma unroll
                for (int other = 0; other < PARTS; ++other) l += sums[other * ROWS + row];
            }
            if (ok && valid && split_row != nullptr) {
                // unnormalised, against m: the merge scales the splits to their common maximum
#pragma unroll
                for (int d = 0; d < MY_DIMS; d += 2)       // (a row of HD + 2 floats is 8-byte aligned)
                    *reinterpret_cast<float2*>(split_row + part * MY_DIMS + d) = make_float2(o[d], o[d + 1]);
                if (part == 0) { split_row[HD] = m; split_row[HD + 1] = l; }
            } else if (ok && valid) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                const int head = item.kv_head * group + row % group;
                bf16* dst = out + ((size_t)(item.q_token + token) * heads + head) * HD + part * MY_DIMS;
#pragma unroll
                for (int piece = 0; piece < MY_DIMS / 8; ++piece) {
                    uint4 packed;
                    packed.x = pack_bf16(o[piece * 8 + 0] * inv, o[piece * 8 + 1] * inv);
                    packed.y = pack_bf16(o[piece * 8 + 2] * inv, o[piece * 8 + 3] * inv);
                    packed.z = pack_bf16(o[piece * 8 + 4] * inv, o[piece * 8 + 5] * inv);
                    packed.w = pack_bf16(o[piece * 8 + 6] * inv, o[piece * 8 + 7] * inv);
                    *reinterpret_cast<uint4*>(dst + piece * 8) = packed;
                }
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

bool supported(int head_dim, int heads, int kv_heads, int page_size) {
    if (head_dim != HD || kv_heads <= 0 || heads % kv_heads != 0) return false;
    const int group = heads / kv_heads;
    if (group > ROWS) return false;          // (a group that does not divide the rows leaves some unused)
    if (page_size < 8 || page_size % 8 != 0) return false;
    // pages divide a tile of 64 keys (and so one of 128), or are whole tiles
    return page_size <= 64 ? 64 % page_size == 0 : page_size % 128 == 0;
}

}  // namespace

// 1 if the tcgen05 prefill kernel takes this geometry (bfloat16 is implied) and the driver has
// the tensor-map encoder.
MLXONE_API int mlxone_attention_tcgen05_supports(int head_dim, int heads, int kv_heads,
                                                 int page_size) {
    return supported(head_dim, heads, kv_heads, page_size) && find_encoder() ? 1 : 0;
}

// Into how many parts, by keys, a launch should cut its items: more than one when there are
// fewer items (tiles of 128 query rows x key heads) than SMs and the contexts (up to
// `max_context` keys) are long enough for at least six tiles of 64 keys a part. The caller then
// gives `partial`, tokens x heads x splits x (64 + 2) floats, and merges it afterwards
// (mlxone_attention_merge).
MLXONE_API int mlxone_attention_tcgen05_splits(int tokens, int requests, int heads, int kv_heads,
                                               int max_context) {
    if (tokens <= 0 || requests <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return 1;
    if (g_sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, device);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    const int tile_tokens = ROWS / (heads / kv_heads);
    if (tile_tokens < 1) return 1;
    const long long items = (long long)((tokens + tile_tokens - 1) / tile_tokens + requests) * kv_heads;
    if (items >= g_sm_count) return 1;
    long long splits = 2LL * g_sm_count / items;
    const long long by_keys = max_context / 64 / 6;
    if (splits > by_keys) splits = by_keys;
    if (splits > 8) splits = 8;
    return splits < 1 ? 1 : (int)splits;
}

// q: [tokens, heads, 64] bfloat16; kv: [2, pages, kv_heads, page_size, 64]; out: [tokens, heads * 64].
// splits > 1 (with partial, see mlxone_attention_tcgen05_splits): the items are cut by keys and
// `out` is left for the merge to write.
MLXONE_API int mlxone_attention_prefill_tcgen05(const void* q, const void* kv, const int* block_table,
                                                int table_width, int page_size, int pages,
                                                const int* request_start, const int* history,
                                                void* out, int tokens, int requests, int heads,
                                                int kv_heads, int head_dim, float scale, int window,
                                                int splits, float* partial, int* error_flag,
                                                cudaStream_t stream) {
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
    const long long value_rows = (long long)pages * kv_heads * page_size;
    MLXONE_REQUIRE(2 * value_rows < (1LL << 31), "attention_prefill_tcgen05: the cache has too many rows");
    if (g_sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, device);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    MLXONE_REQUIRE(splits >= 1 && splits <= 64 && (splits == 1 || partial != nullptr),
                   "attention_prefill_tcgen05: %d splits need a scratch buffer", splits);
    if (splits == 1) partial = nullptr;
    const int token_tiles = (tokens + tile_tokens - 1) / tile_tokens + requests;     // an upper bound
    const long long all_items = (long long)token_tiles * kv_heads * splits;
    // tiles of 64 keys and two blocks an SM when there are items for all of those blocks, or
    // when the items are cut by keys (their parts then run side by side)
    const bool small_tiles = all_items >= 2LL * g_sm_count || splits > 1;
    const int keys = small_tiles ? 64 : 128;
    const int box_keys = page_size < keys ? page_size : keys;
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
    // persistent blocks, as many as the GPU holds at once; more only if a block would get more
    // items than it can list
    const long long resident = (long long)g_sm_count * (small_tiles ? 2 : 1);
    long long blocks = all_items < resident ? all_items : resident;
    if ((all_items + blocks - 1) / blocks > MAX_ITEMS) blocks = (all_items + MAX_ITEMS - 1) / MAX_ITEMS;
    const int shared = small_tiles ? Shape<64>::SHARED_BYTES : Shape<128>::SHARED_BYTES;
    // fewer items than SMs (a prompt's portion beside a step's decodes): every block has one
    // item and walks its key tiles one after the other, so two threads share a row's softmax
    const bool shared_rows = !small_tiles && all_items < g_sm_count;
    const int threads = ((shared_rows ? 2 : 1) * 4 + 2) * 32;
    auto kernel = small_tiles ? attention_tcgen05_kernel<64, 1>
                              : shared_rows ? attention_tcgen05_kernel<128, 2>
                                            : attention_tcgen05_kernel<128, 1>;
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, shared);
    if (err != cudaSuccess) {
        mlxone_set_error("attention_prefill_tcgen05: %s", cudaGetErrorString(err));
        return 2;
    }
    kernel<<<dim3((unsigned)blocks), threads, shared, stream>>>(
        map_q, map_kv, value_rows, block_table, table_width, page_size, box_keys, request_start,
        history, static_cast<bf16*>(out), requests, heads, kv_heads, scale * 1.4426950408889634f,
        window, token_tiles, splits, partial, error_flag);
    MLXONE_LAUNCH_CHECK("attention_prefill_tcgen05");
    return 0;
}
