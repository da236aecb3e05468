// Paged grouped-query attention on tensor cores (bfloat16): a prefill kernel for portions of
// any length and a split-key decode kernel for steps in which every request brings one token.
//
// Both read keys and values only from the request's pages (this step's own keys were written
// there before), 64 keys at a time, copied asynchronously into shared memory while the
// previous 64 are being used. Scores and the softmax statistics are 32-bit; probabilities are
// rounded to bfloat16 for the second product, whose accumulator is 32-bit again.
//
//   prefill: one block = 64 query rows of one (request, query head); 4 warps x 16 rows; all
//            warps walk the same key tiles (two buffers per block).
//   decode:  one block = one (request, key head, split of the keys) and up to 8 of the query
//            heads that share the key head; its 8 warps take different tiles of 32 keys, each
//            through a buffer of its own, and are merged in shared memory. With more than one
//            split the block writes (unnormalised output, max, sum) per head to scratch
//            memory and a second kernel merges the splits.
//
// Head sizes: multiples of 16 up to 128. Anything else runs the general kernel.
#include <cuda_pipeline_primitives.h>

#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int PREFILL_KEYS = 64;  // keys per tile of the prefill kernel
constexpr int DECODE_KEYS = 32;   // and of the decode kernel (smaller: more blocks per SM)
constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

// ------------------------------------------------------------------ small PTX wrappers

__device__ __forceinline__ uint32_t smem_address(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void copy16(void* dst, const void* src, bool live) {
    const int bytes = live ? 16 : 0;          // 0 bytes read: the 16 bytes are filled with zero
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_address(dst)),
                 "l"(src), "r"(bytes));
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void copy_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_address(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_address(p)));
}

// d += a (16x16, row) * b (16x8, col), bfloat16 in, float accumulate
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 2^x for x <= 0 (softmax weights): the hardware approximation, two units in the last place
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// ------------------------------------------------------------------ tiles in shared memory

// A tile row holds HD bfloat16 plus 16 bytes of padding, which keeps the eight rows that one
// ldmatrix reads on different banks for every HD that is a multiple of 16.
template <int HD>
struct Tile {
    static constexpr int STRIDE = HD + 8;                 // elements
    static constexpr int CHUNKS = HD / 8;                 // 16-byte pieces of a row
};

struct Pages {
    const bf16* keys;        // [pages, kv_heads, page_size, HD]
    const bf16* values;
    const int* table;        // this request's row of the block table
    int table_width, page_size, kv_heads, kv_head;
    int page_shift;          // log2(page_size) if it is a power of two, else -1
};

// Copies keys first..first+KEYS-1 of one key head into a K and a V tile; rows outside [lowest,
// last] or without a page are zero. `lanes` threads take part, this one is `lane`.
template <int HD, int KEYS>
__device__ __forceinline__ void load_tile(bf16* k_tile, bf16* v_tile, const Pages& pages, int first,
                                          int lowest, int last, int lane, int lanes) {
    using T = Tile<HD>;
    if (lanes == 32 && pages.page_shift >= 0) {
        // One warp, pages of a power of two: lane j looks up the tile's j-th page once and the
        // warp shares the page numbers by shuffle, so the copy loop has no load in its way.
        const int per_tile = max(KEYS >> pages.page_shift, 1);
        const int block = (first >> pages.page_shift) + lane;
        int my_page = -1;
        if (lane < per_tile && block < pages.table_width) my_page = pages.table[block];
        const int inside = first & (pages.page_size - 1);       // 0 unless pages are larger than a tile
#pragma unroll
        for (int piece = lane; piece < KEYS * T::CHUNKS; piece += 32) {
            const int row = piece / T::CHUNKS, chunk = piece % T::CHUNKS;
            const int key = first + row;
            const int page = __shfl_sync(0xffffffffu, my_page, (inside + row) >> pages.page_shift);
            const bool live = key >= lowest && key <= last && page >= 0;
            const size_t offset =
                live ? (((size_t)page * pages.kv_heads + pages.kv_head) * pages.page_size +
                        ((inside + row) & (pages.page_size - 1))) * HD + chunk * 8
                     : 0;
            copy16(k_tile + row * T::STRIDE + chunk * 8, pages.keys + offset, live);
            copy16(v_tile + row * T::STRIDE + chunk * 8, pages.values + offset, live);
        }
        return;
    }
#pragma unroll 8
    for (int piece = lane; piece < KEYS * T::CHUNKS; piece += lanes) {
        const int row = piece / T::CHUNKS, chunk = piece % T::CHUNKS;
        const int key = first + row;
        bool live = key >= lowest && key <= last;
        size_t offset = 0;
        if (live) {
            const int block = pages.page_shift >= 0 ? key >> pages.page_shift : key / pages.page_size;
            const int within = pages.page_shift >= 0 ? key & (pages.page_size - 1)
                                                      : key - block * pages.page_size;
            const int page = block < pages.table_width ? pages.table[block] : -1;
            live = page >= 0;
            if (live)
                offset = (((size_t)page * pages.kv_heads + pages.kv_head) * pages.page_size +
                          within) * HD + chunk * 8;
        }
        copy16(k_tile + row * T::STRIDE + chunk * 8, pages.keys + offset, live);
        copy16(v_tile + row * T::STRIDE + chunk * 8, pages.values + offset, live);
    }
}

// One warp: 16 query rows (their fragments in `qf`) against one tile of KEYS keys.
// `limit_lo[i]`/`limit_hi[i]` (i = 0: row lane/4, 1: row lane/4 + 8) bound the keys that the row
// may see; with MASKED false the caller has checked that every row sees the whole tile.
// Updates the running max `m` (of score * scale * log2 e), the sum `l` and `o`.
template <int HD, int KEYS, bool MASKED>
__device__ __forceinline__ void attend_tile(const uint32_t (&qf)[HD / 16][4], const bf16* k_tile,
                                            const bf16* v_tile, int first, const int (&limit_lo)[2],
                                            const int (&limit_hi)[2], float scale_log2,
                                            float (&m)[2], float (&l)[2], float (&o)[HD / 8][4],
                                            int lane) {
    using T = Tile<HD>;
    float s[KEYS / 8][4];
#pragma unroll
    for (int j = 0; j < KEYS / 8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) s[j][c] = 0.f;

    const int matrix = lane >> 3, r = lane & 7;
#pragma unroll
    for (int kk = 0; kk < HD / 16; ++kk) {
#pragma unroll
        for (int jj = 0; jj < KEYS / 16; ++jj) {
            uint32_t b[4];
            ldmatrix_x4(b, k_tile + (jj * 16 + r + (matrix >> 1) * 8) * T::STRIDE + kk * 16 +
                               (matrix & 1) * 8);
            mma_16816(s[2 * jj], qf[kk], b[0], b[1]);
            mma_16816(s[2 * jj + 1], qf[kk], b[2], b[3]);
        }
    }

    // the tile's row maxima (of the raw scores; masked ones count as -inf)
    const int t2 = (lane & 3) * 2;
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < KEYS / 8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int i = c >> 1;
            if (MASKED) {
                const int key = first + j * 8 + t2 + (c & 1);
                if (!(key >= limit_lo[i] && key <= limit_hi[i])) s[j][c] = -INFINITY;
            }
            tile_max[i] = fmaxf(tile_max[i], s[j][c]);
        }
    float correction[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
        tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
        const float new_max = fmaxf(m[i], tile_max[i] * scale_log2);
        correction[i] = new_max == -INFINITY ? 1.f : fast_exp2(m[i] - new_max);
        m[i] = new_max;
    }
    float tile_sum[2] = {0.f, 0.f};
    const float shift[2] = {m[0] == -INFINITY ? 0.f : m[0], m[1] == -INFINITY ? 0.f : m[1]};
#pragma unroll
    for (int j = 0; j < KEYS / 8; ++j)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int i = c >> 1;
            const float p = fast_exp2(fmaf(s[j][c], scale_log2, -shift[i]));   // exp2(-inf) = 0
            s[j][c] = p;
            tile_sum[i] += p;
        }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        tile_sum[i] += __shfl_xor_sync(0xffffffffu, tile_sum[i], 1);
        tile_sum[i] += __shfl_xor_sync(0xffffffffu, tile_sum[i], 2);
        l[i] = l[i] * correction[i] + tile_sum[i];
    }
#pragma unroll
    for (int n = 0; n < HD / 8; ++n) {
        o[n][0] *= correction[0]; o[n][1] *= correction[0];
        o[n][2] *= correction[1]; o[n][3] *= correction[1];
    }

    // o += p * v
#pragma unroll
    for (int kk = 0; kk < KEYS / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int nn = 0; nn < HD / 16; ++nn) {
            uint32_t b[4];
            ldmatrix_x4_trans(b, v_tile + (kk * 16 + r + (matrix & 1) * 8) * T::STRIDE + nn * 16 +
                                     (matrix >> 1) * 8);
            mma_16816(o[2 * nn], a, b[0], b[1]);
            mma_16816(o[2 * nn + 1], a, b[2], b[3]);
        }
    }
}

// ------------------------------------------------------------------ prefill

constexpr int PREFILL_WARPS = 4;       // 8 warps (128 rows) measured the same on long prompts
constexpr int ROWS = 16 * PREFILL_WARPS;      // query rows per block

template <int HD>
__global__ void __launch_bounds__(PREFILL_WARPS * 32)
attention_prefill_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv, long long kv_half,
                         const int* __restrict__ block_table, int table_width, int page_size,
                         const int* __restrict__ request_start, const int* __restrict__ history,
                         bf16* __restrict__ out, int requests, int heads, int kv_heads,
                         float scale_log2, int window) {
    using T = Tile<HD>;
    constexpr int KEYS = PREFILL_KEYS;
    extern __shared__ __align__(16) unsigned char shared_bytes[];
    bf16* q_tile = reinterpret_cast<bf16*>(shared_bytes);
    bf16* k_tiles = q_tile + ROWS * T::STRIDE;
    bf16* v_tiles = k_tiles + 2 * KEYS * T::STRIDE;
    __shared__ int found[2];

    // which request and which 64 rows of it this block serves
    if (threadIdx.x == 0) {
        // the last blocks of a causal prompt have the most keys to walk: they go first
        int left = gridDim.x - 1 - blockIdx.x, request = -1, start = 0;
        for (int r = 0; r < requests; ++r) {
            const int tiles = (request_start[r + 1] - request_start[r] + ROWS - 1) / ROWS;
            if (left < tiles) { request = r; start = left * ROWS; break; }
            left -= tiles;
        }
        found[0] = request;
        found[1] = start;
    }
    __syncthreads();
    const int request = found[0];
    if (request < 0) return;
    const int row_start = found[1];
    const int head = blockIdx.y;
    const int first_token = request_start[request];
    const int count = request_start[request + 1] - first_token;
    const int rows = min(ROWS, count - row_start);
    const int before = history[request];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    Pages pages{kv, kv + kv_half, block_table + (size_t)request * table_width, table_width,
                page_size, kv_heads, head / (heads / kv_heads),
                (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1};

    // the query rows of this block (zero beyond the portion's end)
    for (int piece = threadIdx.x; piece < ROWS * T::CHUNKS; piece += PREFILL_WARPS * 32) {
        const int row = piece / T::CHUNKS, chunk = piece % T::CHUNKS;
        const bool live = row < rows;
        const bf16* src = q + ((size_t)(first_token + row_start + (live ? row : 0)) * heads + head) *
                                  HD + chunk * 8;
        copy16(q_tile + row * T::STRIDE + chunk * 8, src, live);
    }
    const int first_position = before + row_start;
    const int last_position = first_position + rows - 1;
    const int lowest = window > 0 ? max(first_position - window + 1, 0) : 0;
    const int tile_first = lowest / KEYS, tile_last = last_position / KEYS;

    load_tile<HD, KEYS>(k_tiles, v_tiles, pages, tile_first * KEYS, lowest, last_position, threadIdx.x,
                  PREFILL_WARPS * 32);
    copy_commit();

    // per-thread rows: lane/4 and lane/4 + 8 of the warp's 16
    int limit_lo[2], limit_hi[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = warp * 16 + (lane >> 2) + i * 8;
        const int position = first_position + row;
        limit_hi[i] = row < rows ? position : -1;
        limit_lo[i] = window > 0 ? max(position - window + 1, 0) : 0;
    }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    float o[HD / 8][4];
#pragma unroll
    for (int n = 0; n < HD / 8; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
    uint32_t qf[HD / 16][4];              // this warp's query rows, loaded once
    bool have_q = false;
    // keys that every row of this warp sees in full: from the largest lower limit to the first
    // row's position (rows beyond the portion's end see nothing, so such a warp always masks)
    const int warp_first = first_position + warp * 16;
    const bool warp_whole = warp * 16 + 15 < rows;
    const int open_lo = window > 0 ? max(warp_first + 15 - window + 1, 0) : 0;

    for (int tile = tile_first; tile <= tile_last; ++tile) {
        const int buffer = (tile - tile_first) & 1;
        if (tile < tile_last) {
            load_tile<HD, KEYS>(k_tiles + (buffer ^ 1) * KEYS * T::STRIDE,
                          v_tiles + (buffer ^ 1) * KEYS * T::STRIDE, pages, (tile + 1) * KEYS,
                          lowest, last_position, threadIdx.x, PREFILL_WARPS * 32);
            copy_commit();
            copy_wait<1>();
        } else {
            copy_wait<0>();
        }
        __syncthreads();
        // a warp whose rows all lie before this tile's keys has nothing to see in it
        const int warp_last = first_position + min(warp * 16 + 15, rows - 1);
        if (warp * 16 < rows && tile * KEYS <= warp_last) {
            if (!have_q) {
                const int matrix = lane >> 3, r = lane & 7;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
                    ldmatrix_x4(qf[kk], q_tile + (warp * 16 + r + (matrix & 1) * 8) * T::STRIDE +
                                            kk * 16 + (matrix >> 1) * 8);
                have_q = true;
            }
            const bf16* k_now = k_tiles + buffer * KEYS * T::STRIDE;
            const bf16* v_now = v_tiles + buffer * KEYS * T::STRIDE;
            const bool open = warp_whole && tile * KEYS >= open_lo &&
                              tile * KEYS + KEYS - 1 <= warp_first;
            if (open)
                attend_tile<HD, KEYS, false>(qf, k_now, v_now, tile * KEYS, limit_lo, limit_hi,
                                             scale_log2, m, l, o, lane);
            else
                attend_tile<HD, KEYS, true>(qf, k_now, v_now, tile * KEYS, limit_lo, limit_hi,
                                            scale_log2, m, l, o, lane);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int row = warp * 16 + (lane >> 2) + i * 8;
        if (row >= rows) continue;
        const float inv = l[i] > 0.f ? 1.f / l[i] : 0.f;
        bf16* dst = out + ((size_t)(first_token + row_start + row) * heads + head) * HD +
                    (lane & 3) * 2;
#pragma unroll
        for (int n = 0; n < HD / 8; ++n)
            *reinterpret_cast<__nv_bfloat162*>(dst + n * 8) =
                __floats2bfloat162_rn(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
    }
}

// ------------------------------------------------------------------ decode (split keys)

__device__ __forceinline__ uint32_t transpose_8x8(uint32_t v) {
    uint32_t out;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;\n" : "=r"(out) : "r"(v));
    return out;
}

constexpr int DECODE_WARPS = 2;
constexpr int DECODE_STAGES = 3;     // tiles a warp keeps in flight or in use
constexpr int DECODE_HEADS = 8;      // query heads per block (the 8-column operand)

// One block = one (request, key head, group of up to 8 query heads, split of the keys).
// Keys are the 16-row operand of the first product (scores^T = K q^T), so no tensor-core row
// is wasted on padding; the probabilities are transposed in registers (movmatrix) and become
// the 8-column operand of the second product (out^T = V^T p^T). Each warp takes tiles of 32
// keys in turn through a ring of its own, which keeps DECODE_STAGES - 1 tiles on their way while
// one is multiplied: the step is bound by the latency of memory unless enough is in flight, and
// small blocks (few warps, many blocks per SM) spread the work evenly. The warps are merged in
// shared memory.
// partial results: [token, head, split] -> HD floats of unnormalised output, then max and sum.
// With CLUSTER the blocks of one (request, key head) form a thread-block cluster (one block per
// split, at most 8): they leave their partial results in their own shared memory, and after a
// barrier over the cluster block r merges head r from the others' shared memory (distributed
// shared memory), so that neither a scratch buffer nor a merge kernel is needed.
// With PREP the kernel starts from the step's fused projection instead of prepared queries: `q` is
// qkv [requests, (heads + 2 kv_heads) * HD], and the kernel applies the per-head RMSNorm and the
// rotation to its own query heads in registers, and to the token's new key where it meets the
// tile that holds the token's position; key and value of the token are put into that tile in
// shared memory and (by one block per request and key head) into the request's page. A step of
// single tokens then needs no kernel of its own for the preparation. HD must be a multiple of 32
// (a rotation pair then sits in one lane) and the rotation covers the whole head or nothing.
struct DecodePrep {
    const float* q_weight = nullptr;      // [HD] or null: no norm
    const float* k_weight = nullptr;
    float eps = 0.f;
    const float* inv_freq = nullptr;      // [HD / 2] or null: no rotation
    bf16* cache = nullptr;                // the writable cache (keys, then values after kv_half)
    int write_kv = 0;
    int* error_flag = nullptr;
};

template <int HD, bool CLUSTER, bool PREP>
__global__ void __launch_bounds__(DECODE_WARPS * 32)
attention_decode_kernel(const bf16* __restrict__ q, const bf16* __restrict__ kv, long long kv_half,
                        const int* __restrict__ block_table, int table_width, int page_size,
                        const int* __restrict__ positions, bf16* __restrict__ out,
                        float* __restrict__ partial, int heads, int kv_heads, int splits,
                        float scale_log2, int window, DecodePrep prep) {
    using T = Tile<HD>;
    constexpr int KEYS = DECODE_KEYS;
    constexpr int ROW_FLOATS = HD + 2;
    extern __shared__ __align__(16) unsigned char shared_bytes[];
    griddep_launch();
    const int group = heads / kv_heads;
    const int groups_of_8 = (group + DECODE_HEADS - 1) / DECODE_HEADS;
    const int kv_head = blockIdx.x / groups_of_8;
    const int head0 = kv_head * group + (blockIdx.x % groups_of_8) * DECODE_HEADS;
    const int rows = min(DECODE_HEADS, kv_head * group + group - head0);
    const int request = blockIdx.y;            // one token per request: token index = request
    const int split = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const int position = positions[request];
    const int lowest = window > 0 ? max(position - window + 1, 0) : 0;
    const int tile_first = lowest / KEYS, tile_count = position / KEYS - tile_first + 1;
    const int per_split = (tile_count + splits - 1) / splits;
    const int my_first = tile_first + split * per_split;
    const int my_last = min(my_first + per_split, tile_first + tile_count) - 1;

    Pages pages{kv, kv + kv_half, block_table + (size_t)request * table_width, table_width,
                page_size, kv_heads, kv_head,
                (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1};
    constexpr int STAGE = 2 * KEYS * T::STRIDE;          // elements of a K and a V tile
    bf16* ring = reinterpret_cast<bf16*>(shared_bytes) + (size_t)warp * DECODE_STAGES * STAGE;

    // The kernel before this one wrote the token's own key and value (and its query): the tiles
    // before the one that holds them are what earlier steps left, and are asked for before that
    // kernel is waited for, so that they are on their way while it finishes.
    int tile = my_first + warp;
    const int newest = position / KEYS;
    auto fetch = [&](int ahead) {
        const int coming = tile + ahead * DECODE_WARPS;
        if (coming <= my_last)
            load_tile<HD, KEYS>(ring + ahead * STAGE, ring + ahead * STAGE + KEYS * T::STRIDE, pages,
                                coming * KEYS, lowest, position, lane, 32);
        copy_commit();
    };
    int ahead = 0;
    // (with PREP nobody writes the cache before this kernel: the token's own row of the newest
    // tile is put into shared memory below, over whatever the copy brought)
    for (; ahead < DECODE_STAGES - 1 && (PREP || tile + ahead * DECODE_WARPS != newest); ++ahead)
        fetch(ahead);
    // PREP: what the preparation needs beside the projection's row depends on the step's
    // positions and on constants only, so it is worked out while the projection still runs:
    // this lane's norm weights and the sines and cosines of its rotation pairs (query layout:
    // dims 16 kk + 2t, +1, +8 + 2t, +9 + 2t; key layout: dims lane + 32 i and that + HD / 2).
    float q_scale[PREP ? HD / 16 : 1][4], q_sine[PREP ? HD / 32 : 1][4], q_cosine[PREP ? HD / 32 : 1][4];
    constexpr int KEY_PAIRS = (HD / 2 + 31) / 32;
    float k_scale_lo[KEY_PAIRS], k_scale_hi[KEY_PAIRS], k_sine[KEY_PAIRS], k_cosine[KEY_PAIRS];
    // the warp that will meet the tile with the token's own position prepares its key
    const bool meets_newest = PREP && prep.write_kv && newest >= tile && newest <= my_last &&
                              (newest - tile) % DECODE_WARPS == 0;
    if (PREP) {
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk)
#pragma unroll
            for (int c = 0; c < 4; ++c)
                q_scale[kk][c] = prep.q_weight != nullptr
                                     ? prep.q_weight[kk * 16 + (c >> 1) * 8 + 2 * t + (c & 1)] : 1.f;
#pragma unroll
        for (int kk = 0; kk < HD / 32; ++kk)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                q_sine[kk][c] = 0.f; q_cosine[kk][c] = 1.f;
                if (prep.inv_freq != nullptr)
                    sincosf((float)position * prep.inv_freq[kk * 16 + (c >> 1) * 8 + 2 * t + (c & 1)],
                            &q_sine[kk][c], &q_cosine[kk][c]);
            }
#pragma unroll
        for (int i = 0; i < KEY_PAIRS; ++i) {
            const int j = lane + 32 * i;
            k_scale_lo[i] = k_scale_hi[i] = 1.f; k_sine[i] = 0.f; k_cosine[i] = 1.f;
            if (meets_newest && j < HD / 2) {
                if (prep.k_weight != nullptr) {
                    k_scale_lo[i] = prep.k_weight[j];
                    k_scale_hi[i] = prep.k_weight[j + HD / 2];
                }
                if (prep.inv_freq != nullptr)
                    sincosf((float)position * prep.inv_freq[j], &k_sine[i], &k_cosine[i]);
            }
        }
    }
    griddep_wait();
    for (; ahead < DECODE_STAGES - 1; ++ahead) fetch(ahead);

    // q^T as the 8-column operand: head g, dims 16 kk + 2t (+1) and + 8
    uint32_t qb[HD / 16][2];
    {
        const bool live = g < rows;
        const size_t row_stride = PREP ? (size_t)(heads + 2 * kv_heads) * HD : (size_t)heads * HD;
        const bf16* row = q + (size_t)request * row_stride + (size_t)(head0 + (live ? g : 0)) * HD;
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
            qb[kk][0] = live ? *reinterpret_cast<const uint32_t*>(row + kk * 16 + 2 * t) : 0u;
            qb[kk][1] = live ? *reinterpret_cast<const uint32_t*>(row + kk * 16 + 8 + 2 * t) : 0u;
        }
        if (PREP) {
            // this lane's 4 values of every 16-wide piece: dims 16 kk + 2t, +1, +8 + 2t, +9 + 2t;
            // the four lanes of a head hold all HD between them
            float v[HD / 16][4];
            float sum = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&qb[kk][0]);
                const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&qb[kk][1]);
                v[kk][0] = __low2float(lo); v[kk][1] = __high2float(lo);
                v[kk][2] = __low2float(hi); v[kk][3] = __high2float(hi);
#pragma unroll
                for (int c = 0; c < 4; ++c) sum += v[kk][c] * v[kk][c];
            }
            if (prep.q_weight != nullptr) {
                sum += __shfl_xor_sync(0xffffffffu, sum, 1);
                sum += __shfl_xor_sync(0xffffffffu, sum, 2);
                const float inv = rsqrtf(sum / (float)HD + prep.eps);
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk)
#pragma unroll
                    for (int c = 0; c < 4; ++c) v[kk][c] = v[kk][c] * inv * q_scale[kk][c];
            }
            if (prep.inv_freq != nullptr) {
                // dimension j of the first half pairs with j + HD / 2: piece kk with piece kk + HD / 32
#pragma unroll
                for (int kk = 0; kk < HD / 32; ++kk)
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const float a = v[kk][c], b = v[kk + HD / 32][c];
                        v[kk][c] = a * q_cosine[kk][c] - b * q_sine[kk][c];
                        v[kk + HD / 32][c] = b * q_cosine[kk][c] + a * q_sine[kk][c];
                    }
            }
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                qb[kk][0] = live ? pack_bf16(v[kk][0], v[kk][1]) : 0u;
                qb[kk][1] = live ? pack_bf16(v[kk][2], v[kk][3]) : 0u;
            }
        }
    }
    // The token's own key and value (the warp that will meet their tile): normed and rotated
    // here from the projection's row, while the first tiles are on their way. Lane e takes dims
    // e, e + 32, ...: a rotation pair (j, j + HD / 2) lies in one lane.
    float k_lo[KEY_PAIRS], k_hi[KEY_PAIRS], v_lo[KEY_PAIRS], v_hi[KEY_PAIRS];
    if (PREP && meets_newest) {
        constexpr int HALF = HD / 2;
        const bf16* row = q + (size_t)request * (heads + 2 * kv_heads) * HD;
        const bf16* k_src = row + (size_t)(heads + kv_head) * HD;
        const bf16* v_src = row + (size_t)(heads + kv_heads + kv_head) * HD;
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < KEY_PAIRS; ++i) {
            const int j = lane + 32 * i;
            const bool mine = j < HALF;
            k_lo[i] = mine ? __bfloat162float(k_src[j]) : 0.f;
            k_hi[i] = mine ? __bfloat162float(k_src[j + HALF]) : 0.f;
            v_lo[i] = mine ? __bfloat162float(v_src[j]) : 0.f;
            v_hi[i] = mine ? __bfloat162float(v_src[j + HALF]) : 0.f;
            sum += k_lo[i] * k_lo[i] + k_hi[i] * k_hi[i];
        }
        if (prep.k_weight != nullptr) {
            sum = warp_sum(sum);
            const float inv = rsqrtf(sum / (float)HD + prep.eps);
#pragma unroll
            for (int i = 0; i < KEY_PAIRS; ++i) {
                k_lo[i] = k_lo[i] * inv * k_scale_lo[i];
                k_hi[i] = k_hi[i] * inv * k_scale_hi[i];
            }
        }
        if (prep.inv_freq != nullptr) {
#pragma unroll
            for (int i = 0; i < KEY_PAIRS; ++i) {
                const float a = k_lo[i], b = k_hi[i];
                k_lo[i] = a * k_cosine[i] - b * k_sine[i];
                k_hi[i] = b * k_cosine[i] + a * k_sine[i];
            }
        }
    }
    const bool head_live[2] = {2 * t < rows, 2 * t + 1 < rows};
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};      // per head 2t, 2t + 1
    float o[HD / 16][4];
#pragma unroll
    for (int d = 0; d < HD / 16; ++d)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[d][c] = 0.f;
    const int matrix = lane >> 3, r = lane & 7;

    for (int stage = 0; tile <= my_last; tile += DECODE_WARPS, stage = (stage + 1) % DECODE_STAGES) {
        copy_wait<DECODE_STAGES - 2>();
        __syncwarp();            // the tile has landed, and every lane is done with the one before
        {
            const int coming = tile + (DECODE_STAGES - 1) * DECODE_WARPS;
            const int into = (stage + DECODE_STAGES - 1) % DECODE_STAGES;
            if (coming <= my_last)
                load_tile<HD, KEYS>(ring + into * STAGE, ring + into * STAGE + KEYS * T::STRIDE,
                                    pages, coming * KEYS, lowest, position, lane, 32);
            copy_commit();
        }
        const bf16* k_tile = ring + stage * STAGE;
        const bf16* v_tile = k_tile + KEYS * T::STRIDE;
        const int first = tile * KEYS;
        if (PREP && tile == newest && prep.write_kv) {
            // The token's own key and value, prepared before the loop: put into the tile over
            // what the copy brought, and written to the request's page by the first block of
            // this key head.
            constexpr int HALF = HD / 2;
            bf16* k_row = const_cast<bf16*>(k_tile) + (size_t)(position - first) * T::STRIDE;
            bf16* v_row = const_cast<bf16*>(v_tile) + (size_t)(position - first) * T::STRIDE;
            const int block = pages.page_shift >= 0 ? position >> pages.page_shift
                                                    : position / page_size;
            const int page = block < table_width ? pages.table[block] : -1;
            const bool writer = blockIdx.x % groups_of_8 == 0 && page >= 0;
            if (page < 0 && lane == 0 && prep.error_flag != nullptr) atomicExch(prep.error_flag, 2);
            const size_t at = (((size_t)(page < 0 ? 0 : page) * kv_heads + kv_head) * page_size +
                               (position - block * page_size)) * HD;
#pragma unroll
            for (int i = 0; i < KEY_PAIRS; ++i) {
                const int j = lane + 32 * i;
                if (j >= HALF) continue;
                const bf16 ka = __float2bfloat16_rn(k_lo[i]), kb = __float2bfloat16_rn(k_hi[i]);
                const bf16 va = __float2bfloat16_rn(v_lo[i]), vb = __float2bfloat16_rn(v_hi[i]);
                k_row[j] = ka; k_row[j + HALF] = kb;
                v_row[j] = va; v_row[j + HALF] = vb;
                if (writer) {
                    prep.cache[at + j] = ka; prep.cache[at + j + HALF] = kb;
                    prep.cache[kv_half + at + j] = va; prep.cache[kv_half + at + j + HALF] = vb;
                }
            }
            __syncwarp();
        }
        float s[KEYS / 16][4];
#pragma unroll
        for (int mt = 0; mt < KEYS / 16; ++mt) {
#pragma unroll
            for (int c = 0; c < 4; ++c) s[mt][c] = 0.f;
#pragma unroll
            for (int kk = 0; kk < HD / 16; ++kk) {
                uint32_t a[4];
                ldmatrix_x4(a, k_tile + (mt * 16 + r + (matrix & 1) * 8) * T::STRIDE + kk * 16 +
                                   (matrix >> 1) * 8);
                mma_16816(s[mt], a, qb[kk][0], qb[kk][1]);
            }
        }
        float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int mt = 0; mt < KEYS / 16; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int key = first + mt * 16 + g + (c >> 1) * 8;
                const bool seen = key >= lowest && key <= position && head_live[c & 1];
                s[mt][c] = seen ? s[mt][c] * scale_log2 : -INFINITY;
                tile_max[c & 1] = fmaxf(tile_max[c & 1], s[mt][c]);
            }
        float correction[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 4));
            tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 8));
            tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 16));
            const float new_max = fmaxf(m[i], tile_max[i]);
            correction[i] = new_max == -INFINITY ? 1.f : fast_exp2(m[i] - new_max);
            m[i] = new_max;
            l[i] *= correction[i];        // l is this thread's share; the lanes are added at the end
        }
        uint32_t pt[KEYS / 16][2];        // probabilities, transposed: head g, keys 2t (+1)
#pragma unroll
        for (int mt = 0; mt < KEYS / 16; ++mt) {
            float p[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                p[c] = m[c & 1] == -INFINITY ? 0.f : fast_exp2(s[mt][c] - m[c & 1]);
                l[c & 1] += p[c];
            }
            pt[mt][0] = transpose_8x8(pack_bf16(p[0], p[1]));
            pt[mt][1] = transpose_8x8(pack_bf16(p[2], p[3]));
        }
#pragma unroll
        for (int d = 0; d < HD / 16; ++d) {
            o[d][0] *= correction[0]; o[d][1] *= correction[1];
            o[d][2] *= correction[0]; o[d][3] *= correction[1];
#pragma unroll
            for (int mt = 0; mt < KEYS / 16; ++mt) {
                uint32_t a[4];
                ldmatrix_x4_trans(a, v_tile + (mt * 16 + r + (matrix >> 1) * 8) * T::STRIDE + d * 16 +
                                         (matrix & 1) * 8);
                mma_16816(o[d], a, pt[mt][0], pt[mt][1]);
            }
        }
    }
    copy_wait<0>();
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 4);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 8);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 16);
    }
    __syncthreads();           // all warps are done with their tiles: reuse them for merging

    // merge the warps: every warp writes (o, m, l) of its heads, then all threads combine
    float* merge = reinterpret_cast<float*>(shared_bytes);      // [warp][head 0..7][HD + 2]
#pragma unroll
    for (int d = 0; d < HD / 16; ++d) {
        float* base = merge + (size_t)warp * DECODE_HEADS * ROW_FLOATS;
        base[(2 * t) * ROW_FLOATS + d * 16 + g] = o[d][0];
        base[(2 * t + 1) * ROW_FLOATS + d * 16 + g] = o[d][1];
        base[(2 * t) * ROW_FLOATS + d * 16 + g + 8] = o[d][2];
        base[(2 * t + 1) * ROW_FLOATS + d * 16 + g + 8] = o[d][3];
    }
    if (g == 0) {
        float* base = merge + (size_t)warp * DECODE_HEADS * ROW_FLOATS;
        base[(2 * t) * ROW_FLOATS + HD] = m[0];
        base[(2 * t) * ROW_FLOATS + HD + 1] = l[0];
        base[(2 * t + 1) * ROW_FLOATS + HD] = m[1];
        base[(2 * t + 1) * ROW_FLOATS + HD + 1] = l[1];
    }
    __syncthreads();
    for (int item = threadIdx.x; item < rows * HD; item += DECODE_WARPS * 32) {
        const int row = item / HD, d = item % HD;
        float top = -INFINITY;
#pragma unroll
        for (int w = 0; w < DECODE_WARPS; ++w)
            top = fmaxf(top, merge[((size_t)w * DECODE_HEADS + row) * ROW_FLOATS + HD]);
        float value = 0.f, sum = 0.f;
#pragma unroll
        for (int w = 0; w < DECODE_WARPS; ++w) {
            const float* src = merge + ((size_t)w * DECODE_HEADS + row) * ROW_FLOATS;
            const float weight = src[HD] == -INFINITY ? 0.f : fast_exp2(src[HD] - top);
            value += src[d] * weight;
            sum += src[HD + 1] * weight;
        }
        const int head = head0 + row;
        if (splits == 1) {
            out[((size_t)request * heads + head) * HD + d] =
                __float2bfloat16_rn(sum > 0.f ? value / sum : 0.f);
        } else if (CLUSTER) {
            float* own = merge + DECODE_WARPS * DECODE_HEADS * ROW_FLOATS + row * ROW_FLOATS;
            own[d] = value;
            if (d == 0) { own[HD] = top; own[HD + 1] = sum; }
        } else {
            float* dst = partial + (((size_t)request * heads + head) * splits + split) * ROW_FLOATS;
            dst[d] = value;
            if (d == 0) { dst[HD] = top; dst[HD + 1] = sum; }
        }
    }
    if (CLUSTER && splits > 1) {
        // every block of the cluster has left its partial results; block `split` merges the
        // heads split, split + splits, ... reading the others' shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;\n"
                     "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
        const uint32_t own_base =
            smem_address(merge + DECODE_WARPS * DECODE_HEADS * ROW_FLOATS);
        for (int item = threadIdx.x; item < rows * HD; item += DECODE_WARPS * 32) {
            const int row = item / HD, d = item % HD;
            if (row % splits != split) continue;
            float top = -INFINITY;
            float tops[8], sums[8], values[8];
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                tops[s] = -INFINITY; sums[s] = 0.f; values[s] = 0.f;
                if (s < splits) {
                    uint32_t remote;
                    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n"
                                 : "=r"(remote) : "r"(own_base + row * ROW_FLOATS * 4), "r"(s));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(tops[s]) : "r"(remote + HD * 4));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(sums[s]) : "r"(remote + (HD + 1) * 4));
                    asm volatile("ld.shared::cluster.f32 %0, [%1];\n" : "=f"(values[s]) : "r"(remote + d * 4));
                    top = fmaxf(top, tops[s]);
                }
            }
            float value = 0.f, sum = 0.f;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const float weight = tops[s] == -INFINITY ? 0.f : fast_exp2(tops[s] - top);
                value += values[s] * weight;
                sum += sums[s] * weight;
            }
            out[((size_t)request * heads + head0 + row) * HD + d] =
                __float2bfloat16_rn(sum > 0.f ? value / sum : 0.f);
        }
        // no block may leave while another still reads its shared memory
        asm volatile("barrier.cluster.arrive.release.aligned;\n"
                     "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
    }
}

// Merges the splits of one (token, head): one warp each. The lanes take the splits' maxima and
// sums side by side, and the loads of the weighted sum are independent of one another, so that
// the kernel costs a few trips to L2 and not one per split.
template <int HD>
__global__ void attention_merge_kernel(const float* __restrict__ partial, bf16* __restrict__ out,
                                       int items, int splits) {
    constexpr int ROW_FLOATS = HD + 2;
    constexpr int MINE = (HD + 31) / 32;
    griddep_launch();
    griddep_wait();
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= items) return;
    const float* base = partial + (size_t)item * splits * ROW_FLOATS;
    // the first HELD splits' values are asked for together with the maxima and sums, before
    // anything is computed from them: one trip to L2 for all of it, not one after the other
    constexpr int HELD = 32;
    float held[HELD][MINE];
#pragma unroll
    for (int j = 0; j < HELD; ++j)
#pragma unroll
        for (int i = 0; i < MINE; ++i) {
            const int d = lane + 32 * i;
            held[j][i] = (j < splits && d < HD) ? base[(size_t)j * ROW_FLOATS + d] : 0.f;
        }
    float its_top = -INFINITY, its_sum = 0.f;          // of split `lane`
    if (lane < splits) {
        its_top = base[(size_t)lane * ROW_FLOATS + HD];
        its_sum = base[(size_t)lane * ROW_FLOATS + HD + 1];
    }
    float top = its_top;
    for (int s = lane + 32; s < splits; s += 32) top = fmaxf(top, base[(size_t)s * ROW_FLOATS + HD]);
    top = warp_max(top);
    float sum = 0.f;
    float value[MINE];
#pragma unroll
    for (int i = 0; i < MINE; ++i) value[i] = 0.f;
    for (int s0 = 0; s0 < splits; s0 += 32) {
        // lane j holds the weight of split s0 + j
        float weight = 0.f;
        if (s0 + lane < splits) {
            const float* src = base + (size_t)(s0 + lane) * ROW_FLOATS;
            const float t = s0 == 0 ? its_top : src[HD];
            weight = t == -INFINITY ? 0.f : fast_exp2(t - top);
            sum += (s0 == 0 ? its_sum : src[HD + 1]) * weight;
        }
        const int count = min(32, splits - s0);
        if (s0 == 0) {
#pragma unroll
            for (int j = 0; j < HELD; ++j) {
                if (j >= count) break;
                const float w = __shfl_sync(0xffffffffu, weight, j);
#pragma unroll
                for (int i = 0; i < MINE; ++i) value[i] = fmaf(held[j][i], w, value[i]);
            }
        }
#pragma unroll 8
        for (int j = s0 == 0 ? HELD : 0; j < count; ++j) {
            const float w = __shfl_sync(0xffffffffu, weight, j);
            const float* src = base + (size_t)(s0 + j) * ROW_FLOATS;
#pragma unroll
            for (int i = 0; i < MINE; ++i) {
                const int d = lane + 32 * i;
                if (d < HD) value[i] = fmaf(src[d], w, value[i]);
            }
        }
    }
    sum = warp_sum(sum);
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
#pragma unroll
    for (int i = 0; i < MINE; ++i) {
        const int d = lane + 32 * i;
        if (d < HD) out[(size_t)item * HD + d] = __float2bfloat16_rn(value[i] * inv);
    }
}

template <int HD>
int launch_prefill(const void* q, const void* kv, long long kv_half, const int* block_table,
                   int table_width, int page_size, const int* request_start, const int* history,
                   void* out, int tokens, int requests, int heads, int kv_heads, float scale,
                   int window, cudaStream_t stream) {
    using T = Tile<HD>;
    const size_t shared = (size_t)(ROWS + 4 * PREFILL_KEYS) * T::STRIDE * 2;
    auto kernel = attention_prefill_kernel<HD>;
    if (shared > 48 * 1024)
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    const dim3 grid((tokens + ROWS - 1) / ROWS + requests, heads);
    kernel<<<grid, PREFILL_WARPS * 32, shared, stream>>>(
        (const bf16*)q, (const bf16*)kv, kv_half, block_table, table_width, page_size,
        request_start, history, (bf16*)out, requests, heads, kv_heads, scale * LOG2E, window);
    return 0;
}

size_t decode_shared_bytes(int head_dim) {
    const size_t tiles = (size_t)DECODE_WARPS * DECODE_STAGES * 2 * DECODE_KEYS * (head_dim + 8) * 2;
    const size_t merge = (size_t)DECODE_WARPS * DECODE_HEADS * (head_dim + 2) * 4;
    return tiles > merge ? tiles : merge;
}

template <int HD, bool PREP>
int launch_decode(const void* q, const void* kv, long long kv_half, const int* block_table,
                  int table_width, int page_size, const int* positions, void* out, float* partial,
                  int requests, int heads, int kv_heads, int splits, float scale, int window,
                  cudaStream_t stream, DecodePrep prep = DecodePrep()) {
    using T = Tile<HD>;
    const size_t shared = decode_shared_bytes(HD);
    const int group = heads / kv_heads;
    const dim3 grid(kv_heads * ((group + DECODE_HEADS - 1) / DECODE_HEADS), requests, splits);
    const float scale_log2 = scale * LOG2E;
    // 2 to 8 splits without a scratch buffer: a cluster of the splits' blocks merges them itself
    if (splits > 1 && splits <= 8 && partial == nullptr) {
        auto kernel = attention_decode_kernel<HD, true, PREP>;
        if (shared > 48 * 1024)
            cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        cudaLaunchConfig_t config = {};
        config.gridDim = grid;
        config.blockDim = dim3(DECODE_WARPS * 32);
        config.dynamicSmemBytes = shared;
        config.stream = stream;
        cudaLaunchAttribute attributes[2];
        attributes[0].id = cudaLaunchAttributeClusterDimension;
        attributes[0].val.clusterDim.x = 1;
        attributes[0].val.clusterDim.y = 1;
        attributes[0].val.clusterDim.z = splits;
        attributes[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[1].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attributes;
        config.numAttrs = mlxone_pdl_enabled() ? 2 : 1;
        const cudaError_t err = cudaLaunchKernelEx(
            &config, kernel, (const bf16*)q, (const bf16*)kv, kv_half, block_table, table_width,
            page_size, positions, (bf16*)out, (float*)nullptr, heads, kv_heads, splits, scale_log2,
            window, prep);
        if (err != cudaSuccess) {
            mlxone_set_error("attention_decode: cluster launch failed: %s", cudaGetErrorString(err));
            return 2;
        }
        return 0;
    }
    auto kernel = attention_decode_kernel<HD, false, PREP>;
    if (shared > 48 * 1024)
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    launch_kernel(kernel, grid, dim3(DECODE_WARPS * 32), shared, stream, true, (const bf16*)q,
                  (const bf16*)kv, kv_half, block_table, table_width, page_size, positions,
                  (bf16*)out, partial, heads, kv_heads, splits, scale_log2, window, prep);
    if (splits > 1) {
        const int items = requests * heads;
        launch_kernel(attention_merge_kernel<HD>, dim3((items + 3) / 4), dim3(128), 0, stream, true,
                      (const float*)partial, (bf16*)out, items, splits);
    }
    return 0;
}

}  // namespace

// How many blocks of the decode kernel an SM holds at once (shared memory and warps), which is
// what the caller sizes the number of key splits by.
MLXONE_API int mlxone_attention_decode_resident(int head_dim) {
    const size_t each = decode_shared_bytes(head_dim) + 1024;
    int blocks = (int)((227 * 1024) / each);
    const int by_warps = 64 / DECODE_WARPS;
    if (blocks > by_warps) blocks = by_warps;
    if (blocks > 32) blocks = 32;
    return blocks < 1 ? 1 : blocks;
}

#define MLXONE_HEAD_DIMS(CALL)                                                       \
    switch (head_dim) {                                                              \
        case 16: CALL(16); break;                                                    \
        case 32: CALL(32); break;                                                    \
        case 48: CALL(48); break;                                                    \
        case 64: CALL(64); break;                                                    \
        case 80: CALL(80); break;                                                    \
        case 96: CALL(96); break;                                                    \
        case 112: CALL(112); break;                                                  \
        case 128: CALL(128); break;                                                  \
        default:                                                                     \
            mlxone_set_error("attention (tensor cores): head size %d is not a multiple of " \
                             "16 up to 128", head_dim);                              \
            return 1;                                                                \
    }

// 1 if the tensor-core kernels take this shape, else 0 (the caller then uses the general one).
MLXONE_API int mlxone_attention_mma_supports(int head_dim, int dtype) {
    return dtype == MLXONE_BF16 && head_dim % 16 == 0 && head_dim >= 16 && head_dim <= 128;
}

MLXONE_API int mlxone_attention_prefill(const void* q, const void* kv, const int* block_table,
                                        int table_width, int page_size, int pages,
                                        const int* request_start, const int* history, void* out,
                                        int tokens, int requests, int heads, int kv_heads,
                                        int head_dim, float scale, int window,
                                        cudaStream_t stream) {
    if (tokens == 0) return 0;
    MLXONE_REQUIRE(tokens > 0 && requests > 0 && heads > 0 && kv_heads > 0 &&
                       heads % kv_heads == 0, "attention_prefill: bad sizes");
    MLXONE_REQUIRE(heads <= 65535, "attention_prefill: too many heads");
    MLXONE_REQUIRE(page_size > 0 && pages > 0 && table_width > 0,
                   "attention_prefill: bad page geometry");
    const long long kv_half = (long long)pages * kv_heads * page_size * head_dim;
#define CALL(HD)                                                                              \
    launch_prefill<HD>(q, kv, kv_half, block_table, table_width, page_size, request_start,    \
                       history, out, tokens, requests, heads, kv_heads, scale, window, stream)
    MLXONE_HEAD_DIMS(CALL)
#undef CALL
    MLXONE_LAUNCH_CHECK("attention_prefill");
    return 0;
}

// Floats of scratch that the decode kernel needs for `splits` > 1.
MLXONE_API long long mlxone_attention_decode_scratch(int requests, int heads, int head_dim,
                                                     int splits) {
    return splits > 1 ? (long long)requests * heads * splits * (head_dim + 2) : 0;
}

MLXONE_API int mlxone_attention_decode(const void* q, const void* kv, const int* block_table,
                                       int table_width, int page_size, int pages,
                                       const int* positions, void* out, float* partial,
                                       int requests, int heads, int kv_heads, int head_dim,
                                       int splits, float scale, int window, cudaStream_t stream) {
    if (requests == 0) return 0;
    MLXONE_REQUIRE(requests > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                   "attention_decode: bad sizes");
    MLXONE_REQUIRE(requests <= 65535 && splits >= 1 && splits <= 65535,
                   "attention_decode: at most 65535 requests and splits");
    MLXONE_REQUIRE(splits <= 8 || partial != nullptr,
                   "attention_decode: more than 8 splits need a scratch buffer");
    MLXONE_REQUIRE(page_size > 0 && pages > 0 && table_width > 0,
                   "attention_decode: bad page geometry");
    const long long kv_half = (long long)pages * kv_heads * page_size * head_dim;
#define CALL(HD)                                                                               \
    launch_decode<HD, false>(q, kv, kv_half, block_table, table_width, page_size, positions, out, \
                             partial, requests, heads, kv_heads, splits, scale, window, stream)
    MLXONE_HEAD_DIMS(CALL)
#undef CALL
    MLXONE_LAUNCH_CHECK("attention_decode");
    return 0;
}

// The merge of key splits alone: partial [items, splits, head_dim + 2] (unnormalised output,
// maximum, sum) -> out [items, head_dim] bfloat16. For kernels that leave their splits to it.
MLXONE_API int mlxone_attention_merge(const float* partial, void* out, int items, int splits,
                                      int head_dim, cudaStream_t stream) {
    if (items == 0) return 0;
    MLXONE_REQUIRE(items > 0 && splits >= 1 && partial != nullptr, "attention_merge: bad sizes");
#define CALL(HD)                                                                                  \
    launch_kernel(attention_merge_kernel<HD>, dim3((items + 3) / 4), dim3(128), 0, stream, true, \
                  partial, (bf16*)out, items, splits)
    MLXONE_HEAD_DIMS(CALL)
#undef CALL
    MLXONE_LAUNCH_CHECK("attention_merge");
    return 0;
}

// 1 if mlxone_attention_decode_fused takes this head size: a multiple of 32 up to 128.
MLXONE_API int mlxone_attention_decode_fused_supports(int head_dim) {
    return head_dim % 32 == 0 && head_dim >= 32 && head_dim <= 128 ? 1 : 0;
}

// Decode attention straight from the step's fused projection: qkv [requests, (heads + 2 kv_heads)
// * head_dim] bfloat16, one token per request. Per-head RMSNorm of queries and keys (q_weight,
// k_weight float32 [head_dim], or null for none), rotation of the whole head by positions *
// inv_freq (float32 [head_dim / 2], or null for none), the token's key and value written into
// its page (write_kv), attention over the request's pages: what mlxone_qk_prep followed by
// mlxone_attention_decode compute, in one kernel. kv is the writable cache.
MLXONE_API int mlxone_attention_decode_fused(const void* qkv, const float* q_weight,
                                             const float* k_weight, float eps,
                                             const float* inv_freq, void* kv,
                                             const int* block_table, int table_width,
                                             int page_size, int pages, const int* positions,
                                             void* out, float* partial, int requests, int heads,
                                             int kv_heads, int head_dim, int splits, float scale,
                                             int window, int write_kv, int* error_flag,
                                             cudaStream_t stream) {
    if (requests == 0) return 0;
    MLXONE_REQUIRE(mlxone_attention_decode_fused_supports(head_dim),
                   "attention_decode_fused: head size %d is no multiple of 32 up to 128", head_dim);
    MLXONE_REQUIRE(requests > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                   "attention_decode_fused: bad sizes");
    MLXONE_REQUIRE(requests <= 65535 && splits >= 1 && splits <= 65535,
                   "attention_decode_fused: at most 65535 requests and splits");
    MLXONE_REQUIRE(splits <= 8 || partial != nullptr,
                   "attention_decode_fused: more than 8 splits need a scratch buffer");
    MLXONE_REQUIRE(page_size > 0 && pages > 0 && table_width > 0,
                   "attention_decode_fused: bad page geometry");
    const long long kv_half = (long long)pages * kv_heads * page_size * head_dim;
    DecodePrep prep;
    prep.q_weight = q_weight; prep.k_weight = k_weight; prep.eps = eps; prep.inv_freq = inv_freq;
    prep.cache = static_cast<bf16*>(kv); prep.write_kv = write_kv; prep.error_flag = error_flag;
    int code = 0;
    switch (head_dim) {
#define CASE(HD)                                                                                  \
        case HD:                                                                                  \
            code = launch_decode<HD, true>(qkv, kv, kv_half, block_table, table_width, page_size, \
                                           positions, out, partial, requests, heads, kv_heads,    \
                                           splits, scale, window, stream, prep);                  \
            break;
        CASE(32) CASE(64) CASE(96) CASE(128)
#undef CASE
        default: break;
    }
    if (code != 0) return code;
    MLXONE_LAUNCH_CHECK("attention_decode_fused");
    return 0;
}

// ------------------------------------------------------------------ no-allocation variant
#include "attention_decode_static.h"

// The partial results of the key splits for callers that cannot allocate (see the header).
// In host code this name is only a handle of the symbol, not a device address: the address
// that kernels may use comes from cudaGetSymbolAddress, per device.
static __device__ __align__(256) float g_static_scratch[MLXONE_STATIC_SCRATCH_FLOATS];

namespace {
// Device addresses of the array, looked up once per device. Threads may race to fill an entry;
// they all store the same value, and the store and load are atomic, so any of them may win.
constexpr int MAX_DEVICES = 64;
float* g_static_scratch_address[MAX_DEVICES] = {};
}  // namespace

MLXONE_API long long mlxone_attention_decode_static_capacity() {
    return MLXONE_STATIC_SCRATCH_FLOATS;
}

MLXONE_API int mlxone_attention_decode_static(const void* q, const void* kv, const int* block_table,
                                              int table_width, int page_size, int pages,
                                              const int* positions, void* out, int requests,
                                              int heads, int kv_heads, int head_dim, int splits,
                                              float scale, int window, cudaStream_t stream) {
    if (requests == 0) return 0;
    MLXONE_REQUIRE(requests > 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0,
                   "attention_decode_static: bad sizes");
    MLXONE_REQUIRE(splits >= 1 && splits <= 65535 && requests <= 65535,
                   "attention_decode_static: at most 65535 requests and splits");
    const long long needed = mlxone_attention_decode_scratch(requests, heads, head_dim, splits);
    MLXONE_REQUIRE(needed <= MLXONE_STATIC_SCRATCH_FLOATS,
                   "attention_decode_static: %d requests x %d heads x %d splits need %lld floats of "
                   "scratch, the fixed array holds %d; use fewer splits or requests per call",
                   requests, heads, splits, needed, MLXONE_STATIC_SCRATCH_FLOATS);
    int device = -1;
    cudaError_t err = cudaGetDevice(&device);
    MLXONE_REQUIRE(err == cudaSuccess && device >= 0,
                   "attention_decode_static: no current device (%s)", cudaGetErrorString(err));
    MLXONE_REQUIRE(device < MAX_DEVICES,
                   "attention_decode_static: device %d; this entry point serves devices 0 to %d",
                   device, MAX_DEVICES - 1);
    float* address = __atomic_load_n(&g_static_scratch_address[device], __ATOMIC_ACQUIRE);
    if (address == nullptr) {
        // once per device, with that device current; not inside a stream capture, where the
        // look-up (which may load the library's device image) is not allowed
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        err = cudaStreamIsCapturing(stream, &capturing);
        MLXONE_REQUIRE(err == cudaSuccess && capturing == cudaStreamCaptureStatusNone,
                       "attention_decode_static: the first call on device %d came inside a stream "
                       "capture; make one call on this device before capturing", device);
        err = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_static_scratch);
        MLXONE_REQUIRE(err == cudaSuccess && address != nullptr,
                       "attention_decode_static: cannot find the scratch array on device %d: %s",
                       device, cudaGetErrorString(err));
        __atomic_store_n(&g_static_scratch_address[device], address, __ATOMIC_RELEASE);
    }
    return mlxone_attention_decode(q, kv, block_table, table_width, page_size, pages, positions,
                                   out, address, requests, heads, kv_heads, head_dim, splits, scale,
                                   window, stream);
}
