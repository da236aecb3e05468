// Matrix products with few rows (decode steps): out[M, N] = a[M, K] * w[N, K]^T, M <= 32,
// bfloat16 operands, 32-bit accumulation. Such a product takes as long as reading w once
// takes, so the kernel is built around streaming w without a pause:
//
//   * persistent blocks, one per SM; a block owns a contiguous range of rows of w (outputs for
//     every token) over the whole K, so no two blocks add into the same output and results do
//     not depend on scheduling. A block walks its range in tiles of 16 rows: whole tiles when
//     there is at least one for every block, else ranges equal to within one row (so that all
//     SMs stream), whose last tile is partly masked (masked rows are neither read nor written);
//   * the block's warps take the 64-wide slices of K of the current tile in turn; every warp
//     copies its slices of w asynchronously through a ring of its own in shared memory, and the
//     ring runs on into the next tile, so the stream never drains inside the kernel;
//   * slices are multiplied on tensor cores (mma m16n8k16: w is the 16-row operand, eight
//     tokens the 8-column one); per tile the warps' partial sums are added in shared memory by
//     all threads, in a fixed tree that is the same for every number of tokens;
//   * the copies of the first slices are issued before the kernel waits for its predecessor
//     (griddep_wait), so weights already stream while the previous kernel finishes;
//   * the activations are read after that wait: into shared memory once per block when the
//     block has several tiles and they fit (as they are, or as the RMSNorm of 32-bit rows, which
//     the kernel then computes itself); else, up to 8 tokens, through the rings beside the
//     weights; else from L2 slice by slice, two slices ahead.
//
// Within a 32-wide piece of K, thread t of a quad reads elements 8t..8t+7 of both operands
// with one 16-byte load and feeds them to two mma instructions; the sum over K does not care
// in which order the products are taken.
//
// Epilogues: store bfloat16 (+ bias); SwiGLU (the block also owns the 16 matching rows of the
// "up" half and writes silu(gate) * up); add into the 32-bit residual stream (red.global.add, one
// addition per address); store float32;
// gated short convolution of a decode step (w = [B rows; C rows; x rows], the block owns the same
// channels of all three and applies the convolution's single-token update, so that neither the
// three projections nor a second kernel touch memory).
#include "common.cuh"

namespace {

using bf16 = __nv_bfloat16;
constexpr int ROWS = 16;          // rows of w per tile
constexpr int SLICE = 64;         // K elements per slice
constexpr int STAGES = 4;         // ring of slices per warp
constexpr int SLICE_BYTES = ROWS * SLICE * 2;
constexpr int WARPS = 16;
constexpr size_t SHARED_LIMIT = 226 * 1024;      // of the 227 KB that a block may ask for

enum : int { STORE_BF16 = 0, SWIGLU = 1, ADD_RESIDUAL = 2, STORE_F32 = 3, GATED_CONV = 4 };

// What the gated-convolution epilogue needs beside the product: one token per request.
struct ConvUpdate {
    const float* kernel = nullptr;     // [channels, taps]
    const float* bias = nullptr;       // [channels] or null
    bf16* state = nullptr;             // [slots, taps - 1, channels]: the last values of B * x
    const int* slots = nullptr;        // per request
    const int* history = nullptr;      // per request: tokens before this one
    int taps = 1;                      // 1..4
    int write_state = 0;
};

__device__ __forceinline__ uint32_t shared_address(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void copy16(uint32_t dst, const void* src, bool live) {
    const int bytes = live ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void copy_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void copy_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// A 16-byte load that is served by L2: the activations were written by the kernel before this
// one, which may still have been running when this block started, so neither the read-only
// path nor a line left in L1 may be used.
__device__ __forceinline__ uint4 load_l2(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// NT: groups of 8 tokens (M <= 8 * NT). RESIDENT: activations live in shared memory.
// NORM (needs RESIDENT): the activations are RMSNorm(source) * norm_weight, computed here from the
// 32-bit rows of `source` while they are brought into shared memory, so the norm needs no
// kernel and no pass over memory of its own.
template <int NT, int EPILOGUE, bool RESIDENT, bool NORM>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const bf16* a, int lda, const bf16* __restrict__ w,
                   const float* __restrict__ bias, void* out, int ldo, int m, int n, int k,
                   int up_offset, const float* source, int source_ld,
                   const float* __restrict__ norm_weight, float eps, ConvUpdate conv,
                   int share_base, int share_extra) {
    // A SwiGLU block splits its warps in two halves: the first on 16 gate rows, the second on
    // the 16 matching up rows (measured faster than tiles of 8 + 8 rows, which balance better
    // but pay the per-tile reduction twice as often).
    constexpr int HALVES = EPILOGUE == SWIGLU ? 2 : 1;
    constexpr int WARPS_K = WARPS / HALVES;
    constexpr int TOKENS = 8 * NT;
    // With up to 8 tokens and no room to keep all activations in shared memory, each slice of
    // activations (8 tokens x 64) travels through the ring beside its slice of w.
    constexpr bool TOKEN_RING = !RESIDENT && NT == 1;
    constexpr int SLOT_BYTES = SLICE_BYTES + (TOKEN_RING ? 8 * SLICE * 2 : 0);
    extern __shared__ __align__(128) unsigned char shared_bytes[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int half = warp / WARPS_K, wk = warp % WARPS_K;
    const int g = lane >> 2, t = lane & 3;
    unsigned char* ring = shared_bytes + (size_t)warp * STAGES * SLOT_BYTES;
    const uint32_t ring_address = shared_address(ring);
    // (gated convolution: every group of 16 channels is three tiles: B, C, x)
    constexpr int PARTS = EPILOGUE == GATED_CONV ? 3 : 1;
    // Gated convolution with up to 8 tokens and the activations in shared memory: the three
    // tiles of a group of channels (B, C, x) leave their partial sums in sections of their own
    // and are added up together after the third, one barrier a group instead of one a tile.
    // (With 16 tokens, or rows too long for shared memory, the sections do not fit; each tile is
    // then added up by itself. Three tiles of output rows a barrier, for the other epilogues,
    // was measured too: slower, 0.6546 against 0.6460 ms a decode step; the last run's three
    // reductions and stores stand at the kernel's end.)
    constexpr bool GROUPED = EPILOGUE == GATED_CONV && NT == 1 && RESIDENT;
    constexpr int SECTIONS = GROUPED ? PARTS : 1;
    // two sets of partial sums, used in turn, so that one block-wide barrier per tile is enough
    float* sums_base = reinterpret_cast<float*>(shared_bytes + (size_t)WARPS * STAGES * SLOT_BYTES);
    unsigned char* resident =
        reinterpret_cast<unsigned char*>(sums_base + 2 * SECTIONS * WARPS * ROWS * TOKENS);

    // this block's rows (of the gate half for SwiGLU) and the tiles that cover them
    // (gated convolution: channels; every group of 16 channels is three tiles: B, C, x)
    const int columns = EPILOGUE == SWIGLU ? up_offset : n / PARTS;
    // With at least a tile for every block, blocks take whole tiles (some one more than others:
    // a tile's fixed cost weighs more than the imbalance); with fewer, the rows are spread to
    // within one row, so that every SM streams.
    // (The shares come from the host as quotient and remainder of tiles, or rows, by blocks: the
    // first `share_extra` blocks take one more. A division here would stand between the
    // kernel's start and its first copy, in every one of a step's products.)
    const int whole_tiles = (columns + ROWS - 1) / ROWS;
    const bool by_tiles = whole_tiles >= (int)gridDim.x;
    const int share_begin = (int)blockIdx.x * share_base + min((int)blockIdx.x, share_extra);
    const int share_end = share_begin + share_base + ((int)blockIdx.x < share_extra ? 1 : 0);
    const int row_begin = by_tiles ? ROWS * share_begin : share_begin;
    const int row_end = by_tiles ? min(columns, ROWS * share_end) : share_end;
    const int tile_count = PARTS * ((row_end - row_begin + ROWS - 1) / ROWS);
    const int slices = (k + SLICE - 1) / SLICE;
    const int mine = slices > wk ? (slices - wk + WARPS_K - 1) / WARPS_K : 0;   // per tile
    const int total = mine * tile_count;                  // this warp's slices over all tiles

    // Copies the next slice of this warp's stream into its ring: 16 rows x 8 pieces of 16 B;
    // piece c of row r is stored at piece c ^ ((r & 1) << 2), which keeps the 16-byte reads of a
    // quarter warp on different banks. A lane copies piece c = lane % 8 of the rows lane / 8,
    // + 4, + 8, + 12. The kernel's time is the number of instructions that a warp issues (four
    // warps a scheduler, each waiting on its own copies), so the walk keeps a pointer and adds
    // to it instead of working the address out for every slice, and a slice that lies inside
    // K and a row that lies inside the block's range are the cases without a test.
    static_assert((STAGES & (STAGES - 1)) == 0, "the ring size must be a power of two");
    const int piece_row = lane >> 3, piece_k = (lane & 7) * 8;
    const uint32_t piece_dst = ring_address + piece_row * 128 + (((lane & 7) ^ ((piece_row & 1) << 2)) << 4);
    const size_t slice_step = (size_t)WARPS_K * SLICE;         // elements between a warp's slices
    const size_t four_rows = (size_t)4 * k;
    int fetch_tile = 0, fetch_slice = 0, fetched = 0;
    const bf16* fetch_from = w;       // piece (piece_row, piece_k) of the next slice
    int fetch_k0 = 0, fetch_rows = 0; // its K offset; rows of its tile from piece_row on
    auto fetch_position = [&]() {     // at the first slice of `fetch_tile`
        const int row0 = row_begin + (fetch_tile / PARTS) * ROWS;
        fetch_k0 = wk * SLICE;
        fetch_rows = row_end - row0 - piece_row;
        fetch_from = w + (size_t)(row0 + half * up_offset + (fetch_tile % PARTS) * columns + piece_row) * k +
                     fetch_k0 + piece_k;
    };
    fetch_position();
    auto fetch = [&]() {
        const uint32_t to = piece_dst + (fetched & (STAGES - 1)) * SLOT_BYTES;
        if (fetch_k0 + SLICE <= k) {
            // rows beyond the block's range are not copied: what the ring holds there only
            // reaches sums that are never stored
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (4 * i < fetch_rows) copy16(to + i * 4 * 128, fetch_from + i * four_rows, true);
        } else {                                       // K ends inside the slice: zeros beyond it
            const bool inside = fetch_k0 + piece_k < k;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bool live = inside && 4 * i < fetch_rows;
                copy16(to + i * 4 * 128, live ? fetch_from + i * four_rows : w, live);
            }
        }
        ++fetched;
        if (++fetch_slice == mine) {
            fetch_slice = 0;
            ++fetch_tile;
            fetch_position();
        } else {
            fetch_from += slice_step;
            fetch_k0 += (int)slice_step;
        }
    };
    // the activations of the next slice of the stream (TOKEN_RING): 8 tokens x 8 pieces, a lane
    // piece lane % 8 of the tokens lane / 8 and lane / 8 + 4
    int token_slice = 0, tokens_fetched = 0;
    const bf16* const tokens_first = a + (size_t)piece_row * lda + wk * SLICE + piece_k;
    const bf16* tokens_from = tokens_first;
    int tokens_k0 = wk * SLICE;
    const uint32_t tokens_dst = piece_dst + SLICE_BYTES;
    const size_t four_tokens = (size_t)4 * lda;
    auto fetch_tokens = [&]() {
        const uint32_t to = tokens_dst + (tokens_fetched & (STAGES - 1)) * SLOT_BYTES;
        const bool inside = tokens_k0 + piece_k < k;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const bool live = inside && piece_row + 4 * i < m;
            copy16(to + i * 4 * 128, live ? tokens_from + i * four_tokens : a, live);
        }
        ++tokens_fetched;
        if (++token_slice == mine) {
            token_slice = 0;
            tokens_from = tokens_first;
            tokens_k0 = wk * SLICE;
        } else {
            tokens_from += slice_step;
            tokens_k0 += (int)slice_step;
        }
    };

#pragma unroll
    for (int p = 0; p < STAGES - 1; ++p) {
        if (p < total) fetch();
        copy_commit();
    }
    // NORM: the norm's weights do not depend on the kernel before this one either. They wait in
    // the space of the partial sums (unused until the first tile ends), behind the few floats
    // through which the warps of a token exchange their sums of squares.
    float* norm_exchange = sums_base;
    float* norm_scale = sums_base + 64;
    if (RESIDENT && NORM) {
        for (int c = threadIdx.x; c * 4 < k; c += WARPS * 32)
            copy16(shared_address(norm_scale + c * 4), norm_weight + c * 4, true);
        copy_commit();
    }
    griddep_launch();
    griddep_wait();            // from here on the predecessor's results may be read

    // resident activations: [token][K] with 16-byte pieces swizzled by the token's parity
    const int resident_stride = ((k + 63) / 64) * 64 * 2;        // bytes per token
    if (RESIDENT && NORM) {
        // All warps: SHARERS warps a token, each a contiguous share of the row. A lane keeps
        // its first HELD pieces (of 8 values) in registers between the sum of squares and the
        // scaling, so that a row of up to SHARERS * 32 * HELD * 8 values crosses from L2 once
        // (longer rows are read again for the scaling); all of a lane's loads are in flight
        // together. The block reads TOKENS rows of 32-bit values where the plain kernel reads
        // 16-bit ones, which is what the norm costs here: no kernel of its own, no pass over
        // memory for its result.
        constexpr int HELD = 4;
        constexpr int SHARERS = WARPS / TOKENS > 0 ? WARPS / TOKENS : 1;
        static_assert(!NORM || TOKENS <= WARPS, "a warp per token at least");
        const int pieces = resident_stride / 16;
        const int share = (pieces + SHARERS - 1) / SHARERS;          // pieces of a warp
        const int token = warp / SHARERS, sharer = warp % SHARERS;
        const int first_piece = sharer * share;
        const int end_piece = min(first_piece + share, pieces);
        unsigned char* row_out = resident + token * resident_stride;
        const float* row = source + (size_t)token * source_ld;
        auto squares = [](const uint4& a0, const uint4& a1) {
            const float v[8] = {__uint_as_float(a0.x), __uint_as_float(a0.y), __uint_as_float(a0.z),
                                __uint_as_float(a0.w), __uint_as_float(a1.x), __uint_as_float(a1.y),
                                __uint_as_float(a1.z), __uint_as_float(a1.w)};
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) sum += v[i] * v[i];
            return sum;
        };
        uint4 lo[HELD], hi[HELD];
        float sum = 0.f;
        if (token < m) {
#pragma unroll
            for (int j = 0; j < HELD; ++j) {
                const int c = first_piece + lane + 32 * j;
                if (c < end_piece && c * 8 < k) {
                    lo[j] = load_l2(row + c * 8);
                    hi[j] = load_l2(row + c * 8 + 4);
                } else {
                    lo[j] = hi[j] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (int j = 0; j < HELD; ++j) sum += squares(lo[j], hi[j]);
            for (int c = first_piece + lane + 32 * HELD; c < end_piece && c * 8 < k; c += 32)
                sum += squares(load_l2(row + c * 8), load_l2(row + c * 8 + 4));
        }
        sum = warp_sum(sum);
        if (lane == 0) norm_exchange[token * SHARERS + sharer] = sum;
        copy_wait<0>();        // the norm's weights (and the ring's first slices) have landed
        __syncthreads();
        float total = 0.f;
#pragma unroll
        for (int i = 0; i < SHARERS; ++i) total += norm_exchange[token * SHARERS + i];
        const float inv = rsqrtf(total / (float)k + eps);
        auto scaled = [&](const uint4& a0, const uint4& a1, int c) {
            const float4 w0 = *reinterpret_cast<const float4*>(norm_scale + c * 8);
            const float4 w1 = *reinterpret_cast<const float4*>(norm_scale + c * 8 + 4);
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(a0.x) * inv * w0.x,
                                                      __uint_as_float(a0.y) * inv * w0.y);
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(a0.z) * inv * w0.z,
                                                      __uint_as_float(a0.w) * inv * w0.w);
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(a1.x) * inv * w1.x,
                                                      __uint_as_float(a1.y) * inv * w1.y);
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(a1.z) * inv * w1.z,
                                                      __uint_as_float(a1.w) * inv * w1.w);
            uint4 packed;
            packed.x = *reinterpret_cast<uint32_t*>(&p0);
            packed.y = *reinterpret_cast<uint32_t*>(&p1);
            packed.z = *reinterpret_cast<uint32_t*>(&p2);
            packed.w = *reinterpret_cast<uint32_t*>(&p3);
            return packed;
        };
        if (token < TOKENS) {
#pragma unroll
            for (int j = 0; j < HELD; ++j) {
                const int c = first_piece + lane + 32 * j;
                if (c < end_piece) {
                    const uint4 packed = (token < m && c * 8 < k) ? scaled(lo[j], hi[j], c)
                                                                  : make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<uint4*>(row_out + ((c ^ ((token & 1) << 2)) << 4)) = packed;
                }
            }
            for (int c = first_piece + lane + 32 * HELD; c < end_piece; c += 32) {
                uint4 packed = make_uint4(0u, 0u, 0u, 0u);
                if (token < m && c * 8 < k)
                    packed = scaled(load_l2(row + c * 8), load_l2(row + c * 8 + 4), c);
                *reinterpret_cast<uint4*>(row_out + ((c ^ ((token & 1) << 2)) << 4)) = packed;
            }
        }
        __syncthreads();
    } else if (RESIDENT) {
        const int pieces = resident_stride / 16;
        for (int token = warp; token < TOKENS; token += WARPS) {       // a warp a token
            const uint32_t row_to = shared_address(resident) + token * resident_stride;
            const bf16* row_from = a + (size_t)token * lda;
            for (int c = lane; c < pieces; c += 32) {
                const bool live = token < m && c * 8 < k;
                copy16(row_to + ((c ^ ((token & 1) << 2)) << 4), live ? row_from + c * 8 : a, live);
            }
        }
        copy_commit();
        copy_wait<0>();        // also completes the ring's first slices; they are needed at once
        __syncthreads();
    }

    // activations of the slice at K offset k0: [piece of 32][token group] -> 16 bytes
    // (resident: a slice is 128 bytes of a token's row, which the swizzle stays inside, so the
    // lane's place within a slice is worked out once)
    const unsigned char* resident_lane[2];
#pragma unroll
    for (int q = 0; q < 2; ++q)
        resident_lane[q] = resident + g * resident_stride + (((q * 4 + t) ^ ((g & 1) << 2)) << 4);
    const bf16* const tokens_lane = a + (size_t)g * lda + t * 8;
    auto load_tokens = [&](int k0, uint4 (&regs)[2][NT]) {
#pragma unroll
        for (int q = 0; q < 2; ++q)
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                if (RESIDENT) {
                    regs[q][nt] = *reinterpret_cast<const uint4*>(
                        resident_lane[q] + nt * 8 * resident_stride + k0 * 2);
                } else {
                    const int token = nt * 8 + g, kk = k0 + q * 32 + t * 8;
                    regs[q][nt] = (token < m && kk < k)
                                      ? load_l2(tokens_lane + (size_t)nt * 8 * lda + kk - t * 8)
                                      : make_uint4(0u, 0u, 0u, 0u);
                }
            }
    };

    float acc[NT][4];
    uint4 tokens_now[2][NT], tokens_next[2][NT], tokens_after[2][NT];
    if (TOKEN_RING) {
        // the activations of the slices whose weights are already on their way, then all of it
        // has to land once; from here on a slice's weights and activations travel together
#pragma unroll
        for (int p = 0; p < STAGES - 1; ++p)
            if (p < total) fetch_tokens();
        copy_commit();
        copy_wait<0>();
        __syncwarp();
    } else if (!RESIDENT && total > 0) {
        // the activations come from L2 two slices ahead (see the slice loop)
        load_tokens(wk * SLICE, tokens_now);
        if (total > 1) load_tokens((wk + (mine > 1 ? 1 : 0) * WARPS_K) * SLICE, tokens_next);
    }
    int next_slice = 2 % max(mine, 1);       // the slice (within a tile) whose tokens are fetched next

    // The sum that this thread finishes after every tile (see below): row `r` of the tile for
    // token `token`, a share of it.
    constexpr int SPLIT = WARPS * 32 / (ROWS * TOKENS);       // threads a sum: 4, 2 or 1
    const int item = threadIdx.x / SPLIT, share = threadIdx.x % SPLIT;
    const int token = item / ROWS, r = item % ROWS;           // rows fastest: neighbours in memory
    const bool owner = share == 0 && token < m;

    // Gated convolution: this thread's B and C, and what its update reads beside the product.
    // Those loads are issued before the group's slices are multiplied, not after: three global
    // round trips in a row at the kernel's end would cost more than the product's stream.
    float held_b = 0.f, held_c = 0.f;
    int conv_position = 0;
    bf16* conv_rows = nullptr;
    float conv_kept[3] = {0.f, 0.f, 0.f}, conv_weight[4] = {0.f, 0.f, 0.f, 0.f}, conv_bias_value = 0.f;
    if (EPILOGUE == GATED_CONV && owner) {
        conv_position = conv.history[token];
        conv_rows = conv.state + (size_t)conv.slots[token] * (conv.taps - 1) * columns;
    }
    int index = 0;
    for (int tile = 0; tile < tile_count; ++tile) {
        if (EPILOGUE == GATED_CONV && tile % PARTS == 0) {
            const int column = row_begin + (tile / PARTS) * ROWS + r;
            if (owner && column < row_end) {
                conv_bias_value = conv.bias != nullptr ? conv.bias[column] : 0.f;
#pragma unroll
                for (int s = 0; s < 4; ++s)
                    if (s < conv.taps) conv_weight[s] = conv.kernel[(size_t)column * conv.taps + s];
#pragma unroll
                for (int s = 0; s < 3; ++s)
                    if (s < conv.taps - 1)     // state row s holds position - (taps - 1) + s; zero before the start
                        conv_kept[s] = conv_position - (conv.taps - 1) + s >= 0
                                           ? __bfloat162float(conv_rows[(size_t)s * columns + column]) : 0.f;
            }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[nt][c] = 0.f;

        // One slice of the stream: `now` holds its activations; without a copy in shared
        // memory, `next` is loaded for the slice after it.
        auto consume = [&](int i, uint4 (&now)[2][NT], uint4 (&next)[2][NT]) {
            copy_wait<STAGES - 2>();
            __syncwarp();
            if (fetched < total) {
                fetch();
                if (TOKEN_RING) fetch_tokens();
            }
            copy_commit();
            const unsigned char* slice = ring + (index & (STAGES - 1)) * SLOT_BYTES;
            if (RESIDENT) {
                load_tokens((wk + i * WARPS_K) * SLICE, now);
            } else if (TOKEN_RING) {
#pragma unroll
                for (int q = 0; q < 2; ++q)
                    now[q][0] = *reinterpret_cast<const uint4*>(
                        slice + SLICE_BYTES + g * 128 + (((q * 4 + t) ^ ((g & 1) << 2)) << 4));
            } else if (index + 2 < total) {
                load_tokens((wk + next_slice * WARPS_K) * SLICE, next);
                if (++next_slice == mine) next_slice = 0;
            }
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                const int c = q * 4 + t;
                const uint4 lo = *reinterpret_cast<const uint4*>(
                    slice + g * 128 + ((c ^ ((g & 1) << 2)) << 4));
                const uint4 hi = *reinterpret_cast<const uint4*>(
                    slice + (g + 8) * 128 + ((c ^ ((g & 1) << 2)) << 4));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    mma_16816(acc[nt], lo.x, hi.x, lo.y, hi.y, now[q][nt].x, now[q][nt].y);
                    mma_16816(acc[nt], lo.z, hi.z, lo.w, hi.w, now[q][nt].z, now[q][nt].w);
                }
            }
            ++index;
        };
        if (RESIDENT || TOKEN_RING) {
            for (int i = 0; i < mine; ++i) consume(i, tokens_now, tokens_next);
        } else {
            // The activations come from L2 two slices ahead, through three sets of registers
            // that change roles: a set is first read two slices after its loads were issued, which
            // is longer than a trip to L2 takes while the weights stream. Three slices a turn;
            // what is left of a tile pays one or two moves between the sets (a move waits for
            // its loads, so it is kept out of the turns).
            auto move = [&](uint4 (&to)[2][NT], const uint4 (&from)[2][NT]) {
#pragma unroll
                for (int q = 0; q < 2; ++q)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt) to[q][nt] = from[q][nt];
            };
            int i = 0;
            for (; i + 2 < mine; i += 3) {
                consume(i, tokens_now, tokens_after);
                consume(i + 1, tokens_next, tokens_now);
                consume(i + 2, tokens_after, tokens_next);
            }
            if (mine - i == 1) {
                // used now, loaded after: next and after hold the two slices to come
                consume(i, tokens_now, tokens_after);
                move(tokens_now, tokens_next);
                move(tokens_next, tokens_after);
            } else if (mine - i == 2) {
                // used now and next, loaded after and now: after and now hold the slices to come
                consume(i, tokens_now, tokens_after);
                consume(i + 1, tokens_next, tokens_now);
                move(tokens_next, tokens_now);
                move(tokens_now, tokens_after);
            }
        }

        // Partial sums of this tile: [warp][token][row 0..15]. Every thread of the block adds a
        // share of one sum (SPLIT threads a sum, neighbours in a warp, each SHARE warps' parts),
        // then the shares meet by shuffles. So that a warp's loads fall on 32 different banks, the
        // rows of every second pair of tokens are stored with halves swapped, and a warp's whole
        // set is turned (its index XOR a multiple of 8 or 16) by the share that will read it.
        constexpr int SHARE = WARPS_K / SPLIT;
        constexpr int TURN = SPLIT == 4 ? 8 : 16;
        static_assert(SPLIT >= 1 && SHARE >= 1 && SPLIT * ROWS * TOKENS == WARPS * 32,
                      "one share of one sum for every thread");
        // (GROUPED: the group's set, this tile's section of it)
        const int set = GROUPED ? (tile / PARTS) & 1 : tile & 1;
        const int section = GROUPED ? tile % PARTS : 0;
        float* sums = sums_base + (size_t)set * SECTIONS * WARPS * ROWS * TOKENS;
        float* mine_sums = sums + (size_t)(section * WARPS + warp) * ROWS * TOKENS;
        auto place = [](int token, int r) { return token * ROWS + (r ^ (((token >> 1) & 1) << 3)); };
        const int my_turn = (wk / SHARE) * TURN;
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            mine_sums[place(nt * 8 + 2 * t, g) ^ my_turn] = acc[nt][0];
            mine_sums[place(nt * 8 + 2 * t + 1, g) ^ my_turn] = acc[nt][1];
            mine_sums[place(nt * 8 + 2 * t, g + 8) ^ my_turn] = acc[nt][2];
            mine_sums[place(nt * 8 + 2 * t + 1, g + 8) ^ my_turn] = acc[nt][3];
        }
        if (GROUPED && section != PARTS - 1) continue;       // the group's last tile adds all three up
        __syncthreads();
        const int column = row_begin + (tile / PARTS) * ROWS + r;
        const float* my_share = sums + (size_t)share * SHARE * ROWS * TOKENS + (place(token, r) ^ (share * TURN));
        // The order of the additions is the same for every number of tokens, so that a token's
        // result does not depend on how many others the call has: the warps' parts in four
        // groups, each added up in turn, then (group 0 + group 1) + (group 2 + group 3). A
        // thread adds 4 / SPLIT of the groups, the shuffles finish the tree.
        constexpr int LEAF = WARPS_K / 4, GROUPS = 4 / SPLIT;
        auto shares_sum = [&](const float* from) {
            float group[GROUPS];
#pragma unroll
            for (int j = 0; j < GROUPS; ++j) {
                group[j] = 0.f;
#pragma unroll
                for (int wi = 0; wi < LEAF; ++wi)
                    group[j] += from[(size_t)(j * LEAF + wi) * ROWS * TOKENS];
            }
            if (GROUPS == 4) return (group[0] + group[1]) + (group[2] + group[GROUPS - 1]);
            if (GROUPS == 2) return group[0] + group[GROUPS - 1];
            return group[0];
        };
        float value = shares_sum(my_share + (size_t)(GROUPED ? PARTS - 1 : 0) * WARPS * ROWS * TOKENS);
        float up = 0.f, first = 0.f, second = 0.f;          // SwiGLU's up; GROUPED: B and C
        if (EPILOGUE == SWIGLU) up = shares_sum(my_share + (size_t)WARPS_K * ROWS * TOKENS);
        if (GROUPED) {
            first = shares_sum(my_share);
            second = shares_sum(my_share + (size_t)WARPS * ROWS * TOKENS);
        }
#pragma unroll
        for (int across = 1; across < SPLIT; across <<= 1) {
            value += __shfl_xor_sync(0xffffffffu, value, across);
            if (EPILOGUE == SWIGLU) up += __shfl_xor_sync(0xffffffffu, up, across);
            if (GROUPED) {
                first += __shfl_xor_sync(0xffffffffu, first, across);
                second += __shfl_xor_sync(0xffffffffu, second, across);
            }
        }
        if (owner && column < row_end) {
            if (bias != nullptr) value += bias[(tile % PARTS) * columns + column];
            if (GROUPED) {
                // the three projections are rounded as if they had been stored
                if (bias != nullptr) { first += bias[column]; second += bias[columns + column]; }
                held_b = __bfloat162float(__float2bfloat16_rn(first));
                held_c = __bfloat162float(__float2bfloat16_rn(second));
            }
            if (EPILOGUE == GATED_CONV) {
                // the three projections are rounded as if they had been stored; a block has one
                // item per thread at most, so B and C wait in registers for x
                value = __bfloat162float(__float2bfloat16_rn(value));
                const int part = tile % PARTS;
                if (part == 0) {
                    held_b = value;
                } else if (part == 1) {
                    held_c = value;
                } else {
                    const float now = __bfloat162float(__float2bfloat16_rn(held_b * value));
                    float y = conv_bias_value;
#pragma unroll
                    for (int s = 0; s < 3; ++s)
                        if (s < conv.taps - 1) y = fmaf(conv_weight[s], conv_kept[s], y);
                    float last_weight = conv_weight[0];
#pragma unroll
                    for (int s = 1; s < 4; ++s)
                        if (s == conv.taps - 1) last_weight = conv_weight[s];
                    y = fmaf(last_weight, now, y);
                    reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] =
                        __float2bfloat16_rn(held_c * y);
                    if (conv.write_state) {
#pragma unroll
                        for (int s = 0; s < 2; ++s)
                            if (s + 1 < conv.taps - 1)
                                conv_rows[(size_t)s * columns + column] = __float2bfloat16_rn(conv_kept[s + 1]);
                        if (conv.taps > 1)
                            conv_rows[(size_t)(conv.taps - 2) * columns + column] = __float2bfloat16_rn(now);
                    }
                }
            } else if (EPILOGUE == SWIGLU) {
                if (bias != nullptr) up += bias[up_offset + column];
                reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] =
                    __float2bfloat16_rn(value / (1.f + expf(-value)) * up);
            } else if (EPILOGUE == STORE_BF16) {
                reinterpret_cast<bf16*>(out)[(size_t)token * ldo + column] =
                    __float2bfloat16_rn(value);
            } else if (EPILOGUE == ADD_RESIDUAL) {
                // added where the value lives (one addition per address, so the result is the
                // same): the thread does not wait for the old value to come and go
                atomicAdd(reinterpret_cast<float*>(out) + (size_t)token * ldo + column, value);
            } else {
                reinterpret_cast<float*>(out)[(size_t)token * ldo + column] = value;
            }
        }
        // no second barrier: the next tile writes the other set of sums, and the one after it
        // comes after the next tile's barrier, which every thread reaches only after this loop
    }
    copy_wait<0>();
}

int g_sm_count = 0;

struct NormInput {
    const float* source = nullptr;
    int ld = 0;
    const float* weight = nullptr;
    float eps = 0.f;
};

template <int NT, int EPILOGUE>
cudaError_t launch(const void* a, int lda, const void* w, const float* bias, void* out, int ldo,
                   int m, int n, int k, int up_offset, cudaStream_t stream,
                   NormInput norm = NormInput(), ConvUpdate conv = ConvUpdate()) {
    if (g_sm_count == 0) {
        int device = 0;
        cudaGetDevice(&device);
        cudaDeviceGetAttribute(&g_sm_count, cudaDevAttrMultiProcessorCount, device);
        if (g_sm_count <= 0) g_sm_count = 148;
    }
    constexpr int PARTS = EPILOGUE == GATED_CONV ? 3 : 1;
    const int columns = EPILOGUE == SWIGLU ? up_offset : n / PARTS;
    const int grid = columns < g_sm_count ? columns : g_sm_count;
    const int whole_tiles = (columns + ROWS - 1) / ROWS;
    const int tiles_a_block = PARTS * (whole_tiles >= grid ? (whole_tiles + grid - 1) / grid : 1);
    // what the blocks share out: whole tiles when there is one for every block, else rows
    const int units = whole_tiles >= grid ? whole_tiles : columns;
    const int share_base = units / grid, share_extra = units % grid;
    const size_t rings = (size_t)WARPS * STAGES * SLICE_BYTES;
    // (the gated convolution with up to 8 tokens and resident activations keeps a section of
    // sums for each of its three tiles)
    auto sums_for = [](bool with_resident) {
        const size_t sections = EPILOGUE == GATED_CONV && NT == 1 && with_resident ? 3 : 1;
        return (size_t)2 * sections * WARPS * ROWS * 8 * NT * sizeof(float);
    };
    const size_t resident = (size_t)8 * NT * ((k + 63) / 64) * 64 * 2;
    // activations in shared memory pay off when a block reuses them for several tiles
    const bool fits = NT <= 2 && rings + sums_for(true) + resident <= SHARED_LIMIT;
    const bool use_resident = fits && (norm.source != nullptr || tiles_a_block >= 2);
    const size_t sums = sums_for(use_resident);
    const size_t token_ring = !use_resident && NT == 1 ? (size_t)WARPS * STAGES * 8 * SLICE * 2 : 0;
    const size_t shared = rings + token_ring + sums + (use_resident ? resident : 0);
    cudaError_t err;
    if (norm.source != nullptr) {
        // (the norm's weights wait in the space of the partial sums, behind 64 floats)
        if (!fits || NT > 2 || (size_t)(64 + k) * sizeof(float) > sums) return cudaErrorInvalidValue;
        constexpr bool WITH_NORM = NT <= 2;
        auto kernel = skinny_gemm_kernel<NT, EPILOGUE, WITH_NORM, WITH_NORM>;
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (err != cudaSuccess) return err;
        return launch_kernel(kernel, dim3(grid), dim3(WARPS * 32), shared, stream, true,
                             (const bf16*)nullptr, 0, (const bf16*)w, bias, out, ldo, m, n, k,
                             up_offset, norm.source, norm.ld, norm.weight, norm.eps, conv,
                             share_base, share_extra);
    }
    if (use_resident) {
        auto kernel = skinny_gemm_kernel<NT, EPILOGUE, (NT <= 2), false>;
        err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
        if (err != cudaSuccess) return err;
        return launch_kernel(kernel, dim3(grid), dim3(WARPS * 32), shared, stream, true,
                             (const bf16*)a, lda, (const bf16*)w, bias, out, ldo, m, n, k,
                             up_offset, (const float*)nullptr, 0, (const float*)nullptr, 0.f, conv,
                             share_base, share_extra);
    }
    auto kernel = skinny_gemm_kernel<NT, EPILOGUE, false, false>;
    err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (err != cudaSuccess) return err;
    return launch_kernel(kernel, dim3(grid), dim3(WARPS * 32), shared, stream, true, (const bf16*)a,
                         lda, (const bf16*)w, bias, out, ldo, m, n, k, up_offset,
                         (const float*)nullptr, 0, (const float*)nullptr, 0.f, conv,
                             share_base, share_extra);
}

template <int EPILOGUE>
cudaError_t launch_for_rows(const void* a, int lda, const void* w, const float* bias, void* out,
                            int ldo, int m, int n, int k, int up_offset, cudaStream_t stream,
                            NormInput norm = NormInput(), ConvUpdate conv = ConvUpdate()) {
    if (m <= 8)
        return launch<1, EPILOGUE>(a, lda, w, bias, out, ldo, m, n, k, up_offset, stream, norm, conv);
    if (m <= 16)
        return launch<2, EPILOGUE>(a, lda, w, bias, out, ldo, m, n, k, up_offset, stream, norm, conv);
    return launch<4, EPILOGUE>(a, lda, w, bias, out, ldo, m, n, k, up_offset, stream, norm, conv);
}

}  // namespace

// Most rows (tokens) that the skinny product takes; more go to the library product.
MLXONE_API int mlxone_gemm_skinny_max_rows() { return 32; }

// epilogue: 0 = out bf16 [m, n]; 1 = SwiGLU, w is [gate rows; up rows] with n = 2 * width, out
// bf16 [m, width]; 2 = out is the float32 residual [m, n], added in place; 3 = out float32.
MLXONE_API int mlxone_gemm_skinny(const void* a, int lda, const void* w, const float* bias,
                                  void* out, int ldo, int m, int n, int k, int epilogue,
                                  cudaStream_t stream) {
    if (m == 0 || n == 0) return 0;
    MLXONE_REQUIRE(m > 0 && m <= 32, "gemm_skinny: %d rows, at most 32", m);
    MLXONE_REQUIRE(n > 0 && k > 0 && k % 8 == 0 && lda % 8 == 0,
                   "gemm_skinny: K (%d) and the row stride of a (%d) must be multiples of 8", k, lda);
    MLXONE_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                   "gemm_skinny: operands must be 16-byte aligned");
    MLXONE_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_skinny: unknown epilogue %d", epilogue);
    MLXONE_REQUIRE(epilogue != SWIGLU || n % 2 == 0, "gemm_skinny: SwiGLU needs an even n");
    cudaError_t err;
    switch (epilogue) {
        case STORE_BF16:
            err = launch_for_rows<STORE_BF16>(a, lda, w, bias, out, ldo, m, n, k, 0, stream); break;
        case SWIGLU:
            err = launch_for_rows<SWIGLU>(a, lda, w, bias, out, ldo, m, n, k, n / 2, stream); break;
        case ADD_RESIDUAL:
            err = launch_for_rows<ADD_RESIDUAL>(a, lda, w, bias, out, ldo, m, n, k, 0, stream); break;
        default:
            err = launch_for_rows<STORE_F32>(a, lda, w, bias, out, ldo, m, n, k, 0, stream); break;
    }
    if (err != cudaSuccess) {
        mlxone_set_error("gemm_skinny: launch failed: %s", cudaGetErrorString(err));
        return 2;
    }
    MLXONE_LAUNCH_CHECK("gemm_skinny");
    return 0;
}

// The short convolution's decode step in the product's epilogue: a [m, k] (one token per request)
// times w = [B rows; C rows; x rows] ([3 * channels, k]), then per channel g = B * x, the
// convolution over the kept values of g and this one, times C; out [m, channels] bfloat16; the
// state [slots, taps - 1, channels] is shifted when write_state is set. Up to 4 taps.
MLXONE_API int mlxone_gemm_skinny_conv(const void* a, int lda, const void* w, const float* bias,
                                       void* out, int m, int channels, int k,
                                       const float* conv_kernel, const float* conv_bias,
                                       void* state, const int* slots, const int* history, int taps,
                                       int write_state, cudaStream_t stream) {
    if (m == 0 || channels == 0) return 0;
    MLXONE_REQUIRE(m > 0 && m <= 32, "gemm_skinny_conv: %d rows, at most 32", m);
    MLXONE_REQUIRE(channels > 0 && k > 0 && k % 8 == 0 && lda % 8 == 0,
                   "gemm_skinny_conv: K (%d) and the row stride of a (%d) must be multiples of 8", k, lda);
    MLXONE_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                   "gemm_skinny_conv: operands must be 16-byte aligned");
    MLXONE_REQUIRE(taps >= 1 && taps <= 4, "gemm_skinny_conv: kernel width %d is not in 1..4", taps);
    ConvUpdate conv;
    conv.kernel = conv_kernel; conv.bias = conv_bias; conv.state = static_cast<bf16*>(state);
    conv.slots = slots; conv.history = history; conv.taps = taps; conv.write_state = write_state;
    const cudaError_t err = launch_for_rows<GATED_CONV>(a, lda, w, bias, out, channels, m,
                                                        3 * channels, k, 0, stream, NormInput(), conv);
    if (err != cudaSuccess) {
        mlxone_set_error("gemm_skinny_conv: launch failed: %s", cudaGetErrorString(err));
        return 2;
    }
    MLXONE_LAUNCH_CHECK("gemm_skinny_conv");
    return 0;
}

// Rows and K up to which mlxone_gemm_skinny_norm applies the norm itself.
MLXONE_API int mlxone_gemm_skinny_norm_fits(int m, int k) {
    if (m < 1 || m > 16 || k % 8 != 0) return 0;
    const size_t rings = (size_t)WARPS * STAGES * SLICE_BYTES;
    const int nt = m <= 8 ? 1 : 2;
    const size_t sums = (size_t)2 * WARPS * ROWS * 8 * nt * sizeof(float);
    const size_t resident = (size_t)8 * nt * ((k + 63) / 64) * 64 * 2;
    return rings + sums + resident <= SHARED_LIMIT && (size_t)(64 + k) * sizeof(float) <= sums ? 1 : 0;
}

// Rows and K up to which mlxone_gemm_skinny_conv_norm applies the norm itself (its partial sums
// take more room than the plain product's).
MLXONE_API int mlxone_gemm_skinny_conv_norm_fits(int m, int k) {
    if (!mlxone_gemm_skinny_norm_fits(m, k)) return 0;
    const int nt = m <= 8 ? 1 : 2;
    const size_t rings = (size_t)WARPS * STAGES * SLICE_BYTES;
    const size_t sums = (size_t)2 * (nt == 1 ? 3 : 1) * WARPS * ROWS * 8 * nt * sizeof(float);
    const size_t resident = (size_t)8 * nt * ((k + 63) / 64) * 64 * 2;
    return rings + sums + resident <= SHARED_LIMIT ? 1 : 0;
}

// As mlxone_gemm_skinny_conv with a = RMSNorm(source; norm_weight, eps) in bfloat16, the norm
// applied while the rows are brought in (sizes as for mlxone_gemm_skinny_norm_fits).
MLXONE_API int mlxone_gemm_skinny_conv_norm(const float* source, int source_ld,
                                            const float* norm_weight, float eps, const void* w,
                                            const float* bias, void* out, int m, int channels, int k,
                                            const float* conv_kernel, const float* conv_bias,
                                            void* state, const int* slots, const int* history,
                                            int taps, int write_state, cudaStream_t stream) {
    if (m == 0 || channels == 0) return 0;
    MLXONE_REQUIRE(mlxone_gemm_skinny_conv_norm_fits(m, k), "gemm_skinny_conv_norm: %d rows of %d do not fit", m, k);
    MLXONE_REQUIRE(channels > 0 && source_ld % 4 == 0 &&
                       (reinterpret_cast<uintptr_t>(source) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(norm_weight) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                   "gemm_skinny_conv_norm: operands must be 16-byte aligned");
    MLXONE_REQUIRE(taps >= 1 && taps <= 4, "gemm_skinny_conv_norm: kernel width %d is not in 1..4", taps);
    ConvUpdate conv;
    conv.kernel = conv_kernel; conv.bias = conv_bias; conv.state = static_cast<bf16*>(state);
    conv.slots = slots; conv.history = history; conv.taps = taps; conv.write_state = write_state;
    NormInput norm;
    norm.source = source; norm.ld = source_ld; norm.weight = norm_weight; norm.eps = eps;
    const cudaError_t err = launch_for_rows<GATED_CONV>(nullptr, 0, w, bias, out, channels, m,
                                                        3 * channels, k, 0, stream, norm, conv);
    if (err != cudaSuccess) {
        mlxone_set_error("gemm_skinny_conv_norm: launch failed: %s", cudaGetErrorString(err));
        return 2;
    }
    MLXONE_LAUNCH_CHECK("gemm_skinny_conv_norm");
    return 0;
}

// As mlxone_gemm_skinny with a = RMSNorm(source; norm_weight, eps) in bfloat16, the norm applied
// while the rows are brought in. source: float32 [m, k] with row stride source_ld.
MLXONE_API int mlxone_gemm_skinny_norm(const float* source, int source_ld,
                                       const float* norm_weight, float eps, const void* w,
                                       const float* bias, void* out, int ldo, int m, int n, int k,
                                       int epilogue, cudaStream_t stream) {
    if (m == 0 || n == 0) return 0;
    MLXONE_REQUIRE(mlxone_gemm_skinny_norm_fits(m, k), "gemm_skinny_norm: %d rows of %d do not fit", m, k);
    MLXONE_REQUIRE(n > 0 && source_ld % 4 == 0 &&
                       (reinterpret_cast<uintptr_t>(source) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(norm_weight) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(w) & 15) == 0,
                   "gemm_skinny_norm: operands must be 16-byte aligned");
    MLXONE_REQUIRE(epilogue >= 0 && epilogue <= 3, "gemm_skinny_norm: unknown epilogue %d", epilogue);
    MLXONE_REQUIRE(epilogue != SWIGLU || n % 2 == 0, "gemm_skinny_norm: SwiGLU needs an even n");
    NormInput norm;
    norm.source = source; norm.ld = source_ld; norm.weight = norm_weight; norm.eps = eps;
    cudaError_t err;
    switch (epilogue) {
        case STORE_BF16:
            err = launch_for_rows<STORE_BF16>(nullptr, 0, w, bias, out, ldo, m, n, k, 0, stream, norm); break;
        case SWIGLU:
            err = launch_for_rows<SWIGLU>(nullptr, 0, w, bias, out, ldo, m, n, k, n / 2, stream, norm); break;
        case ADD_RESIDUAL:
            err = launch_for_rows<ADD_RESIDUAL>(nullptr, 0, w, bias, out, ldo, m, n, k, 0, stream, norm); break;
        default:
            err = launch_for_rows<STORE_F32>(nullptr, 0, w, bias, out, ldo, m, n, k, 0, stream, norm); break;
    }
    if (err != cudaSuccess) {
        mlxone_set_error("gemm_skinny_norm: launch failed: %s", cudaGetErrorString(err));
        return 2;
    }
    MLXONE_LAUNCH_CHECK("gemm_skinny_norm");
    return 0;
}
