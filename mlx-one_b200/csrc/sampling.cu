// Token selection from 32-bit logits: argmax, and temperature sampling with top-k and
// top-p truncation and a counter-based random number per (seed, step).
//
// The truncation rule is the reference's (src/mlx_one/text/sampling.py:56-88): probabilities
// p = softmax(logits / T); rank by descending p with ties in token order; keep the first
// top_k; of those keep the shortest prefix whose mass reaches top_p * (kept mass). The kept
// set is found without sorting: the k-th largest probability and the top-p boundary are
// located by bisection over the bit patterns of the non-negative floats, and ties at a
// boundary are admitted in token order. The draw then walks the kept tokens in token order
// (the reference walks them in rank order; both draw from the same distribution):
// u = uniform(seed, step) * kept mass, the first kept token whose running mass reaches u.
//
// uniform(seed, step) is a splitmix64 hash of seed * 0x9E3779B97F4A7C15 + (step + 1) *
// 0xBF58476D1CE4E5B9, top 24 bits / 2^24, so a request's draws do not depend on what else is
// in the batch.
//
// Scratch: `probabilities` [rows, vocab] float, written by the kernel (softmax numerators),
// kept for the caller to inspect.
#include "common.cuh"

namespace {

constexpr int THREADS = 512;

__device__ __forceinline__ double block_sum_double(double v, double* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        double t = lane < warps ? scratch[lane] : 0.0;
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1)
            t += __shfl_xor_sync(0xffffffffu, t, offset);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

// Index of the largest value of a row, the lowest index among equals. All threads of the
// block call it; thread 0 gets the result.
__device__ __forceinline__ int block_argmax(const float* __restrict__ row, int vocab) {
    __shared__ float best_value[THREADS / 32];
    __shared__ int best_index[THREADS / 32];
    float value = -INFINITY;
    int index = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = row[i];
        if (v > value || (v == value && i < index)) { value = v; index = i; }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other > value || (other == value && other_index < index)) {
            value = other; index = other_index;
        }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_value[warp] = value; best_index[warp] = index; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < THREADS / 32; ++w)
            if (best_value[w] > value || (best_value[w] == value && best_index[w] < index)) {
                value = best_value[w]; index = best_index[w];
            }
    }
    return index == 0x7fffffff ? 0 : index;
}

__global__ void __launch_bounds__(THREADS)
argmax_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out) {
    griddep_launch();
    griddep_wait();
    const int index = block_argmax(logits + (size_t)blockIdx.x * vocab, vocab);
    if (threadIdx.x == 0) out[blockIdx.x] = index;
}

__device__ __forceinline__ float uniform_from(long long seed, int step) {
    unsigned long long z = (unsigned long long)seed * 0x9E3779B97F4A7C15ull +
                           (unsigned long long)(step + 1) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z = z ^ (z >> 31);
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

// Per row: temperature[r] <= 0 -> argmax. top_k[r] <= 0 -> no top-k. top_p[r] >= 1 -> none.
__global__ void __launch_bounds__(THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const long long* __restrict__ seed, const int* __restrict__ step,
              float* __restrict__ probabilities, int* __restrict__ out) {
    __shared__ float fscratch[33];
    __shared__ double dscratch[33];
    __shared__ int iscratch[33];
    __shared__ int chosen;
    __shared__ double carried_mass;
    __shared__ int carried_ties;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    float* p = probabilities + (size_t)r * vocab;
    const int tid = threadIdx.x;
    if (!(temperature[r] > 0.f)) {          // greedy row in a mixed batch
        const int index = block_argmax(row, vocab);
        if (tid == 0) out[r] = index;
        return;
    }

    // ---- probabilities (numerators of the softmax)
    float local_max = -INFINITY;
    for (int i = tid; i < vocab; i += blockDim.x) local_max = fmaxf(local_max, row[i]);
    const float top = block_max(local_max, fscratch);
    const float inv_t = 1.0f / temperature[r];
    for (int i = tid; i < vocab; i += blockDim.x) p[i] = expf((row[i] - top) * inv_t);
    __syncthreads();

    auto count_ge = [&](unsigned bits) {
        int c = 0;
        for (int i = tid; i < vocab; i += blockDim.x) c += __float_as_uint(p[i]) >= bits;
        // integer block sum through the double path keeps one reduction routine
        return (long long)(block_sum_double((double)c, dscratch) + 0.5);
    };

    // ---- top-k: kth = bits of the k-th largest probability, ties_k of its ties are kept
    unsigned kth = 0u;
    const int k = top_k[r];
    if (k > 0 && k < vocab) {
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned candidate = kth | (1u << bit);
            if (count_ge(candidate) >= k) kth = candidate;
        }
    }
    long long above_k = 0;
    double mass_above_k = 0.0;
    {
        int c = 0, e = 0;
        double m = 0.0;
        for (int i = tid; i < vocab; i += blockDim.x) {
            const unsigned b = __float_as_uint(p[i]);
            if (b > kth) { ++c; m += (double)p[i]; }
            e += b == kth;
        }
        above_k = (long long)(block_sum_double((double)c, dscratch) + 0.5);
        mass_above_k = block_sum_double(m, dscratch);
        const long long equal_k = (long long)(block_sum_double((double)e, dscratch) + 0.5);
        iscratch[0] = 0;
        __syncthreads();
        if (tid == 0)
            iscratch[0] = (int)((k > 0 && k < vocab) ? min((long long)k - above_k, equal_k) : equal_k);
        __syncthreads();
    }
    const int ties_k = iscratch[0];
    const double kth_value = (double)__uint_as_float(kth);
    const double kept_mass = mass_above_k + ties_k * kth_value;

    // ---- top-p inside the kept set: boundary value `edge`, ties_edge of its ties are kept
    unsigned edge = kth;
    int ties_edge = ties_k;
    double mass_above_edge = mass_above_k;
    const float nucleus = top_p[r];
    if (nucleus < 1.0f) {
        const double cutoff = (double)nucleus * kept_mass;
        // mass of kept tokens with probability >= x, for x >= kth
        auto mass_ge = [&](unsigned bits) {
            double m = 0.0;
            for (int i = tid; i < vocab; i += blockDim.x) {
                const unsigned b = __float_as_uint(p[i]);
                if (b >= bits && b > kth) m += (double)p[i];
            }
            m = block_sum_double(m, dscratch);
            return bits <= kth ? m + ties_k * kth_value : m;
        };
        unsigned found = 0u;
        for (int bit = 30; bit >= 0; --bit) {
            const unsigned candidate = found | (1u << bit);
            const unsigned probe = candidate < kth ? kth : candidate;
            if (mass_ge(probe) >= cutoff) found = candidate;
        }
        edge = found < kth ? kth : found;
        int e = 0;
        double m = 0.0;
        for (int i = tid; i < vocab; i += blockDim.x) {
            const unsigned b = __float_as_uint(p[i]);
            if (b > edge) m += (double)p[i];
            e += b == edge;
        }
        mass_above_edge = block_sum_double(m, dscratch);
        long long available = (long long)(block_sum_double((double)e, dscratch) + 0.5);
        if (edge == kth) available = ties_k;
        const double edge_value = (double)__uint_as_float(edge);
        long long need = 1;
        if (edge_value > 0.0) need = (long long)ceil((cutoff - mass_above_edge) / edge_value);
        need = max(1ll, min(need, available));
        ties_edge = (int)need;
    }
    const double edge_value = (double)__uint_as_float(edge);
    const double total = mass_above_edge + ties_edge * edge_value;
    const double target = (double)uniform_from(seed[r], step[r]) * total;

    // ---- walk kept tokens in token order until the running mass reaches the target
    if (tid == 0) { chosen = 0x7fffffff; carried_mass = 0.0; carried_ties = 0; }
    __syncthreads();
    int last_kept = -1;
    for (int base = 0; base < vocab; base += blockDim.x) {
        const int i = base + tid;
        unsigned b = 0u;
        float value = 0.f;
        if (i < vocab) { value = p[i]; b = __float_as_uint(value); }
        const int is_tie = (i < vocab && b == edge) ? 1 : 0;
        // inclusive scan of tie flags over the block
        int tie_rank = is_tie;
        const int lane = tid & 31, warp = tid >> 5;
        for (int offset = 1; offset < 32; offset <<= 1) {
            const int other = __shfl_up_sync(0xffffffffu, tie_rank, offset);
            if (lane >= offset) tie_rank += other;
        }
        if (lane == 31) iscratch[warp] = tie_rank;
        __syncthreads();
        int tie_offset = carried_ties;
        for (int w = 0; w < warp; ++w) tie_offset += iscratch[w];
        tie_rank += tie_offset;
        const bool kept = i < vocab && (b > edge || (is_tie && tie_rank <= ties_edge));
        double mass = kept ? (double)value : 0.0;
        double running = mass;
        for (int offset = 1; offset < 32; offset <<= 1) {
            const double other = __shfl_up_sync(0xffffffffu, running, offset);
            if (lane >= offset) running += other;
        }
        if (lane == 31) dscratch[warp] = running;
        __syncthreads();
        double mass_offset = carried_mass;
        for (int w = 0; w < warp; ++w) mass_offset += dscratch[w];
        running += mass_offset;
        if (kept) {
            last_kept = i;
            if (running >= target) atomicMin(&chosen, i);
        }
        __syncthreads();
        if (tid == blockDim.x - 1) { carried_mass = running; carried_ties = tie_rank; }
        __syncthreads();
        if (chosen != 0x7fffffff) break;
    }
    if (chosen == 0x7fffffff) {
        // rounding left the running mass just below the target: take the last kept token
        __syncthreads();
        if (tid == 0) iscratch[32] = -1;
        __syncthreads();
        atomicMax(&iscratch[32], last_kept);
        __syncthreads();
        if (tid == 0) out[r] = max(iscratch[32], 0);
    } else if (tid == 0) {
        out[r] = chosen;
    }
}

}  // namespace

// After a decode step whose tokens were chosen on the device: the chosen token becomes the
// request's next input, its position moves on by one, and the token is recorded in
// record[*counter, r]. Lets decode steps follow one another without the host.
__global__ void decode_advance_kernel(const int* __restrict__ chosen, int* __restrict__ token_ids,
                                      int* __restrict__ positions, int* __restrict__ history,
                                      int* __restrict__ record, int* __restrict__ counter,
                                      int requests, int max_steps) {
    griddep_launch();
    griddep_wait();
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    const int step = *counter;
    if (r < requests) {
        token_ids[r] = chosen[r];
        positions[r] += 1;
        history[r] += 1;
        if (step < max_steps) record[(size_t)step * requests + r] = chosen[r];
    }
    __syncthreads();
    if (blockIdx.x == 0 && threadIdx.x == 0) *counter = step + 1;
}

// Token ids that the device chose in an earlier step, kept per request so that a later step can
// take its input from here instead of from the host: published[index of request] = token.
__global__ void publish_tokens_kernel(const int* __restrict__ chosen, const int* __restrict__ index,
                                      int* __restrict__ published, int count, int capacity) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count && index[i] >= 0 && index[i] < capacity) published[index[i]] = chosen[i];
}

// token_ids[t] = published[source[t]] wherever source[t] >= 0 (else the host's id stays).
__global__ void resolve_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ source,
                                      const int* __restrict__ published, int count, int capacity) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count && source[i] >= 0 && source[i] < capacity) token_ids[i] = published[source[i]];
}

MLXONE_API int mlxone_publish_tokens(const int* chosen, const int* index, int* published, int count,
                                     int capacity, cudaStream_t stream) {
    if (count == 0) return 0;
    MLXONE_REQUIRE(count > 0 && capacity > 0, "publish_tokens: bad sizes");
    launch_kernel(publish_tokens_kernel, dim3((count + 255) / 256), dim3(256), 0, stream, true, chosen,
                  index, published, count, capacity);
    MLXONE_LAUNCH_CHECK("publish_tokens");
    return 0;
}

MLXONE_API int mlxone_resolve_tokens(int* token_ids, const int* source, const int* published,
                                     int count, int capacity, cudaStream_t stream) {
    if (count == 0) return 0;
    MLXONE_REQUIRE(count > 0 && capacity > 0, "resolve_tokens: bad sizes");
    launch_kernel(resolve_tokens_kernel, dim3((count + 255) / 256), dim3(256), 0, stream, true,
                  token_ids, source, published, count, capacity);
    MLXONE_LAUNCH_CHECK("resolve_tokens");
    return 0;
}

MLXONE_API int mlxone_decode_advance(const int* chosen, int* token_ids, int* positions,
                                     int* history, int* record, int* counter, int requests,
                                     int max_steps, cudaStream_t stream) {
    MLXONE_REQUIRE(requests > 0 && requests <= 1024, "decode_advance: 1..1024 requests");
    launch_kernel(decode_advance_kernel, dim3(1), dim3(1024), 0, stream, true, chosen, token_ids,
                  positions, history, record, counter, requests, max_steps);
    MLXONE_LAUNCH_CHECK("decode_advance");
    return 0;
}

// Argmax in two stages for wide rows: stage 1 reduces pieces of ARGMAX_PIECE entries to
// (value, index) pairs in scratch, stage 2 reduces the pairs. Few rows then still fill the GPU.
constexpr int ARGMAX_PIECE = 2048;

__global__ void __launch_bounds__(256)
argmax_pieces_kernel(const float* __restrict__ logits, int vocab, int pieces,
                     float* __restrict__ piece_value, int* __restrict__ piece_index) {
    __shared__ float best_value[8];
    __shared__ int best_index[8];
    griddep_launch();
    griddep_wait();
    const float* row = logits + (size_t)blockIdx.y * vocab;
    const int begin = blockIdx.x * ARGMAX_PIECE, end = min(begin + ARGMAX_PIECE, vocab);
    float value = -INFINITY;
    int index = 0x7fffffff;
    for (int i = begin + threadIdx.x; i < end; i += 256) {
        const float v = row[i];
        if (v > value || (v == value && i < index)) { value = v; index = i; }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other > value || (other == value && other_index < index)) {
            value = other; index = other_index;
        }
    }
    if ((threadIdx.x & 31) == 0) { best_value[threadIdx.x >> 5] = value; best_index[threadIdx.x >> 5] = index; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (best_value[w] > value || (best_value[w] == value && best_index[w] < index)) {
                value = best_value[w]; index = best_index[w];
            }
        piece_value[(size_t)blockIdx.y * pieces + blockIdx.x] = value;
        piece_index[(size_t)blockIdx.y * pieces + blockIdx.x] = index;
    }
}

__global__ void argmax_merge_kernel(const float* __restrict__ piece_value,
                                    const int* __restrict__ piece_index, int pieces,
                                    int* __restrict__ out) {
    griddep_launch();
    griddep_wait();
    const int lane = threadIdx.x;
    float value = -INFINITY;
    int index = 0x7fffffff;
    for (int i = lane; i < pieces; i += 32) {
        const float v = piece_value[(size_t)blockIdx.x * pieces + i];
        const int at = piece_index[(size_t)blockIdx.x * pieces + i];
        if (v > value || (v == value && at < index)) { value = v; index = at; }
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, value, offset);
        const int other_index = __shfl_xor_sync(0xffffffffu, index, offset);
        if (other > value || (other == value && other_index < index)) {
            value = other; index = other_index;
        }
    }
    if (lane == 0) out[blockIdx.x] = index == 0x7fffffff ? 0 : index;
}

// Entries of float/int scratch that mlxone_argmax needs for rows of `vocab` entries (0: none).
MLXONE_API int mlxone_argmax_scratch(int rows, int vocab) {
    const int pieces = (vocab + ARGMAX_PIECE - 1) / ARGMAX_PIECE;
    return pieces > 1 ? rows * pieces : 0;
}

MLXONE_API int mlxone_argmax(const float* logits, int rows, int vocab, int* out,
                             float* piece_value, int* piece_index, cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && vocab > 0 && rows <= 65535, "argmax: bad sizes");
    const int pieces = (vocab + ARGMAX_PIECE - 1) / ARGMAX_PIECE;
    if (pieces == 1 || piece_value == nullptr || piece_index == nullptr) {
        launch_kernel(argmax_kernel, dim3(rows), dim3(THREADS), 0, stream, true, logits, vocab, out);
    } else {
        launch_kernel(argmax_pieces_kernel, dim3(pieces, rows), dim3(256), 0, stream, true, logits,
                      vocab, pieces, piece_value, piece_index);
        launch_kernel(argmax_merge_kernel, dim3(rows), dim3(32), 0, stream, true,
                      (const float*)piece_value, (const int*)piece_index, pieces, out);
    }
    MLXONE_LAUNCH_CHECK("argmax");
    return 0;
}

MLXONE_API int mlxone_sample(const float* logits, int rows, int vocab, const float* temperature,
                             const int* top_k, const float* top_p, const long long* seed,
                             const int* step, float* probabilities, int* out,
                             cudaStream_t stream) {
    if (rows == 0) return 0;
    MLXONE_REQUIRE(rows > 0 && vocab > 0, "sample: bad sizes");
    MLXONE_REQUIRE(probabilities != nullptr, "sample: scratch for probabilities is missing");
    sample_kernel<<<rows, THREADS, 0, stream>>>(logits, vocab, temperature, top_k, top_p, seed,
                                               step, probabilities, out);
    MLXONE_LAUNCH_CHECK("sample");
    return 0;
}
