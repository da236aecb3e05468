// Token selection from 32-bit logits: argmax, and temperature sampling with top-k and
// top-p truncation and a counter-based random number per (seed, step).
//
// The truncation rule is the reference's (src/mlx_one/text/sampling.py:56-88): probabilities
// p = softmax(logits / T); rank by descending p with ties in token order; keep the first
// top_k; of those keep the shortest prefix whose mass reaches top_p * (kept mass). The kept
// set is found without sorting: the k-th largest probability and the top-p boundary are
// located by a radix search over the bit patterns of the non-negative floats (three histogram
// passes each, 11 + 11 + 9 bits), and ties at a boundary are admitted in token order. The draw
// then takes the first kept token, in token order, whose running mass passes u * kept mass
// (the reference walks them in rank order; both draw from the same distribution), with
// u = uniform(seed, step).
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

// Index of the largest value of a row, the lowest index among equals. All threads of the
// block call it; thread 0 gets the result.
__device__ __forceinline__ int block_argmax(const float* __restrict__ row, int vocab) {
    __shared__ float best_value[32];
    __shared__ int best_index[32];
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
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
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

// ---- sampling
//
// Masses are summed as integers: a probability p in [0, 1] counts floor(p * 2^43). Integer sums
// do not depend on the order of the additions, so histograms can be filled with atomics and a
// row's draw is the same in every run. A vocabulary of 2^20 tokens cannot overflow 64 bits.
constexpr int SAMPLE_THREADS = 1024;
constexpr int TOP_BUCKETS = 2048;                   // first digit: 11 bits
constexpr int LOW_BUCKETS = 1024;                   // second and third digit: 10 bits each
constexpr float FIXED_ONE = 8796093022208.0f;       // 2^43

__device__ __forceinline__ unsigned long long fixed_mass(float p) {
    return (unsigned long long)(p * FIXED_ONE);
}

// The bit pattern of a non-negative float orders like the float. Its 31 bits are searched in
// three digits of 11, 10 and 10 bits, from the top.
__device__ __forceinline__ unsigned digit_of(unsigned bits, int level) {
    return level == 0 ? bits >> 20 : level == 1 ? (bits >> 10) & 0x3FFu : bits & 0x3FFu;
}
__device__ __forceinline__ unsigned digits_above(unsigned bits, int level) {
    return level == 0 ? 0u : level == 1 ? bits >> 20 : bits >> 10;
}

// f(i, row[i]) for every i < n, each by one thread of the block, with 16-byte loads where the
// row allows them. The order of the calls is not the order of i.
template <typename F>
__device__ __forceinline__ void visit_row(const float* row, int n, F&& f) {
    const int head = min(n, (int)(((16u - (unsigned)((size_t)row & 15u)) & 15u) >> 2));
    if ((int)threadIdx.x < head) f((int)threadIdx.x, row[threadIdx.x]);
    const float4* body = reinterpret_cast<const float4*>(row + head);
    const int quads = (n - head) >> 2;
#pragma unroll 4
    for (int q = threadIdx.x; q < quads; q += blockDim.x) {
        const float4 v = body[q];
        const int i = head + 4 * q;
        f(i, v.x); f(i + 1, v.y); f(i + 2, v.z); f(i + 3, v.w);
    }
    const int i = head + 4 * quads + (int)threadIdx.x;
    if (i < n) f(i, row[i]);
}

// Counts and masses of a run of entries of one bucket, added to the shared histogram when the
// bucket changes: equal neighbours then cost one atomic, not one each.
struct BucketRun {
    unsigned digit = 0xffffffffu, count = 0u;
    unsigned long long mass = 0ull;
    // A 64-bit sum in shared memory as two 32-bit atomics: the low word's wrap-around is seen in
    // the value it held before, and carried into the high word. Exact in any order.
    __device__ __forceinline__ void flush(unsigned* count_of, unsigned long long* mass_of) {
        if (count) {
            atomicAdd(&count_of[digit], count);
            unsigned* words = reinterpret_cast<unsigned*>(mass_of + digit);
            const unsigned low = (unsigned)mass, high = (unsigned)(mass >> 32);
            const unsigned before = atomicAdd(&words[0], low);
            const unsigned carry = before + low < before ? 1u : 0u;
            if (high + carry) atomicAdd(&words[1], high + carry);
        }
    }
    __device__ __forceinline__ void add(unsigned d, float value, unsigned* count_of,
                                        unsigned long long* mass_of) {
        if (d != digit) {
            flush(count_of, mass_of);
            digit = d; count = 0u; mass = 0ull;
        }
        ++count;
        mass += fixed_mass(value);
    }
};

// Exclusive prefix sum over the block, in thread order; *total gets the sum. scratch: 33 entries.
__device__ __forceinline__ unsigned long long block_scan_exclusive(unsigned long long v,
                                                                   unsigned long long* scratch,
                                                                   unsigned long long* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    unsigned long long inclusive = v;
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
        const unsigned long long other = __shfl_up_sync(0xffffffffu, inclusive, offset);
        if (lane >= offset) inclusive += other;
    }
    __syncthreads();
    if (lane == 31) scratch[warp] = inclusive;
    __syncthreads();
    if (warp == 0) {
        const unsigned long long mine = lane < warps ? scratch[lane] : 0ull;
        unsigned long long sum = mine;
#pragma unroll
        for (int offset = 1; offset < 32; offset <<= 1) {
            const unsigned long long other = __shfl_up_sync(0xffffffffu, sum, offset);
            if (lane >= offset) sum += other;
        }
        scratch[lane] = sum - mine;
        if (lane == 31) scratch[32] = sum;
    }
    __syncthreads();
    if (total != nullptr) *total = scratch[32];
    return scratch[warp] + inclusive - v;
}

// The highest bucket d with above(d) + hist[d] >= need, above(d) being base + the sum of hist
// over the buckets beyond d. found[0] = d, found_above[0] = above(d). Where nothing reaches
// `need` the lowest bucket is taken. All threads call it; results are read after it returns.
template <typename T>
__device__ __forceinline__ void find_bucket(const T* hist, int buckets, unsigned long long need,
                                            unsigned long long base, unsigned long long* scratch,
                                            int* found, unsigned long long* found_above) {
    constexpr int PER = TOP_BUCKETS / SAMPLE_THREADS;
    unsigned long long h[PER], local = 0ull;
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int j = threadIdx.x * PER + e;             // position from the top
        h[e] = j < buckets ? (unsigned long long)hist[buckets - 1 - j] : 0ull;
        local += h[e];
    }
    if (threadIdx.x == 0) *found = -1;
    unsigned long long total;
    unsigned long long running = base + block_scan_exclusive(local, scratch, &total);
#pragma unroll
    for (int e = 0; e < PER; ++e) {
        const int j = threadIdx.x * PER + e;
        if (j < buckets && running < need && running + h[e] >= need) {
            *found = buckets - 1 - j;
            *found_above = running;
        }
        running += h[e];
    }
    __syncthreads();
    if (*found < 0) {
        __syncthreads();
        if (threadIdx.x == 0) {
            *found = 0;
            *found_above = base + total - (unsigned long long)hist[0];
        }
        __syncthreads();
    }
}

// Per row: temperature[r] <= 0 -> argmax. top_k[r] <= 0 -> no top-k. top_p[r] >= 1 -> none.
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const long long* __restrict__ seed, const int* __restrict__ step,
              float* probabilities, int* __restrict__ out) {
    __shared__ unsigned top_count[TOP_BUCKETS];              // first digit, all entries
    __shared__ unsigned long long top_mass[TOP_BUCKETS];
    __shared__ unsigned count_of[LOW_BUCKETS];               // a lower digit, entries of one prefix
    __shared__ unsigned long long mass_of[LOW_BUCKETS];
    __shared__ unsigned long long scan_scratch[33];
    __shared__ unsigned long long warp_ties[32], warp_mass[32];
    __shared__ float fscratch[33];
    __shared__ int found;
    __shared__ unsigned long long found_above;
    __shared__ int chosen;
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * vocab;
    float* p = probabilities + (size_t)r * vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!(temperature[r] > 0.f)) {          // greedy row in a mixed batch
        const int index = block_argmax(row, vocab);
        if (tid == 0) out[r] = index;
        return;
    }

    // ---- probabilities (numerators of the softmax; the largest is exactly 1) and the
    // histogram of their first digit
    float local_max = -INFINITY;
    visit_row(row, vocab, [&](int, float v) { local_max = fmaxf(local_max, v); });
    const float top = block_max(local_max, fscratch);
    const float inv_t = 1.0f / temperature[r];
    for (int b = tid; b < TOP_BUCKETS; b += blockDim.x) { top_count[b] = 0u; top_mass[b] = 0ull; }
    __syncthreads();
    const int k = top_k[r];
    const bool top_k_on = k > 0 && k < vocab;
    const float nucleus = top_p[r];
    unsigned long long local_zeros = 0ull, local_mass = 0ull;
    if (top_k_on || nucleus < 1.0f) {
        BucketRun run;
        visit_row(row, vocab, [&](int i, float v) {
            const float value = expf((v - top) * inv_t);
            p[i] = value;
            const unsigned bits = __float_as_uint(value);
            local_zeros += bits == 0u;
            run.add(bits >> 20, value, top_count, top_mass);
        });
        run.flush(top_count, top_mass);
    } else {
        visit_row(row, vocab, [&](int i, float v) {
            const float value = expf((v - top) * inv_t);
            p[i] = value;
            local_zeros += __float_as_uint(value) == 0u;
            local_mass += fixed_mass(value);
        });
    }
    __syncthreads();

    // Histogram, by the digit at `level` (1 or 2), of the entries whose higher digits are
    // `prefix` and, with above_only, whose pattern lies beyond `floor_bits`.
    auto histogram = [&](int level, unsigned prefix, bool above_only, unsigned floor_bits) {
        __syncthreads();
        for (int b = tid; b < LOW_BUCKETS; b += blockDim.x) { count_of[b] = 0u; mass_of[b] = 0ull; }
        __syncthreads();
        BucketRun run;
        visit_row(p, vocab, [&](int, float value) {
            const unsigned bits = __float_as_uint(value);
            if ((!above_only || bits > floor_bits) && digits_above(bits, level) == prefix)
                run.add(digit_of(bits, level), value, count_of, mass_of);
        });
        run.flush(count_of, mass_of);
        __syncthreads();
    };
    auto mass_beyond = [&](const unsigned long long* hist, int buckets, int d) {
        unsigned long long beyond = 0ull, sum;
        for (int b = d + 1 + tid; b < buckets; b += blockDim.x) beyond += hist[b];
        block_scan_exclusive(beyond, scan_scratch, &sum);
        return sum;
    };

    // ---- top-k: kth = pattern of the k-th largest probability, ties_k of its ties are kept
    unsigned kth = 0u;
    unsigned long long above_k = 0ull, mass_above_k = 0ull, equal_k = 0ull;
    if (top_k_on) {
        find_bucket(top_count, TOP_BUCKETS, (unsigned long long)k, 0ull, scan_scratch, &found,
                    &found_above);
        unsigned prefix = (unsigned)found;
        above_k = found_above;
        mass_above_k = mass_beyond(top_mass, TOP_BUCKETS, found);
        for (int level = 1; level < 3; ++level) {
            histogram(level, prefix, false, 0u);
            find_bucket(count_of, LOW_BUCKETS, (unsigned long long)k, above_k, scan_scratch, &found,
                        &found_above);
            const int d = found;
            above_k = found_above;
            mass_above_k += mass_beyond(mass_of, LOW_BUCKETS, d);
            if (level == 2) equal_k = count_of[d];
            prefix = (prefix << 10) | (unsigned)d;
        }
        kth = prefix;
    } else {
        unsigned long long zeros;
        if (nucleus < 1.0f) mass_above_k = mass_beyond(top_mass, TOP_BUCKETS, -1);
        else block_scan_exclusive(local_mass, scan_scratch, &mass_above_k);
        block_scan_exclusive(local_zeros, scan_scratch, &zeros);
        above_k = (unsigned long long)vocab - zeros;
        equal_k = zeros;
    }
    const unsigned long long ties_k =
        top_k_on ? min((unsigned long long)k - above_k, equal_k) : equal_k;
    const unsigned long long kth_mass = fixed_mass(__uint_as_float(kth));
    const unsigned long long kept_mass = mass_above_k + ties_k * kth_mass;

    // ---- top-p inside the kept set: boundary pattern `edge`, ties_edge of its ties are kept
    unsigned edge = kth;
    unsigned long long ties_edge = ties_k, mass_above_edge = mass_above_k;
    if (nucleus < 1.0f) {
        unsigned long long cutoff = (unsigned long long)((double)nucleus * (double)kept_mass);
        cutoff = max(1ull, min(cutoff, kept_mass));
        // First digit: the buckets beyond the one of kth hold kept entries only; if they do not
        // reach the cutoff, the boundary lies in the bucket of kth.
        const int kth_top = (int)(kth >> 20);
        const unsigned long long beyond_kth_top = mass_beyond(top_mass, TOP_BUCKETS, kth_top);
        unsigned prefix = (unsigned)kth_top;
        unsigned long long above = beyond_kth_top, available = 0ull;
        if (cutoff <= beyond_kth_top) {
            find_bucket(top_mass, TOP_BUCKETS, cutoff, 0ull, scan_scratch, &found, &found_above);
            prefix = (unsigned)found;
            above = found_above;
        }
        for (int level = 1; level < 3; ++level) {
            histogram(level, prefix, true, kth);
            if (digits_above(kth, level) == prefix) {        // the kept ties of the top-k boundary
                if (tid == 0) {
                    count_of[digit_of(kth, level)] += (unsigned)ties_k;
                    mass_of[digit_of(kth, level)] += ties_k * kth_mass;
                }
                __syncthreads();
            }
            find_bucket(mass_of, LOW_BUCKETS, cutoff, above, scan_scratch, &found, &found_above);
            const int d = found;
            above = found_above;
            if (level == 2) available = count_of[d];
            prefix = (prefix << 10) | (unsigned)d;
        }
        edge = prefix < kth ? kth : prefix;
        mass_above_edge = above;
        const unsigned long long edge_mass = fixed_mass(__uint_as_float(edge));
        unsigned long long need = 1ull;
        if (edge_mass > 0ull && cutoff > above) need = (cutoff - above + edge_mass - 1ull) / edge_mass;
        ties_edge = max(1ull, min(need, available));
    }
    const unsigned long long edge_mass = fixed_mass(__uint_as_float(edge));
    const unsigned long long total = mass_above_edge + ties_edge * edge_mass;
    unsigned long long target =
        (unsigned long long)((double)uniform_from(seed[r], step[r]) * (double)total);
    if (total > 0ull && target >= total) target = total - 1ull;

    // ---- the first kept token, in token order, whose running mass passes the target. Each warp
    // owns a stretch of consecutive tokens; the warp in whose stretch the target falls walks it.
    const int warps = blockDim.x >> 5;
    const int stretch = (((vocab + warps - 1) / warps) + 31) & ~31;
    const int begin = min(warp * stretch, vocab), end = min(begin + stretch, vocab);
    unsigned long long ties_here = 0ull, mass_here = 0ull;
#pragma unroll 4
    for (int i = begin + lane; i < end; i += 32) {
        const float value = p[i];
        const unsigned bits = __float_as_uint(value);
        if (bits > edge) mass_here += fixed_mass(value);
        ties_here += bits == edge;
    }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
        ties_here += __shfl_xor_sync(0xffffffffu, ties_here, offset);
        mass_here += __shfl_xor_sync(0xffffffffu, mass_here, offset);
    }
    __syncthreads();
    if (lane == 0) { warp_ties[warp] = ties_here; warp_mass[warp] = mass_here; }
    if (tid == 0) chosen = -1;
    __syncthreads();
    unsigned long long ties_before = 0ull, mass_before = 0ull;
    for (int w = 0; w < warp; ++w) {
        const unsigned long long admitted =
            ties_before >= ties_edge ? 0ull : min(warp_ties[w], ties_edge - ties_before);
        mass_before += warp_mass[w] + admitted * edge_mass;
        ties_before += warp_ties[w];
    }
    {
        const unsigned long long admitted =
            ties_before >= ties_edge ? 0ull : min(ties_here, ties_edge - ties_before);
        mass_here += admitted * edge_mass;
    }
    if (mass_before <= target && target < mass_before + mass_here) {       // one warp
        unsigned long long running = mass_before, ties_seen = ties_before;
        for (int base = begin; base < end; base += 32) {
            const int i = base + lane;
            float value = 0.f;
            unsigned bits = 0u;
            if (i < end) { value = p[i]; bits = __float_as_uint(value); }
            const bool tie = i < end && bits == edge;
            const unsigned tie_lanes = __ballot_sync(0xffffffffu, tie);
            const unsigned long long tie_rank =
                ties_seen + (unsigned long long)__popc(tie_lanes & ((2u << lane) - 1u));
            const bool kept = i < end && (bits > edge || (tie && tie_rank <= ties_edge));
            const unsigned long long mine = !kept ? 0ull : tie ? edge_mass : fixed_mass(value);
            unsigned long long inclusive = mine;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const unsigned long long other = __shfl_up_sync(0xffffffffu, inclusive, offset);
                if (lane >= offset) inclusive += other;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, kept && running + inclusive > target);
            if (hit) {
                if (lane == 0) chosen = base + __ffs(hit) - 1;
                break;
            }
            running += __shfl_sync(0xffffffffu, inclusive, 31);
            ties_seen += (unsigned long long)__popc(tie_lanes);
        }
    }
    __syncthreads();
    if (chosen < 0) {
        // cannot happen while the kept mass is positive; the most probable token is always kept
        __syncthreads();
        if (tid == 0) chosen = 0x7fffffff;
        __syncthreads();
        for (int i = tid; i < vocab; i += blockDim.x)
            if (p[i] == 1.0f) atomicMin(&chosen, i);
        __syncthreads();
        if (tid == 0) out[r] = chosen == 0x7fffffff ? 0 : chosen;
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
    MLXONE_REQUIRE(vocab <= (1 << 20), "sample: at most 2^20 tokens in the vocabulary");
    sample_kernel<<<rows, SAMPLE_THREADS, 0, stream>>>(logits, vocab, temperature, top_k, top_p, seed,
                                               step, probabilities, out);
    MLXONE_LAUNCH_CHECK("sample");
    return 0;
}
