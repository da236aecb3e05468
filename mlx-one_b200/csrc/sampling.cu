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
// A row is shared by the blocks of a thread-block cluster (eight, four, two or one, by the number
// of rows); each block counts its stretch of the row and adds its counts to every block's
// histogram through distributed shared memory.
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

// Counts and masses of a run of entries of one bucket, handed to `flush(digit, count, mass)`
// when the bucket changes: equal neighbours then cost one update of the histogram, not one each.
struct BucketRun {
    unsigned digit = 0xffffffffu, count = 0u;
    unsigned long long mass = 0ull;
    template <typename Flush>
    __device__ __forceinline__ void add(unsigned d, float value, Flush&& flush) {
        if (d != digit) {
            if (count) flush(digit, count, mass);
            digit = d; count = 0u; mass = 0ull;
        }
        ++count;
        mass += fixed_mass(value);
    }
    template <typename Flush>
    __device__ __forceinline__ void finish(Flush&& flush) {
        if (count) flush(digit, count, mass);
        count = 0u;
    }
};

// A 64-bit sum in this block's shared memory as two 32-bit atomics: the low word's wrap-around
// is seen in the value it held before, and carried into the high word. Exact in any order.
__device__ __forceinline__ void add_wide(unsigned long long* sum, unsigned long long value) {
    unsigned* words = reinterpret_cast<unsigned*>(sum);
    const unsigned low = (unsigned)value, high = (unsigned)(value >> 32);
    const unsigned before = atomicAdd(&words[0], low);
    const unsigned carry = before + low < before ? 1u : 0u;
    if (high + carry) atomicAdd(&words[1], high + carry);
}

// ---- the blocks of one row form a thread-block cluster and reach one another's shared memory
__device__ __forceinline__ unsigned cluster_rank() {
    unsigned rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    return rank;
}
// A barrier over all threads of the cluster; what they wrote before it (also into other blocks'
// shared memory) is visible after it.
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
// The address, in the cluster's shared window, of block `rank`'s copy of a shared variable.
__device__ __forceinline__ unsigned in_block(const void* local, unsigned rank) {
    const unsigned address = (unsigned)__cvta_generic_to_shared(local);
    unsigned mapped;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(mapped) : "r"(address), "r"(rank));
    return mapped;
}
__device__ __forceinline__ void remote_add(unsigned address, unsigned value) {
    asm volatile("red.shared::cluster.add.u32 [%0], %1;\n" :: "r"(address), "r"(value) : "memory");
}
__device__ __forceinline__ void remote_add(unsigned address, unsigned long long value) {
    asm volatile("red.shared::cluster.add.u64 [%0], %1;\n" :: "r"(address), "l"(value) : "memory");
}
__device__ __forceinline__ void remote_store(unsigned address, unsigned long long value) {
    asm volatile("st.shared::cluster.u64 [%0], %1;\n" :: "r"(address), "l"(value) : "memory");
}
__device__ __forceinline__ void remote_store(unsigned address, float value) {
    asm volatile("st.shared::cluster.f32 [%0], %1;\n" :: "r"(address), "f"(value) : "memory");
}
__device__ __forceinline__ void remote_store(unsigned address, int value) {
    asm volatile("st.shared::cluster.s32 [%0], %1;\n" :: "r"(address), "r"(value) : "memory");
}

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
// CLUSTER blocks share a row: block `rank` owns a stretch of consecutive tokens. Every block
// holds the whole histograms (each adds what it counted to every block's copy), so all blocks
// take the same decisions without asking one another.
constexpr int SAMPLE_SHARED_BYTES = TOP_BUCKETS * (2 * 8 + 2 * 4);

template <int CLUSTER>
__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
              const int* __restrict__ top_k, const float* __restrict__ top_p,
              const long long* __restrict__ seed, const int* __restrict__ step,
              float* probabilities, int* __restrict__ out) {
    extern __shared__ __align__(16) unsigned char sample_shared[];
    // first digit, all entries of the row; then this block's own count of it, whose room is used
    // afterwards, zeroed, for two histograms of a lower digit that take turns
    unsigned long long* top_mass = reinterpret_cast<unsigned long long*>(sample_shared);
    unsigned long long* own_mass = top_mass + TOP_BUCKETS;
    unsigned* top_count = reinterpret_cast<unsigned*>(own_mass + TOP_BUCKETS);
    unsigned* own_count = top_count + TOP_BUCKETS;
    __shared__ unsigned long long scan_scratch[33];
    __shared__ unsigned long long warp_ties[32], warp_mass[32];
    __shared__ unsigned long long block_zeros[CLUSTER], block_mass[CLUSTER];
    __shared__ unsigned long long block_ties[CLUSTER], block_kept[CLUSTER];
    __shared__ float block_top[CLUSTER];
    __shared__ float fscratch[33];
    __shared__ int found;
    __shared__ unsigned long long found_above;
    __shared__ int chosen;
    const int r = blockIdx.x / CLUSTER;
    const unsigned rank = CLUSTER > 1 ? cluster_rank() : 0u;
    const float* row = logits + (size_t)r * vocab;
    float* p = probabilities + (size_t)r * vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (!(temperature[r] > 0.f)) {          // greedy row in a mixed batch: the first block's work
        if (rank == 0u) {
            const int index = block_argmax(row, vocab);
            if (tid == 0) out[r] = index;
        }
        return;
    }
    // this block's tokens: a stretch whose start keeps the 16-byte steps of the row
    const int share = (((vocab + CLUSTER - 1) / CLUSTER) + 3) & ~3;
    const int first = min((int)rank * share, vocab);
    const int mine = min(share, vocab - first);

    for (int b = tid; b < TOP_BUCKETS; b += blockDim.x) {
        top_count[b] = 0u; top_mass[b] = 0ull; own_count[b] = 0u; own_mass[b] = 0ull;
    }
    // ---- probabilities (numerators of the softmax; the largest is exactly 1) and the
    // histogram of their first digit
    float local_max = -INFINITY;
    visit_row(row + first, mine, [&](int, float v) { local_max = fmaxf(local_max, v); });
    local_max = block_max(local_max, fscratch);
    if (tid < CLUSTER) remote_store(in_block(&block_top[rank], tid), local_max);
    cluster_sync();
    float top = block_top[0];
#pragma unroll
    for (int t = 1; t < CLUSTER; ++t) top = fmaxf(top, block_top[t]);
    const float inv_t = 1.0f / temperature[r];
    const int k = top_k[r];
    const bool top_k_on = k > 0 && k < vocab;
    const float nucleus = top_p[r];
    const bool truncating = top_k_on || nucleus < 1.0f;
    unsigned long long local_zeros = 0ull, local_mass = 0ull;
    if (truncating) {
        BucketRun run;
        auto to_own = [&](unsigned d, unsigned count, unsigned long long mass) {
            atomicAdd(&own_count[d], count);
            add_wide(&own_mass[d], mass);
        };
        visit_row(row + first, mine, [&](int i, float v) {
            const float value = expf((v - top) * inv_t);
            p[first + i] = value;
            const unsigned bits = __float_as_uint(value);
            local_zeros += bits == 0u;
            run.add(bits >> 20, value, to_own);
        });
        run.finish(to_own);
    } else {
        visit_row(row + first, mine, [&](int i, float v) {
            const float value = expf((v - top) * inv_t);
            p[first + i] = value;
            local_zeros += __float_as_uint(value) == 0u;
            local_mass += fixed_mass(value);
        });
    }
    {
        unsigned long long zeros_here, mass_here;
        block_scan_exclusive(local_zeros, scan_scratch, &zeros_here);
        block_scan_exclusive(local_mass, scan_scratch, &mass_here);
        if (tid < CLUSTER) {
            remote_store(in_block(&block_zeros[rank], tid), zeros_here);
            remote_store(in_block(&block_mass[rank], tid), mass_here);
        }
    }
    // what this block counted goes to every block's histogram, and its own room is left zeroed
    for (int b = tid; b < TOP_BUCKETS; b += blockDim.x) {
        const unsigned count = own_count[b];
        if (count) {
            const unsigned long long mass = own_mass[b];
#pragma unroll
            for (int t = 0; t < CLUSTER; ++t) {
                remote_add(in_block(&top_count[b], t), count);
                remote_add(in_block(&top_mass[b], t), mass);
            }
            own_count[b] = 0u;
            own_mass[b] = 0ull;
        }
    }
    cluster_sync();
    unsigned long long zeros = 0ull, plain_mass = 0ull;
#pragma unroll
    for (int t = 0; t < CLUSTER; ++t) { zeros += block_zeros[t]; plain_mass += block_mass[t]; }

    // Histogram, by the digit at `level` (1 or 2), of the row's entries whose higher digits are
    // `prefix` and, with above_only, whose pattern lies beyond `floor_bits`: every block adds
    // its stretch's entries to every block's copy. The two copies take turns, and the one for
    // the next call is zeroed before this call's barrier, after which blocks may add to it.
    int turn = 0;
    unsigned* count_of = own_count;
    unsigned long long* mass_of = own_mass;
    auto histogram = [&](int level, unsigned prefix, bool above_only, unsigned floor_bits) {
        __syncthreads();
        count_of = own_count + turn * LOW_BUCKETS;
        mass_of = own_mass + turn * LOW_BUCKETS;
        unsigned* next_count = own_count + (turn ^ 1) * LOW_BUCKETS;
        unsigned long long* next_mass = own_mass + (turn ^ 1) * LOW_BUCKETS;
        for (int b = tid; b < LOW_BUCKETS; b += blockDim.x) { next_count[b] = 0u; next_mass[b] = 0ull; }
        BucketRun run;
        auto to_all = [&](unsigned d, unsigned count, unsigned long long mass) {
#pragma unroll
            for (int t = 0; t < CLUSTER; ++t) {
                remote_add(in_block(&count_of[d], t), count);
                remote_add(in_block(&mass_of[d], t), mass);
            }
        };
        visit_row(p + first, mine, [&](int, float value) {
            const unsigned bits = __float_as_uint(value);
            if ((!above_only || bits > floor_bits) && digits_above(bits, level) == prefix)
                run.add(digit_of(bits, level), value, to_all);
        });
        run.finish(to_all);
        cluster_sync();
        turn ^= 1;
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
        mass_above_k = nucleus < 1.0f ? mass_beyond(top_mass, TOP_BUCKETS, -1) : plain_mass;
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
    // owns a stretch of consecutive tokens of its block's stretch; the warp in whose stretch the
    // target falls walks it.
    const int warps = blockDim.x >> 5;
    const int stretch = (((mine + warps - 1) / warps) + 31) & ~31;
    const int begin = first + min(warp * stretch, mine), end = min(begin + stretch, first + mine);
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
    if (tid < CLUSTER) {             // this block's ties and mass beyond the edge, for every block
        unsigned long long ties_sum = 0ull, mass_sum = 0ull;
        for (int w = 0; w < warps; ++w) { ties_sum += warp_ties[w]; mass_sum += warp_mass[w]; }
        remote_store(in_block(&block_ties[rank], tid), ties_sum);
        remote_store(in_block(&block_kept[rank], tid), mass_sum);
    }
    cluster_sync();
    // ties are admitted in token order: blocks before this one, then warps before this one
    unsigned long long ties_before = 0ull, mass_before = 0ull;
    auto pass_over = [&](unsigned long long ties, unsigned long long mass) {
        const unsigned long long admitted =
            ties_before >= ties_edge ? 0ull : min(ties, ties_edge - ties_before);
        mass_before += mass + admitted * edge_mass;
        ties_before += ties;
    };
    for (int t = 0; t < (int)rank; ++t) pass_over(block_ties[t], block_kept[t]);
    for (int w = 0; w < warp; ++w) pass_over(warp_ties[w], warp_mass[w]);
    {
        const unsigned long long admitted =
            ties_before >= ties_edge ? 0ull : min(ties_here, ties_edge - ties_before);
        mass_here += admitted * edge_mass;
    }
    if (mass_before <= target && target < mass_before + mass_here) {       // one warp of the row
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
            const unsigned long long weight = !kept ? 0ull : tie ? edge_mass : fixed_mass(value);
            unsigned long long inclusive = weight;
#pragma unroll
            for (int offset = 1; offset < 32; offset <<= 1) {
                const unsigned long long other = __shfl_up_sync(0xffffffffu, inclusive, offset);
                if (lane >= offset) inclusive += other;
            }
            const unsigned hit = __ballot_sync(0xffffffffu, kept && running + inclusive > target);
            if (hit) {
                if (lane == 0) remote_store(in_block(&chosen, 0u), base + __ffs(hit) - 1);
                break;
            }
            running += __shfl_sync(0xffffffffu, inclusive, 31);
            ties_seen += (unsigned long long)__popc(tie_lanes);
        }
    }
    cluster_sync();            // also: no block leaves while another may write to its memory
    if (rank != 0u) return;
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
    // No early start for what follows: kernels of the next step read positions before they wait
    // for their predecessors (the decode attention asks for its old keys then), so the next
    // step begins only when this kernel has ended.
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
// With `report`, the tokens are also left there one after the other, followed by the value of the
// kernels' error flag: what the host reads back after a step, in one copy.
__global__ void publish_tokens_kernel(const int* __restrict__ chosen, const int* __restrict__ index,
                                      int* __restrict__ published, int count, int capacity,
                                      int* __restrict__ report, const int* __restrict__ error_flag) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count && index[i] >= 0 && index[i] < capacity) published[index[i]] = chosen[i];
    if (report != nullptr) {
        if (i < count) report[i] = chosen[i];
        if (i == count) report[count] = error_flag != nullptr ? *error_flag : 0;
    }
}

// token_ids[t] = published[source[t]] wherever source[t] >= 0 (else the host's id stays).
__global__ void resolve_tokens_kernel(int* __restrict__ token_ids, const int* __restrict__ source,
                                      const int* __restrict__ published, int count, int capacity) {
    griddep_launch();
    griddep_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count && source[i] >= 0 && source[i] < capacity) token_ids[i] = published[source[i]];
}

// report: null, or count + 1 entries (the tokens, then the error flag's value).
MLXONE_API int mlxone_publish_tokens(const int* chosen, const int* index, int* published, int count,
                                     int capacity, int* report, const int* error_flag,
                                     cudaStream_t stream) {
    if (count == 0) return 0;
    MLXONE_REQUIRE(count > 0 && capacity > 0, "publish_tokens: bad sizes");
    launch_kernel(publish_tokens_kernel, dim3((count + 256) / 256), dim3(256), 0, stream, true, chosen,
                  index, published, count, capacity, report, error_flag);
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
    // As many blocks per row as let all rows run at once: a cluster lies within one of the
    // GPU's eight groups of SMs, which hold two clusters of eight blocks, four of four.
    const int cluster = rows <= 16 ? 8 : rows <= 32 ? 4 : rows <= 64 ? 2 : 1;
    auto launch = [&](auto kernel) {
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             SAMPLE_SHARED_BYTES);
        cudaLaunchConfig_t config = {};
        config.gridDim = dim3(rows * cluster);
        config.blockDim = dim3(SAMPLE_THREADS);
        config.dynamicSmemBytes = SAMPLE_SHARED_BYTES;
        config.stream = stream;
        cudaLaunchAttribute attribute[1];
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = cluster;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        return cudaLaunchKernelEx(&config, kernel, logits, vocab, temperature, top_k, top_p, seed,
                                  step, probabilities, out);
    };
    const cudaError_t err = cluster == 8   ? launch(sample_kernel<8>)
                            : cluster == 4 ? launch(sample_kernel<4>)
                            : cluster == 2 ? launch(sample_kernel<2>)
                                           : launch(sample_kernel<1>);
    if (err != cudaSuccess) {
        mlxone_set_error("sample: launch failed: %s", cudaGetErrorString(err));
        return 1;
    }
    MLXONE_LAUNCH_CHECK("sample");
    return 0;
}
