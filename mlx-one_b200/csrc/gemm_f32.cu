// True 32-bit matrix product: out[M, N] = a[M, K] * w[N, K]^T (+ bias[N]).
//
// Plain FMA on CUDA cores, no tensor cores and no reduced-precision mode. Every output
// element is accumulated over k = 0 .. K-1 in that order by one thread, so a row's result
// does not depend on how many other rows the call has or on where its tile lies.
#include "common.cuh"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool VEC>
__global__ void __launch_bounds__(256) gemm_f32_kernel(const float* __restrict__ a, int lda,
                                                       const float* __restrict__ w, int ldw,
                                                       const float* __restrict__ bias,
                                                       float* __restrict__ out, int ldo, int m,
                                                       int n, int k) {
    __shared__ float as[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int row0 = blockIdx.y * BM, col0 = blockIdx.x * BN;
    const int ty = tid / 16, tx = tid % 16;      // 16 x 16 threads, each 4 x 4 outputs
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    const int load_row = tid / 4;                // 0..63
    const int load_k = (tid % 4) * 4;            // 0, 4, 8, 12
    for (int k0 = 0; k0 < k; k0 += BK) {
        float av[4] = {0.f, 0.f, 0.f, 0.f}, wv[4] = {0.f, 0.f, 0.f, 0.f};
        const int ar = row0 + load_row, wr = col0 + load_row, kk = k0 + load_k;
        if (VEC) {
            if (ar < m && kk < k) {
                const float4 v = *reinterpret_cast<const float4*>(a + (size_t)ar * lda + kk);
                av[0] = v.x; av[1] = v.y; av[2] = v.z; av[3] = v.w;
            }
            if (wr < n && kk < k) {
                const float4 v = *reinterpret_cast<const float4*>(w + (size_t)wr * ldw + kk);
                wv[0] = v.x; wv[1] = v.y; wv[2] = v.z; wv[3] = v.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (ar < m && kk + i < k) av[i] = a[(size_t)ar * lda + kk + i];
                if (wr < n && kk + i < k) wv[i] = w[(size_t)wr * ldw + kk + i];
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            as[load_k + i][load_row] = av[i];
            ws[load_k + i][load_row] = wv[i];
        }
        __syncthreads();
#pragma unroll
        for (int kk2 = 0; kk2 < BK; ++kk2) {
            float ar4[TM], wr4[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) ar4[i] = as[kk2][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) wr4[j] = ws[kk2][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar4[i], wr4[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int r = row0 + ty * TM + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int c = col0 + tx * TN + j;
            if (c < n) out[(size_t)r * ldo + c] = acc[i][j] + (bias ? bias[c] : 0.f);
        }
    }
}

}  // namespace

MLXONE_API int mlxone_gemm_f32(const float* a, int lda, const float* w, int ldw,
                               const float* bias, float* out, int ldo, int m, int n, int k,
                               cudaStream_t stream) {
    if (m == 0 || n == 0) return 0;
    MLXONE_REQUIRE(m > 0 && n > 0 && k > 0, "gemm_f32: bad sizes m=%d n=%d k=%d", m, n, k);
    MLXONE_REQUIRE(lda >= k && ldw >= k && ldo >= n, "gemm_f32: leading dimension too small");
    const dim3 grid(ceil_div_host(n, BN), ceil_div_host(m, BM));
    MLXONE_REQUIRE(grid.y <= 65535, "gemm_f32: too many rows (%d)", m);
    const bool vec = k % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(a) & 15) == 0 &&
                     (reinterpret_cast<uintptr_t>(w) & 15) == 0;
    if (vec)
        gemm_f32_kernel<true><<<grid, 256, 0, stream>>>(a, lda, w, ldw, bias, out, ldo, m, n, k);
    else
        gemm_f32_kernel<false><<<grid, 256, 0, stream>>>(a, lda, w, ldw, bias, out, ldo, m, n, k);
    MLXONE_LAUNCH_CHECK("gemm_f32");
    return 0;
}
