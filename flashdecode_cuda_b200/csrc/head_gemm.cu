// One small matrix product per head:
//
//     out[t, h, n] = sum_k a[t, h, k] * w[h, n, k]        a [T, heads, K], w [heads, N, K], out [T, heads, N]
//
// (a per-head change of basis: a latent-attention mixer folds every head's key
// expansion into its queries this way, and expands every head's attended latent
// into values).  CUDA cores, float accumulation, k ascending in one fmaf chain
// per output, so no bit of a row depends on what else is in the step; float or
// bfloat16 storage.  A CTA takes 32 rows x 64 columns of one head.
#include "common.cuh"

namespace fd {

constexpr int HG_MT = 32, HG_NT = 64, HG_KT = 32, HG_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(HG_THREADS)
head_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w, T* __restrict__ out, int T_rows, int heads, int N,
                 int K) {
    __shared__ float a_s[HG_MT][HG_KT + 1];
    __shared__ float b_s[HG_NT][HG_KT + 1];
    const int h = blockIdx.z;
    const int m0 = blockIdx.y * HG_MT, n0 = blockIdx.x * HG_NT;
    const int tid = threadIdx.x;
    const T* ah = a + (size_t)h * K;                 // row stride heads * K
    const T* wh = w + (size_t)h * N * K;
    const size_t lda = (size_t)heads * K, ldo = (size_t)heads * N;
    const int ty = tid / 16, tx = tid % 16;          // rows 2 ty, 2 ty + 1; columns tx + 16 j
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += HG_KT) {
        for (int i = tid; i < HG_MT * HG_KT; i += HG_THREADS) {
            const int r = i / HG_KT, kk = i - r * HG_KT;
            a_s[r][kk] = (m0 + r < T_rows && k0 + kk < K) ? to_float(ah[(size_t)(m0 + r) * lda + k0 + kk]) : 0.f;
        }
        for (int i = tid; i < HG_NT * HG_KT; i += HG_THREADS) {
            const int c = i / HG_KT, kk = i - c * HG_KT;
            b_s[c][kk] = (n0 + c < N && k0 + kk < K) ? to_float(wh[(size_t)(n0 + c) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < HG_KT; ++kk) {
            const float a0 = a_s[2 * ty][kk], a1 = a_s[2 * ty + 1][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float b = b_s[tx + 16 * j][kk];
                acc[0][j] = fmaf(a0, b, acc[0][j]);
                acc[1][j] = fmaf(a1, b, acc[1][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int r = m0 + 2 * ty + i;
        if (r >= T_rows) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx + 16 * j;
            if (c < N) out[(size_t)r * ldo + (size_t)h * N + c] = from_float<T>(acc[i][j]);
        }
    }
}

// Steps of few rows in bfloat16 (K a multiple of 8): a warp per output column (head, n) reads that row of w once in
// 16-byte pieces and takes it against every row of a; eight warps per CTA.
template <int MAXT>
__global__ void __launch_bounds__(256)
head_gemv_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ w, __nv_bfloat16* __restrict__ out,
                 int T_rows, int heads, int N, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int col = blockIdx.x * 8 + warp;
    if (col >= heads * N) return;
    const int h = col / N;
    const __nv_bfloat16* wr = w + (size_t)col * K;
    const __nv_bfloat16* ah = a + (size_t)h * K;
    const size_t lda = (size_t)heads * K;
    float acc[MAXT];
#pragma unroll
    for (int t = 0; t < MAXT; ++t) acc[t] = 0.f;
    for (int c = lane * 8; c < K; c += 256) {
        const uint4 wv = *reinterpret_cast<const uint4*>(wr + c);
        const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
        for (int t = 0; t < MAXT; ++t) {
            if (t < T_rows) {
                const uint4 av = *reinterpret_cast<const uint4*>(ah + t * lda + c);
                const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&av);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    acc[t] = fmaf(__low2float(w2[e]), __low2float(a2[e]), acc[t]);
                    acc[t] = fmaf(__high2float(w2[e]), __high2float(a2[e]), acc[t]);
                }
            }
        }
    }
#pragma unroll
    for (int t = 0; t < MAXT; ++t) {
        if (t < T_rows) {
            const float v = warp_sum(acc[t]);
            if (lane == 0) out[(size_t)t * heads * N + col] = __float2bfloat16_rn(v);
        }
    }
}

}  // namespace fd

using namespace fd;

extern "C" int fd_head_gemm(const void* a, const void* w, void* out, int dtype, int T, int heads, int N, int K,
                            cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(heads > 0 && heads <= 65535 && N > 0 && K > 0, -2, "head_gemm: %d heads, N %d, K %d", heads, N, K);
    if (dtype == 1 && T <= 16 && K % 8 == 0 && (uintptr_t)a % 16 == 0 && (uintptr_t)w % 16 == 0) {
        const dim3 g((unsigned)((heads * (long long)N + 7) / 8));
        if (T <= 8)
            return launch("head_gemm", head_gemv_kernel<8>, g, dim3(256), 0, stream, dim3(1, 1, 1), (const __nv_bfloat16*)a,
                          (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, heads, N, K);
        return launch("head_gemm", head_gemv_kernel<16>, g, dim3(256), 0, stream, dim3(1, 1, 1), (const __nv_bfloat16*)a,
                      (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, heads, N, K);
    }
    dim3 grid((N + HG_NT - 1) / HG_NT, (T + HG_MT - 1) / HG_MT, heads);
    FD_REQUIRE(grid.y <= 65535, -2, "head_gemm: %d rows are too many", T);
    if (dtype == 0)
        return launch("head_gemm", head_gemm_kernel<float>, grid, dim3(HG_THREADS), 0, stream, dim3(1, 1, 1),
                      (const float*)a, (const float*)w, (float*)out, T, heads, N, K);
    return launch("head_gemm", head_gemm_kernel<__nv_bfloat16>, grid, dim3(HG_THREADS), 0, stream, dim3(1, 1, 1),
                  (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, (__nv_bfloat16*)out, T, heads, N, K);
}
