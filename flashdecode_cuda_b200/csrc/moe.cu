// Routed feed-forward (mixture of experts), all decisions on the device:
//
//  * moe_route: per token, router logits in float (one output per warp pass, k in
//    lane order), softmax over all router outputs, the `top` largest of score +
//    correction (ties: the lower index), and the chosen scores over their sum;
//  * moe_align: the (token, choice) pairs that go to an expert with weights,
//    grouped by expert, each group padded to whole row tiles, with the expert of
//    every tile and the number of tiles;
//  * moe_gemm: one CTA per (row tile, column tile): rows gathered through the
//    grouping, the tile's expert's matrix, k ascending in one fmaf chain per
//    output (no bit depends on what else is in the step); epilogue relu^2 into
//    the grouped activations, or float rows for the combine;
//  * moe_combine: per token, sum over its choices of weight * (expert row, or the
//    token's own input for an identity expert), plus the shared expert's row.
//
// Router outputs e >= n_experts are identity experts: they have no weights and
// pass their input on.
#include <math.h>

#include "common.cuh"

namespace fd {

constexpr int ROUTE_THREADS = 128;
constexpr int MOE_MT = 32;          // rows of a tile
constexpr int MOE_NT = 64;          // columns of a tile
constexpr int MOE_KT = 32;          // k step
constexpr int MOE_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const T* __restrict__ x, const T* __restrict__ w, const float* __restrict__ correction,
                 int* __restrict__ ids, float* __restrict__ wts, int H, int n_out, int top) {
    extern __shared__ float z_s[];         // [n_out] logits, then scores; [n_out] choice scores
    float* c_s = z_s + n_out;
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* xr = x + (size_t)t * H;
    for (int o = warp; o < n_out; o += ROUTE_THREADS / 32) {
        const T* wr = w + (size_t)o * H;
        float acc = 0.f;
        for (int k = lane; k < H; k += 32) acc = fmaf(to_float(wr[k]), to_float(xr[k]), acc);
        acc = warp_sum(acc);
        if (lane == 0) z_s[o] = acc;
    }
    __syncthreads();
    if (warp != 0) return;
    float m = -INFINITY;
    for (int o = lane; o < n_out; o += 32) m = fmaxf(m, z_s[o]);
    m = warp_max(m);
    float sum = 0.f;
    for (int o = lane; o < n_out; o += 32) {
        const float e = expf(z_s[o] - m);
        z_s[o] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    for (int o = lane; o < n_out; o += 32) {
        const float s = z_s[o] / sum;
        z_s[o] = s;
        c_s[o] = s + (correction != nullptr ? correction[o] : 0.f);
    }
    __syncwarp();
    float chosen_sum = 0.f;
    for (int c = 0; c < top; ++c) {
        float best = -INFINITY;
        int bi = 0x7fffffff;
        for (int o = lane; o < n_out; o += 32) {
            const float v = c_s[o];
            if (v > best) { best = v; bi = o; }          // ascending o: the lower index wins a tie
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (bi == 0x7fffffff) bi = 0;                     // every score NaN: keep the indices in range
        if (lane == 0) {
            ids[(size_t)t * top + c] = bi;
            c_s[bi] = -INFINITY;
        }
        chosen_sum += z_s[bi];
        __syncwarp();
    }
    const float inv = 1.f / (chosen_sum + 1e-20f);
    for (int c = lane; c < top; c += 32) wts[(size_t)t * top + c] = z_s[ids[(size_t)t * top + c]] * inv;
}

// One CTA.  ids [P] router outputs of the P = tokens * top pairs.  Leaves pair_pos [P] (row of the pair in the grouped
// order, -1 for an identity expert), sorted_pair [cap] (pair of a grouped row, -1 for padding), tile_expert [cap / MT]
// and n_tiles.
__global__ void moe_align_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ pair_pos,
                                 int* __restrict__ sorted_pair, int* __restrict__ tile_expert, int* __restrict__ n_tiles,
                                 int cap) {
    extern __shared__ int a_s[];           // [E] counts, [E] offsets, [E] fill
    int* cnt = a_s;
    int* off = a_s + E;
    int* fill = a_s + 2 * E;
    __shared__ int total_s;
    for (int e = threadIdx.x; e < E; e += blockDim.x) { cnt[e] = 0; fill[e] = 0; }
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= 0 && e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int run = 0;
        for (int e = 0; e < E; ++e) {
            off[e] = run;
            const int tiles = (cnt[e] + MOE_MT - 1) / MOE_MT;
            for (int i = 0; i < tiles; ++i) tile_expert[run / MOE_MT + i] = e;
            run += tiles * MOE_MT;
        }
        total_s = run;
        *n_tiles = run / MOE_MT;
    }
    __syncthreads();
    const int total = min(total_s, cap);
    for (int i = threadIdx.x; i < total; i += blockDim.x) sorted_pair[i] = -1;
    __syncthreads();
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        int pos = -1;
        if (e >= 0 && e < E) {
            pos = off[e] + atomicAdd(&fill[e], 1);
            if (pos < cap) sorted_pair[pos] = p; else pos = -1;
        }
        pair_pos[p] = pos;
    }
}

// MODE 0: a[row] = x[sorted_pair[row] / top], out = relu(acc)^2 as T into act [cap, N]
// MODE 1: a[row] = act[row],                  out = acc as float into y [cap, N]
template <typename T, int MODE>
__global__ void __launch_bounds__(MOE_THREADS)
moe_gemm_kernel(const T* __restrict__ a, const T* __restrict__ w, void* __restrict__ out,
                const int* __restrict__ sorted_pair, const int* __restrict__ tile_expert,
                const int* __restrict__ n_tiles, int top, int N, int K) {
    const int tile = blockIdx.y;
    if (tile >= *n_tiles) return;
    __shared__ float a_s[MOE_MT][MOE_KT + 1];
    __shared__ float b_s[MOE_NT][MOE_KT + 1];
    __shared__ int row_s[MOE_MT];
    const int e = tile_expert[tile];
    const int n0 = blockIdx.x * MOE_NT;
    const int tid = threadIdx.x;
    if (tid < MOE_MT) {
        const int pr = sorted_pair[tile * MOE_MT + tid];
        row_s[tid] = pr < 0 ? -1 : (MODE == 0 ? pr / top : tile * MOE_MT + tid);
    }
    __syncthreads();
    const T* we = w + (size_t)e * N * K;
    const int ty = tid / 16, tx = tid % 16;        // rows 2 ty, 2 ty + 1; columns tx + 16 j
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
    for (int k0 = 0; k0 < K; k0 += MOE_KT) {
        for (int i = tid; i < MOE_MT * MOE_KT; i += MOE_THREADS) {
            const int r = i / MOE_KT, kk = i - r * MOE_KT;
            const int src = row_s[r];
            a_s[r][kk] = (src >= 0 && k0 + kk < K) ? to_float(a[(size_t)src * K + k0 + kk]) : 0.f;
        }
        for (int i = tid; i < MOE_NT * MOE_KT; i += MOE_THREADS) {
            const int c = i / MOE_KT, kk = i - c * MOE_KT;
            b_s[c][kk] = (n0 + c < N && k0 + kk < K) ? to_float(we[(size_t)(n0 + c) * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll 8
        for (int kk = 0; kk < MOE_KT; ++kk) {
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
        const int r = 2 * ty + i;
        if (row_s[r] < 0) continue;
        const size_t orow = (size_t)(tile * MOE_MT + r) * N;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int c = n0 + tx + 16 * j;
            if (c >= N) continue;
            if (MODE == 0) {
                const float v = fmaxf(acc[i][j], 0.f);
                static_cast<T*>(out)[orow + c] = from_float<T>(v * v);
            } else {
                static_cast<float*>(out)[orow + c] = acc[i][j];
            }
        }
    }
}

template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const T* __restrict__ x, const T* __restrict__ shared,
                                   const int* __restrict__ ids, const float* __restrict__ wts,
                                   const int* __restrict__ pair_pos, T* __restrict__ out, int H, int top, int E) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float acc = 0.f;
        for (int c = 0; c < top; ++c) {
            const size_t p = t * top + c;
            const float wgt = wts[p];
            if (ids[p] >= E) {
                acc = fmaf(wgt, to_float(x[t * H + i]), acc);
            } else {
                const int pos = pair_pos[p];
                if (pos >= 0) acc = fmaf(wgt, y[(size_t)pos * H + i], acc);
            }
        }
        if (shared != nullptr) acc += to_float(shared[t * H + i]);
        out[t * H + i] = from_float<T>(acc);
    }
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

extern "C" int fd_moe_tile_rows() { return MOE_MT; }

// x [T, H] and w [n_out, H] of type dtype (0 float32, 1 bfloat16); correction [n_out] float or null;
// ids [T, top] int32 and wts [T, top] float come back.
extern "C" int fd_moe_route(const void* x, const void* w, int dtype, const float* correction, int* ids, float* wts,
                            int T, int H, int n_out, int top, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(n_out >= 1 && top >= 1 && top <= n_out && n_out <= 4096, -2,
               "moe_route: %d choices of %d router outputs (at most 4096)", top, n_out);
    const size_t smem = 2 * (size_t)n_out * sizeof(float);
    if (dtype == 0)
        return launch("moe_route", moe_route_kernel<float>, dim3(T), dim3(ROUTE_THREADS), smem, stream, dim3(1, 1, 1),
                      (const float*)x, (const float*)w, correction, ids, wts, H, n_out, top);
    return launch("moe_route", moe_route_kernel<bf16>, dim3(T), dim3(ROUTE_THREADS), smem, stream, dim3(1, 1, 1),
                  (const bf16*)x, (const bf16*)w, correction, ids, wts, H, n_out, top);
}

// cap: rows of the grouped buffers, at least P rounded up to whole tiles plus one tile per expert.
extern "C" int fd_moe_align(const int* ids, int P, int E, int* pair_pos, int* sorted_pair, int* tile_expert,
                            int* n_tiles, int cap, cudaStream_t stream) {
    FD_REQUIRE(E >= 1 && E <= 4096, -2, "moe_align: %d experts (1..4096)", E);
    const long long worst = (long long)P + (long long)(E < P ? E : P) * (MOE_MT - 1);     // every group's last tile nearly empty
    FD_REQUIRE(cap % MOE_MT == 0 && (long long)cap >= (worst + MOE_MT - 1) / MOE_MT * MOE_MT, -2,
               "moe_align: %d grouped rows cannot hold %d pairs of %d experts", cap, P, E);
    return launch("moe_align", moe_align_kernel, dim3(1), dim3(1024), 3 * (size_t)E * sizeof(int), stream, dim3(1, 1, 1),
                  ids, P, E, pair_pos, sorted_pair, tile_expert, n_tiles, cap);
}

// mode 0: a = x [T, K], out = act [cap, N] (dtype) = relu(x W_e^T)^2;  mode 1: a = act [cap, K], out = y [cap, N] float.
// w [E, N, K].
extern "C" int fd_moe_gemm(const void* a, const void* w, void* out, int dtype, int mode, const int* sorted_pair,
                           const int* tile_expert, const int* n_tiles, int cap, int top, int N, int K,
                           cudaStream_t stream) {
    if (cap == 0) return 0;
    FD_REQUIRE(cap % MOE_MT == 0 && N > 0 && K > 0, -2, "moe_gemm: bad sizes");
    dim3 grid((N + MOE_NT - 1) / MOE_NT, cap / MOE_MT);
    FD_REQUIRE(grid.y <= 65535, -2, "moe_gemm: %d row tiles are too many", (int)grid.y);
#define FD_MG(T_, M_)                                                                                                \
    return launch("moe_gemm", moe_gemm_kernel<T_, M_>, grid, dim3(MOE_THREADS), 0, stream, dim3(1, 1, 1), (const T_*)a, \
                  (const T_*)w, out, sorted_pair, tile_expert, n_tiles, top, N, K)
    if (dtype == 0) { if (mode == 0) FD_MG(float, 0); FD_MG(float, 1); }
    if (mode == 0) FD_MG(bf16, 0);
    FD_MG(bf16, 1);
#undef FD_MG
}

extern "C" int fd_moe_combine(const float* y, const void* x, const void* shared, const int* ids, const float* wts,
                              const int* pair_pos, void* out, int dtype, int T, int H, int top, int E,
                              cudaStream_t stream) {
    if (T == 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (dtype == 0)
        return launch("moe_combine", moe_combine_kernel<float>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1), y,
                      (const float*)x, (const float*)shared, ids, wts, pair_pos, (float*)out, H, top, E);
    return launch("moe_combine", moe_combine_kernel<bf16>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1), y,
                  (const bf16*)x, (const bf16*)shared, ids, wts, pair_pos, (bf16*)out, H, top, E);
}
