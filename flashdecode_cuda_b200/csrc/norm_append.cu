// What stands between an attention mixer's packed projection and its attention
// kernel when nothing is rotated: q and k are each normed over their WHOLE
// projection (all heads at once, before they are split into heads), q goes to
// its buffer, k and v to the paged cache at the token's position.
//
//   proj  [T, ld]: columns [0, nq) are q, [nq, nq + nk) are k, [nq + nk, nq + nk + nv) are v
//   q_out [T, nq]                      q / sqrt(mean(q^2) + eps) * q_w   (q_w null: q as it is)
//   k_pool [blocks, n_kv, block_size, nk / n_kv]   the same with k_w
//   v_pool [blocks, n_kv, block_size, nv / n_kv]   nv == 0: no values are kept (the keys serve as values)
//   k_rows [T, nk] (optional)          the normed k once more as plain rows, for a product that follows
// nq == 0: there is no q (the rows are keys and values only).
// q_count / k_count: how many of q's and k's columns are real (the rest are zero padding that brings head sizes to
// multiples of 8): the means of the squares are taken over these counts.  0: all of them.
//
// With n_kv = 1 and nv = 0 the "key" is any normed vector per position, e.g. the
// low-rank latent that a latent-attention mixer makes its keys and values from.
// Sums of squares and the norm are float; a CTA per token.
#include "common.cuh"

namespace fd {

template <typename T>
__global__ void norm_append_kernel(const T* __restrict__ proj, int ld, T* __restrict__ q_out,
                                   const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                   const int* __restrict__ tok_row, const int* __restrict__ tok_pos,
                                   const int* __restrict__ row_slot, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                   const int* __restrict__ block_table, int max_blocks, int num_blocks, int block_size,
                                   int nq, int nk, int nv, int n_kv, int write_kv, T* __restrict__ k_rows, int q_count, int k_count,
                                   int* status) {
    __shared__ float red[40];
    const int t = blockIdx.x;
    const int slot = row_slot[tok_row[t]];
    if (slot < 0) return;             // padding row of a fixed-size batch
    const T* row = proj + (size_t)t * ld;
    float sq = 0.f, sk = 0.f;
    if (q_w != nullptr)
        for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = to_float(row[i]); sq += v * v; }
    if (k_w != nullptr)
        for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = to_float(row[nq + i]); sk += v * v; }
    const float rq = q_w != nullptr ? rsqrtf(block_sum(sq, red) / (float)q_count + eps) : 1.f;
    const float rk = k_w != nullptr ? rsqrtf(block_sum(sk, red) / (float)k_count + eps) : 1.f;
    T* qo = q_out + (size_t)t * nq;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) {
        const float v = to_float(row[i]);
        qo[i] = q_w != nullptr ? from_float<T>(v * rq * q_w[i]) : row[i];
    }
    if (k_rows != nullptr) {
        T* kr = k_rows + (size_t)t * nk;
        for (int i = threadIdx.x; i < nk; i += blockDim.x) {
            const float v = to_float(row[nq + i]);
            kr[i] = k_w != nullptr ? from_float<T>(v * rk * k_w[i]) : row[nq + i];
        }
    }
    if (!write_kv) return;
    const int pos = tok_pos[t];
    const int blk = pos >= 0 && pos / block_size < max_blocks ? block_table[(size_t)slot * max_blocks + pos / block_size] : -1;
    if (blk < 0 || blk >= num_blocks) {
        if (threadIdx.x == 0) set_status(status, STATUS_BAD_BLOCK);
        return;
    }
    const int d = nk / n_kv;
    T* kd = k_pool + ((size_t)blk * n_kv * block_size + (pos % block_size)) * d;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int h = i / d, j = i - h * d;
        const float v = to_float(row[nq + i]);
        kd[(size_t)h * block_size * d + j] = k_w != nullptr ? from_float<T>(v * rk * k_w[i]) : row[nq + i];
    }
    if (nv > 0) {
        const int dv = nv / n_kv;
        T* vd = v_pool + ((size_t)blk * n_kv * block_size + (pos % block_size)) * dv;
        for (int i = threadIdx.x; i < nv; i += blockDim.x) {
            const int h = i / dv, j = i - h * dv;
            vd[(size_t)h * block_size * dv + j] = row[nq + nk + i];
        }
    }
}

// The same in 16-byte pieces: every segment, head size and row stride a multiple of VEC = 16 / sizeof(T) elements and
// every pointer 16-byte aligned.  The arithmetic per element is that of the kernel above.
template <typename T>
__global__ void norm_append_vec_kernel(const T* __restrict__ proj, int ld, T* __restrict__ q_out,
                                       const float* __restrict__ q_w, const float* __restrict__ k_w, float eps,
                                       const int* __restrict__ tok_row, const int* __restrict__ tok_pos,
                                       const int* __restrict__ row_slot, T* __restrict__ k_pool, T* __restrict__ v_pool,
                                       const int* __restrict__ block_table, int max_blocks, int num_blocks, int block_size,
                                       int nq, int nk, int nv, int n_kv, int write_kv, T* __restrict__ k_rows, int q_count, int k_count,
                                   int* status) {
    constexpr int VEC = 16 / sizeof(T);
    __shared__ float red[40];
    const int t = blockIdx.x;
    const int slot = row_slot[tok_row[t]];
    if (slot < 0) return;
    const T* row = proj + (size_t)t * ld;
    auto load = [&](int at, float* f) -> uint4 {
        const uint4 raw = *reinterpret_cast<const uint4*>(row + at);
        const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int j = 0; j < VEC; ++j) f[j] = to_float(e[j]);
        return raw;
    };
    float sq = 0.f, sk = 0.f;
    if (q_w != nullptr)
        for (int c = threadIdx.x * VEC; c < nq; c += blockDim.x * VEC) {
            float f[VEC];
            load(c, f);
#pragma unroll
            for (int j = 0; j < VEC; ++j) sq += f[j] * f[j];
        }
    if (k_w != nullptr)
        for (int c = threadIdx.x * VEC; c < nk; c += blockDim.x * VEC) {
            float f[VEC];
            load(nq + c, f);
#pragma unroll
            for (int j = 0; j < VEC; ++j) sk += f[j] * f[j];
        }
    const float rq = q_w != nullptr ? rsqrtf(block_sum(sq, red) / (float)q_count + eps) : 1.f;
    const float rk = k_w != nullptr ? rsqrtf(block_sum(sk, red) / (float)k_count + eps) : 1.f;
    // one piece of the row at `at`, scaled by r * w[...] if w is given, as it goes to memory
    auto piece = [&](int at, const float* w, float r) -> uint4 {
        float f[VEC];
        const uint4 raw = load(at, f);
        if (w == nullptr) return raw;
        uint4 o;
        T* e = reinterpret_cast<T*>(&o);
#pragma unroll
        for (int j = 0; j < VEC; ++j) e[j] = from_float<T>(f[j] * r * w[j]);
        return o;
    };
    for (int c = threadIdx.x * VEC; c < nq; c += blockDim.x * VEC)
        *reinterpret_cast<uint4*>(q_out + (size_t)t * nq + c) = piece(c, q_w ? q_w + c : nullptr, rq);
    T* kd = nullptr;
    T* vd = nullptr;
    const int d = nk / n_kv, dv = nv / n_kv;
    if (write_kv) {
        const int pos = tok_pos[t];
        const int blk = pos >= 0 && pos / block_size < max_blocks ? block_table[(size_t)slot * max_blocks + pos / block_size] : -1;
        if (blk < 0 || blk >= num_blocks) {
            if (threadIdx.x == 0) set_status(status, STATUS_BAD_BLOCK);
        } else {
            kd = k_pool + ((size_t)blk * n_kv * block_size + (pos % block_size)) * d;
            if (nv > 0) vd = v_pool + ((size_t)blk * n_kv * block_size + (pos % block_size)) * dv;
        }
    }
    if (kd != nullptr || k_rows != nullptr)
        for (int c = threadIdx.x * VEC; c < nk; c += blockDim.x * VEC) {
            const uint4 o = piece(nq + c, k_w ? k_w + c : nullptr, rk);
            if (k_rows != nullptr) *reinterpret_cast<uint4*>(k_rows + (size_t)t * nk + c) = o;
            if (kd != nullptr) {
                const int h = c / d, j = c - h * d;
                *reinterpret_cast<uint4*>(kd + (size_t)h * block_size * d + j) = o;
            }
        }
    if (vd != nullptr)
        for (int c = threadIdx.x * VEC; c < nv; c += blockDim.x * VEC) {
            const int h = c / dv, j = c - h * dv;
            *reinterpret_cast<uint4*>(vd + (size_t)h * block_size * dv + j) = *reinterpret_cast<const uint4*>(row + nq + nk + c);
        }
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// dtype (0 float32, 1 bfloat16): proj, q_out and the pools alike.  q_w [nq], k_w [nk]: float or null.
extern "C" int fd_norm_append(const void* proj, int ld, void* q_out, int dtype, const float* q_w, const float* k_w,
                              float eps, const int* tok_row, const int* tok_pos, const int* row_slot, void* k_pool,
                              void* v_pool, const int* block_table, int max_blocks, int num_blocks, int block_size, int T,
                              int nq, int nk, int nv, int n_kv, int write_kv, void* k_rows, int q_count, int k_count,
                              int* status, cudaStream_t stream) {
    if (T == 0) return 0;
    if (q_count <= 0) q_count = nq;
    if (k_count <= 0) k_count = nk;
    FD_REQUIRE(nq >= 0 && (nq == 0 || q_out != nullptr) && nk > 0 && nv >= 0 && n_kv > 0 && nk % n_kv == 0 && nv % n_kv == 0 && ld >= nq + nk + nv, -2,
               "norm_append: %d + %d + %d columns of %d for %d key heads", nq, nk, nv, ld, n_kv);
    FD_REQUIRE(block_size > 0 && (nv == 0 || v_pool != nullptr), -2, "norm_append: bad cache arguments");
    const int threads = nq + nk >= 1024 ? 256 : 128;
    const int vec = dtype == 0 ? 4 : 8;
    const int d = nk / n_kv, dv = nv / n_kv;
    auto al = [](const void* p) { return (uintptr_t)p % 16 == 0; };
    if (nq % vec == 0 && d % vec == 0 && dv % vec == 0 && ld % vec == 0 && al(proj) && al(q_out) && al(k_pool) && al(v_pool) &&
        al(k_rows) && al(q_w) && al(k_w)) {
        if (dtype == 0)
            return launch("norm_append", norm_append_vec_kernel<float>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                          (const float*)proj, ld, (float*)q_out, q_w, k_w, eps, tok_row, tok_pos, row_slot, (float*)k_pool,
                          (float*)v_pool, block_table, max_blocks, num_blocks, block_size, nq, nk, nv, n_kv, write_kv,
                          (float*)k_rows, q_count, k_count, status);
        return launch("norm_append", norm_append_vec_kernel<bf16>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                      (const bf16*)proj, ld, (bf16*)q_out, q_w, k_w, eps, tok_row, tok_pos, row_slot, (bf16*)k_pool,
                      (bf16*)v_pool, block_table, max_blocks, num_blocks, block_size, nq, nk, nv, n_kv, write_kv,
                      (bf16*)k_rows, q_count, k_count, status);
    }
    if (dtype == 0)
        return launch("norm_append", norm_append_kernel<float>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                      (const float*)proj, ld, (float*)q_out, q_w, k_w, eps, tok_row, tok_pos, row_slot, (float*)k_pool,
                      (float*)v_pool, block_table, max_blocks, num_blocks, block_size, nq, nk, nv, n_kv, write_kv,
                      (float*)k_rows, q_count, k_count, status);
    return launch("norm_append", norm_append_kernel<bf16>, dim3(T), dim3(threads), 0, stream, dim3(1, 1, 1),
                  (const bf16*)proj, ld, (bf16*)q_out, q_w, k_w, eps, tok_row, tok_pos, row_slot, (bf16*)k_pool,
                  (bf16*)v_pool, block_table, max_blocks, num_blocks, block_size, nq, nk, nv, n_kv, write_kv,
                  (bf16*)k_rows, q_count, k_count, status);
}
