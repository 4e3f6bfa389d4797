// A residual stream of several lanes: lanes [T, S, H] float.
//
// A sub-layer reads one mixture of the lanes and writes back into all of them:
//
//     u      = sum_s a[s] X[s]                        (read weights a [S])
//     y      = f(norm(u))                             (the sub-layer, other kernels)
//     X'[t]  = sum_s M[s, t] X[s] + b[t] * (g * y)    (M [S, S] indexed [from, to], b [S], g [H] per channel)
//
// lanes_norm is the one kernel between two sub-layers: it applies the update the
// sub-layer before left pending (y, g, M, b; all lanes from the old ones), then
// reads the mixture for the next one (a) and norms it:
//
//     out = u / sqrt(mean(u^2) + eps) * w
//
// Everything is float; y may be bfloat16 or float partial sums of a split
// product, `out` float or bfloat16.  `rows` gathers (the final norm at the
// wanted rows only, with a = ones: the lanes added up).  With S = 1, M = b = a =
// 1 this is the ordinary residual sum with a per-channel scale on the
// sub-layer's output.
#include "common.cuh"

namespace fd {

constexpr int LANES_MAX = 8;

template <typename T> __device__ __forceinline__ void load_vec(const T* p, float* v, int n);
template <> __device__ __forceinline__ void load_vec<float>(const float* p, float* v, int n) {
    if (n == 4) { const float4 r = *reinterpret_cast<const float4*>(p); v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
    else v[0] = p[0];
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float* v, int n) {
    if (n == 4) {
        const uint2 r = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&r.x), b = *reinterpret_cast<const __nv_bfloat162*>(&r.y);
        v[0] = __low2float(a); v[1] = __high2float(a); v[2] = __low2float(b); v[3] = __high2float(b);
    } else v[0] = __bfloat162float(p[0]);
}
template <typename T> __device__ __forceinline__ void store_vec(T* p, const float* v, int n);
template <> __device__ __forceinline__ void store_vec<float>(float* p, const float* v, int n) {
    if (n == 4) *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    else p[0] = v[0];
}
template <> __device__ __forceinline__ void store_vec<__nv_bfloat16>(__nv_bfloat16* p, const float* v, int n) {
    if (n == 4) {
        uint2 r;
        *reinterpret_cast<__nv_bfloat162*>(&r.x) = __floats2bfloat162_rn(v[0], v[1]);
        *reinterpret_cast<__nv_bfloat162*>(&r.y) = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(p) = r;
    } else p[0] = __float2bfloat16_rn(v[0]);
}

// LM: the most lanes this instantiation holds in registers (2, 4 or 8: with 8 the kernel needs 121 registers and two CTAs
// fit an SM; most models have 2 to 4 lanes).
// VEC = 4: a thread takes four neighbouring channels of every lane (16-byte loads and stores; H a multiple of 4 and
// all pointers 16-byte aligned); VEC = 1: any width.  The arithmetic per channel is the same in both.
template <typename TD, typename TO, int VEC, int LM>
__global__ void lanes_norm_kernel(const TD* __restrict__ y, int n_parts, size_t part_stride,
                                  const float* __restrict__ gain, const float* __restrict__ mix,
                                  const float* __restrict__ back, float* __restrict__ lanes, int write_lanes,
                                  const float* __restrict__ read, const float* __restrict__ w, float eps,
                                  TO* __restrict__ out, const int* __restrict__ rows, int H, int S) {
    extern __shared__ __align__(16) float ln_smem[];
    float* u_s = ln_smem;                          // H floats
    float* red = ln_smem + ((H + 3) & ~3);         // 33 floats
    float* c_s = red + 36;                         // mix [S * S], back [S], read [S]
    const int j = blockIdx.x;
    const int r = rows ? rows[j] : j;
    for (int i = threadIdx.x; i < S * S + 2 * S; i += blockDim.x) {
        float v;
        if (i < S * S) v = mix != nullptr ? mix[i] : ((i / S) == (i % S) ? 1.f : 0.f);
        else if (i < S * S + S) v = back != nullptr ? back[i - S * S] : 1.f;
        else v = read != nullptr ? read[i - S * S - S] : 1.f;
        c_s[i] = v;
    }
    __syncthreads();
    const float* m_s = c_s;
    const float* b_s = c_s + S * S;
    const float* a_s = b_s + S;
    float* base = lanes + (size_t)r * S * H;
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float x[LM][VEC];
#pragma unroll
        for (int s = 0; s < LM; ++s) {
            if (s < S) load_vec<float>(base + (size_t)s * H + i, x[s], VEC);
            else {
#pragma unroll
                for (int e = 0; e < VEC; ++e) x[s][e] = 0.f;
            }
        }
        float u[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) u[e] = 0.f;
        if (y != nullptr) {
            float z[VEC];
            load_vec<TD>(y + (size_t)r * H + i, z, VEC);
            for (int p = 1; p < n_parts; ++p) {
                float zp[VEC];
                load_vec<TD>(y + p * part_stride + (size_t)r * H + i, zp, VEC);
#pragma unroll
                for (int e = 0; e < VEC; ++e) z[e] += zp[e];
            }
            if (gain != nullptr) {
                float g[VEC];
                load_vec<float>(gain + i, g, VEC);
#pragma unroll
                for (int e = 0; e < VEC; ++e) z[e] *= g[e];
            }
#pragma unroll
            for (int t = 0; t < LM; ++t) {
                if (t < S) {
                    float n[VEC];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) n[e] = 0.f;
#pragma unroll
                    for (int s = 0; s < LM; ++s)
                        if (s < S) {
                            const float m = m_s[s * S + t];
#pragma unroll
                            for (int e = 0; e < VEC; ++e) n[e] = fmaf(m, x[s][e], n[e]);
                        }
                    const float bt = b_s[t], at = a_s[t];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) {
                        n[e] = fmaf(bt, z[e], n[e]);
                        u[e] = fmaf(at, n[e], u[e]);
                    }
                    if (write_lanes) store_vec<float>(base + (size_t)t * H + i, n, VEC);
                }
            }
        } else {
#pragma unroll
            for (int t = 0; t < LM; ++t)
                if (t < S) {
                    const float at = a_s[t];
#pragma unroll
                    for (int e = 0; e < VEC; ++e) u[e] = fmaf(at, x[t][e], u[e]);
                }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) { u_s[i + e] = u[e]; ss += u[e] * u[e]; }
    }
    const float total = block_sum(ss, red);
    const float rstd = rsqrtf(total / (float)H + eps);
    TO* orow = out + (size_t)j * H;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float wv[VEC], o[VEC];
        load_vec<float>(w + i, wv, VEC);
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = u_s[i + e] * rstd * wv[e];
        store_vec<TO>(orow + i, o, VEC);
    }
}

// lanes[t, s, :] = src[t, :] for every lane s.
__global__ void lanes_fill_kernel(const float* __restrict__ src, float* __restrict__ lanes, int H, int S) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = src[t * H + i];
        for (int s = 0; s < S; ++s) lanes[(t * S + s) * H + i] = v;
    }
}

// out[t, :] = sum over the lanes, after the pending update if there is one (for traces and tests).
template <typename TD>
__global__ void lanes_sum_kernel(const TD* __restrict__ y, const float* __restrict__ gain, const float* __restrict__ mix,
                                 const float* __restrict__ back, const float* __restrict__ lanes, float* __restrict__ out,
                                 int H, int S) {
    const size_t t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float z = 0.f;
        if (y != nullptr) {
            z = to_float(y[t * H + i]);
            if (gain != nullptr) z *= gain[i];
        }
        float acc = 0.f;
        for (int to = 0; to < S; ++to) {
            float n = 0.f;
            for (int s = 0; s < S; ++s) {
                const float m = y == nullptr || mix == nullptr ? (s == to ? 1.f : 0.f) : mix[s * S + to];
                n = fmaf(m, lanes[(t * S + s) * H + i], n);
            }
            if (y != nullptr) n = fmaf(back != nullptr ? back[to] : 1.f, z, n);
            acc += n;
        }
        out[t * H + i] = acc;
    }
}

}  // namespace fd

using namespace fd;
typedef __nv_bfloat16 bf16;

// y (y_dtype: 0 float32, 1 bfloat16; n_parts > 1: float partial sums part_stride elements apart) may be null: nothing
// pending.  gain [H], mix [S, S], back [S], read [S] are float and may be null (ones; mix: the unit matrix).  w [H]
// float.  out (out_dtype) [n_out, H]; rows [n_out] or null.
extern "C" int fd_lanes_norm(const void* y, int y_dtype, int n_parts, long long part_stride, const float* gain,
                             const float* mix, const float* back, float* lanes, int write_lanes, const float* read,
                             const float* w, float eps, void* out, int out_dtype, const int* rows, int n_out, int H, int S,
                             cudaStream_t stream) {
    if (n_out == 0) return 0;
    FD_REQUIRE(H > 0 && S >= 1 && S <= LANES_MAX, -2, "lanes_norm: width %d, %d lanes (1..%d)", H, S, LANES_MAX);
    FD_REQUIRE(y == nullptr || (n_parts >= 1 && (n_parts == 1 || y_dtype == 0)), -2, "lanes_norm: partial sums must be float");
    const size_t smem = (((H + 3) & ~3) + 36 + S * S + 2 * S) * sizeof(float);
    FD_REQUIRE(smem <= 200 * 1024, -2, "lanes_norm: width %d needs %zu bytes of shared memory (max 200 KB)", H, smem);
    const bool vec = H % 4 == 0 && (size_t)part_stride % 4 == 0 && (uintptr_t)y % 16 == 0 && (uintptr_t)gain % 16 == 0 &&
                     (uintptr_t)lanes % 16 == 0 && (uintptr_t)w % 16 == 0 && (uintptr_t)out % 16 == 0;
    const int threads = vec ? (H >= 2048 ? 256 : 128) : (H >= 2048 ? 512 : (H >= 512 ? 256 : 128));
#define FD_LN1(TD_, TO_, V_)                                                                                         \
    do {                                                                                                             \
        auto k = S <= 2 ? lanes_norm_kernel<TD_, TO_, V_, 2> : (S <= 4 ? lanes_norm_kernel<TD_, TO_, V_, 4>             \
                                                                       : lanes_norm_kernel<TD_, TO_, V_, 8>);           \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        return launch("lanes_norm", k, dim3(n_out), dim3(threads), smem, stream, dim3(1, 1, 1), (const TD_*)y, n_parts, \
                      (size_t)part_stride, gain, mix, back, lanes, write_lanes, read, w, eps, (TO_*)out, rows, H, S); \
    } while (0)
#define FD_LN(TD_, TO_) do { if (vec) FD_LN1(TD_, TO_, 4); FD_LN1(TD_, TO_, 1); } while (0)
    if (y_dtype == 0 && out_dtype == 0) FD_LN(float, float);
    if (y_dtype == 0 && out_dtype == 1) FD_LN(float, bf16);
    if (y_dtype == 1 && out_dtype == 1) FD_LN(bf16, bf16);
#undef FD_LN
#undef FD_LN1
    return fail(-2, "lanes_norm: unsupported dtypes y=%d out=%d", y_dtype, out_dtype);
}

extern "C" int fd_lanes_fill(const float* src, float* lanes, int T, int H, int S, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(H > 0 && S >= 1, -2, "lanes_fill: width %d, %d lanes", H, S);
    return launch("lanes_fill", lanes_fill_kernel, dim3(T), dim3(H >= 512 ? 256 : 128), 0, stream, dim3(1, 1, 1), src,
                  lanes, H, S);
}

extern "C" int fd_lanes_sum(const void* y, int y_dtype, const float* gain, const float* mix, const float* back,
                            const float* lanes, float* out, int T, int H, int S, cudaStream_t stream) {
    if (T == 0) return 0;
    FD_REQUIRE(H > 0 && S >= 1, -2, "lanes_sum: width %d, %d lanes", H, S);
    if (y_dtype == 0)
        return launch("lanes_sum", lanes_sum_kernel<float>, dim3(T), dim3(128), 0, stream, dim3(1, 1, 1), (const float*)y,
                      gain, mix, back, lanes, out, H, S);
    return launch("lanes_sum", lanes_sum_kernel<bf16>, dim3(T), dim3(128), 0, stream, dim3(1, 1, 1), (const bf16*)y, gain,
                  mix, back, lanes, out, H, S);
}
