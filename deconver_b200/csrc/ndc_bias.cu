// Bias of the channels-first linear layer: y[b, c, :] += bias[c], and its gradient
// gbias[c] = sum over samples and positions of gy[b, c, :]; and the same bias fused with the
// erf-form GELU that follows the first projection of the network's MLP: a = gelu(h + bias) in
// one pass over h, and gh = ga * gelu'(h + bias) with the bias gradient in one pass over (ga, h).
//
// The 1x1 projection itself is a library GEMM; what the library adds around it, a broadcast add
// that is not vectorised and a reduction with one block per output, is slow at the small per-GPU
// batches of a batch-sharded training step.  Both are plain HBM-bound passes here: every
// (sample, channel) slab is split over as many CTAs as fill the GPU, 16-byte accesses, sums in a
// fixed order (no atomics).
#include <cstdarg>
#include <cstdio>

#include "ndc_b200.h"
#include "ndc_common.cuh"
#include "ndc_slab.cuh"

namespace {

using namespace ndc::slab;

thread_local char g_bias_err[256] = "";

int bias_fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_bias_err, sizeof(g_bias_err), fmt, ap);
    va_end(ap);
    return status;
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) bias_add_kernel(T* __restrict__ y, long long sp, int channels,
                                                       int nsplit, const float* __restrict__ bias) {
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    T* ys = y + slab * sp;
    const float b = bias[slab % channels];
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    if (VEC) {
        for (long long i = begin + (long long)threadIdx.x * N; i < end; i += (long long)kNT * N) {
            float v[N];
            Vec16<T>::unpack(*reinterpret_cast<const typename Vec16<T>::raw*>(ys + i), v);
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] += b;
            *reinterpret_cast<typename Vec16<T>::raw*>(ys + i) = Vec16<T>::pack(v);
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT)
            ys[i] = ndc::from_f32<T>(ndc::to_f32(ys[i]) + b);
    }
}

// partial[slab * nsplit + part] = sum of the part
template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) bias_grad_partial_kernel(const T* __restrict__ gy, long long sp,
                                                                int nsplit, float* __restrict__ partial) {
    __shared__ float scratch[2 * kNT / 32];
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    const T* gs = gy + slab * sp;
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    float s1 = 0.0f, s2 = 0.0f;     // two interleaved sums: shorter dependency chains
    if (VEC) {
        for (long long i = begin + (long long)threadIdx.x * N; i < end; i += (long long)kNT * N) {
            float v[N];
            Vec16<T>::unpack(__ldg(reinterpret_cast<const typename Vec16<T>::raw*>(gs + i)), v);
#pragma unroll
            for (int j = 0; j < N; j += 2) { s1 += v[j]; s2 += v[j + 1]; }
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT) s1 += ndc::to_f32(gs[i]);
    }
    cta_sum2(s1, s2, scratch);
    if (threadIdx.x == 0) partial[slab * nsplit + part] = s1 + s2;
}

__global__ void bias_grad_final_kernel(const float* __restrict__ partial, int batch, int channels, int nsplit,
                                       float* __restrict__ gbias) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float s = 0.0f;
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < nsplit; ++i) s += partial[((long long)b * channels + c) * nsplit + i];
    gbias[c] = s;
}

constexpr int kGeluUnroll = 4;     // 16-byte loads in flight per thread and tensor

// erf by the rational approximation 7.1.26 of Abramowitz and Stegun (absolute error below
// 1.5e-7 over the real line), with the hardware reciprocal and exponential: 1 - erf(|x|) =
// t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) exp(-x^2), t = 1 / (1 + p |x|).  The library erff plus
// a separate exponential made the GELU passes arithmetic-bound at 3.6-4 TB/s.  `e` returns
// exp(-x^2), which the derivative needs as well.
__device__ __forceinline__ float erf_as(float x, float& e) {
    const float ax = fabsf(x);
    const float t = __frcp_rn(fmaf(0.3275911f, ax, 1.0f));
    float p = fmaf(1.061405429f, t, -1.453152027f);
    p = fmaf(p, t, 1.421413741f);
    p = fmaf(p, t, -0.284496736f);
    p = fmaf(p, t, 0.254829592f);
    e = __expf(-ax * ax);
    return copysignf(fmaf(-p * t, e, 1.0f), x);
}
__device__ __forceinline__ float gelu_f(float u) {
    float e;
    return 0.5f * u * (1.0f + erf_as(u * 0.70710678118654752440f, e));
}
// d/du [u * Phi(u)] = Phi(u) + u * phi(u), phi(u) = exp(-u^2 / 2) / sqrt(2 pi)
__device__ __forceinline__ float gelu_grad_f(float u) {
    float e;
    const float cdf = 0.5f * (1.0f + erf_as(u * 0.70710678118654752440f, e));
    return fmaf(u, 0.39894228040143267794f * e, cdf);
}

// The same arithmetic on two elements at a time: the adds, multiplies and multiply-adds are
// two-lane `*.rn.f32x2` instructions (each lane rounds like the scalar form), the reciprocal and
// the exponential stay per lane.  About 12 instructions per element instead of 20: the
// vectorised GELU passes were bound by instruction issue, not by memory.
typedef unsigned long long f2;
__device__ __forceinline__ f2 f2_pack(float lo, float hi) {
    f2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void f2_unpack(f2 p, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ f2 f2_fma(f2 a, f2 b, f2 c) {
    f2 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ f2 f2_mul(f2 a, f2 b) {
    f2 r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2 f2_add(f2 a, f2 b) {
    f2 r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ f2 f2_dup(float v) { return f2_pack(v, v); }
__device__ __forceinline__ float ex2_approx(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// cdf = Phi(u) for both lanes; e = exp(-u^2 / 2) for both lanes
__device__ __forceinline__ f2 gelu_cdf2(f2 u, f2& e) {
    float u0, u1;
    f2_unpack(u, u0, u1);
    const f2 au = f2_pack(fabsf(u0), fabsf(u1));
    // x = u / sqrt(2): t = 1 / (1 + p |x|), e = exp(-x^2) = exp2(-u^2 * log2(e) / 2)
    float d0, d1;
    f2_unpack(f2_fma(f2_dup(0.3275911f * 0.70710678118654752440f), au, f2_dup(1.0f)), d0, d1);
    const f2 t = f2_pack(__frcp_rn(d0), __frcp_rn(d1));
    f2 p = f2_fma(f2_dup(1.061405429f), t, f2_dup(-1.453152027f));
    p = f2_fma(p, t, f2_dup(1.421413741f));
    p = f2_fma(p, t, f2_dup(-0.284496736f));
    p = f2_fma(p, t, f2_dup(0.254829592f));
    float s0, s1;
    f2_unpack(f2_mul(f2_mul(u, u), f2_dup(-0.72134752044448170368f)), s0, s1);
    e = f2_pack(ex2_approx(s0), ex2_approx(s1));
    // 1 - erf(|x|) = p t e;  Phi = 0.5 + copysign(0.5 - 0.5 p t e, u)
    float h0, h1;
    f2_unpack(f2_fma(f2_mul(p, t), f2_mul(e, f2_dup(-0.5f)), f2_dup(0.5f)), h0, h1);
    return f2_add(f2_pack(copysignf(h0, u0), copysignf(h1, u1)), f2_dup(0.5f));
}
__device__ __forceinline__ f2 gelu2(f2 u) {
    f2 e;
    return f2_mul(u, gelu_cdf2(u, e));
}
__device__ __forceinline__ f2 gelu_grad2(f2 u) {
    f2 e;
    const f2 cdf = gelu_cdf2(u, e);
    return f2_fma(u, f2_mul(e, f2_dup(0.39894228040143267794f)), cdf);
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) bias_gelu_fwd_kernel(const T* __restrict__ h, T* __restrict__ out,
                                                            long long sp, int channels, int nsplit,
                                                            const float* __restrict__ bias) {
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    const T* hs = h + slab * sp;
    T* os = out + slab * sp;
    const float b = bias ? bias[slab % channels] : 0.0f;
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    if (VEC) {
        // kGeluUnroll independent 16-byte loads per thread are issued before the first erf: the
        // arithmetic of one vector is long enough to leave the memory pipe idle otherwise
        typedef typename Vec16<T>::raw Raw;
        const long long step = (long long)kNT * N;
        const f2 b2 = f2_dup(b);
        long long i = begin + (long long)threadIdx.x * N;
        for (; i + (kGeluUnroll - 1) * step < end; i += kGeluUnroll * step) {
            Raw r[kGeluUnroll];
#pragma unroll
            for (int u = 0; u < kGeluUnroll; ++u) r[u] = __ldg(reinterpret_cast<const Raw*>(hs + i + u * step));
#pragma unroll
            for (int u = 0; u < kGeluUnroll; ++u) {
                float v[N];
                Vec16<T>::unpack(r[u], v);
#pragma unroll
                for (int j = 0; j < N; j += 2)
                    f2_unpack(gelu2(f2_add(f2_pack(v[j], v[j + 1]), b2)), v[j], v[j + 1]);
                *reinterpret_cast<Raw*>(os + i + u * step) = Vec16<T>::pack(v);
            }
        }
        for (; i < end; i += step) {
            float v[N];
            Vec16<T>::unpack(__ldg(reinterpret_cast<const Raw*>(hs + i)), v);
#pragma unroll
            for (int j = 0; j < N; j += 2)
                f2_unpack(gelu2(f2_add(f2_pack(v[j], v[j + 1]), b2)), v[j], v[j + 1]);
            *reinterpret_cast<Raw*>(os + i) = Vec16<T>::pack(v);
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT)
            os[i] = ndc::from_f32<T>(gelu_f(ndc::to_f32(hs[i]) + b));
    }
}

// gh = ga * gelu'(h + bias), rounded to the storage type; partial[slab * nsplit + part] = the
// sum of the rounded values of the part (what a separate pass over gh would add up)
template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) bias_gelu_bwd_kernel(const T* __restrict__ ga, const T* __restrict__ h,
                                                            T* __restrict__ gh, long long sp, int channels,
                                                            int nsplit, const float* __restrict__ bias,
                                                            float* __restrict__ partial) {
    __shared__ float scratch[2 * kNT / 32];
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    const T* gs = ga + slab * sp;
    const T* hs = h + slab * sp;
    T* os = gh + slab * sp;
    const float b = bias ? bias[slab % channels] : 0.0f;
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    float s1 = 0.0f, s2 = 0.0f;
    if (VEC) {
        typedef typename Vec16<T>::raw Raw;
        const long long step = (long long)kNT * N;
        const f2 b2 = f2_dup(b);
        auto one = [&](const Raw& rg, const Raw& rh, long long at) {
            float g[N], v[N];
            Vec16<T>::unpack(rg, g);
            Vec16<T>::unpack(rh, v);
#pragma unroll
            for (int j = 0; j < N; j += 2)
                f2_unpack(f2_mul(f2_pack(g[j], g[j + 1]), gelu_grad2(f2_add(f2_pack(v[j], v[j + 1]), b2))),
                          g[j], g[j + 1]);
            const Raw r = Vec16<T>::pack(g);
            *reinterpret_cast<Raw*>(os + at) = r;
            Vec16<T>::unpack(r, g);
#pragma unroll
            for (int j = 0; j < N; j += 2) { s1 += g[j]; s2 += g[j + 1]; }
        };
        long long i = begin + (long long)threadIdx.x * N;
        for (; i + (kGeluUnroll - 1) * step < end; i += kGeluUnroll * step) {
            Raw rg[kGeluUnroll], rh[kGeluUnroll];
#pragma unroll
            for (int u = 0; u < kGeluUnroll; ++u) {
                rg[u] = __ldg(reinterpret_cast<const Raw*>(gs + i + u * step));
                rh[u] = __ldg(reinterpret_cast<const Raw*>(hs + i + u * step));
            }
#pragma unroll
            for (int u = 0; u < kGeluUnroll; ++u) one(rg[u], rh[u], i + u * step);
        }
        for (; i < end; i += step)
            one(__ldg(reinterpret_cast<const Raw*>(gs + i)), __ldg(reinterpret_cast<const Raw*>(hs + i)), i);
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT) {
            const T r = ndc::from_f32<T>(ndc::to_f32(gs[i]) * gelu_grad_f(ndc::to_f32(hs[i]) + b));
            os[i] = r;
            s1 += ndc::to_f32(r);
        }
    }
    if (partial) {
        cta_sum2(s1, s2, scratch);
        if (threadIdx.x == 0) partial[slab * nsplit + part] = s1 + s2;
    }
}

int check(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype) {
    if (batch <= 0 || channels <= 0 || spatial <= 0)
        return bias_fail(NDC_ERR_INVALID, "bias: batch, channels and spatial size must be positive");
    if (dtype != NDC_F32 && dtype != NDC_BF16)
        return bias_fail(NDC_ERR_INVALID, "bias: dtype must be NDC_F32 or NDC_BF16");
    if ((long long)batch * channels * kMaxSplit > 0x7fffffffLL)
        return bias_fail(NDC_ERR_UNSUPPORTED, "bias: batch * channels is too large");
    return NDC_OK;
}

}  // namespace

extern "C" {

const char* ndc_bias_last_error(void) { return g_bias_err; }

size_t ndc_bias_grad_workspace_bytes(int32_t batch, int32_t channels) {
    if (batch <= 0 || channels <= 0) return 0;
    return (size_t)batch * channels * kMaxSplit * sizeof(float);
}

int ndc_bias_add(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, void* y,
                 const float* bias, void* stream) {
    if (!y || !bias) return bias_fail(NDC_ERR_INVALID, "bias add: y and bias must not be NULL");
    int st = check(batch, channels, spatial, dtype);
    if (st != NDC_OK) return st;
    const long long slabs = (long long)batch * channels;
    const int nsplit = choose_split(slabs, spatial);
    const bool vec = spatial % (dtype == NDC_BF16 ? 8 : 4) == 0 && ((uintptr_t)y % 16) == 0;
    const unsigned grid = (unsigned)(slabs * nsplit);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == NDC_F32) {
        if (vec) bias_add_kernel<float, true><<<grid, kNT, 0, s>>>((float*)y, spatial, channels, nsplit, bias);
        else bias_add_kernel<float, false><<<grid, kNT, 0, s>>>((float*)y, spatial, channels, nsplit, bias);
    } else {
        typedef __nv_bfloat16 bf16;
        if (vec) bias_add_kernel<bf16, true><<<grid, kNT, 0, s>>>((bf16*)y, spatial, channels, nsplit, bias);
        else bias_add_kernel<bf16, false><<<grid, kNT, 0, s>>>((bf16*)y, spatial, channels, nsplit, bias);
    }
    ndc::launched();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return bias_fail(NDC_ERR_CUDA, "bias add: %s", cudaGetErrorString(e));
    return NDC_OK;
}

int ndc_bias_grad(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void* gy,
                  float* gbias, void* workspace, size_t workspace_bytes, void* stream) {
    if (!gy || !gbias) return bias_fail(NDC_ERR_INVALID, "bias gradient: gy and gbias must not be NULL");
    int st = check(batch, channels, spatial, dtype);
    if (st != NDC_OK) return st;
    if (!workspace || workspace_bytes < ndc_bias_grad_workspace_bytes(batch, channels))
        return bias_fail(NDC_ERR_WORKSPACE, "bias gradient: workspace of %zu bytes needed",
                         ndc_bias_grad_workspace_bytes(batch, channels));
    const long long slabs = (long long)batch * channels;
    const int nsplit = choose_split(slabs, spatial);
    const bool vec = spatial % (dtype == NDC_BF16 ? 8 : 4) == 0 && ((uintptr_t)gy % 16) == 0;
    const unsigned grid = (unsigned)(slabs * nsplit);
    cudaStream_t s = (cudaStream_t)stream;
    float* partial = (float*)workspace;
    if (dtype == NDC_F32) {
        if (vec) bias_grad_partial_kernel<float, true><<<grid, kNT, 0, s>>>((const float*)gy, spatial, nsplit, partial);
        else bias_grad_partial_kernel<float, false><<<grid, kNT, 0, s>>>((const float*)gy, spatial, nsplit, partial);
    } else {
        typedef __nv_bfloat16 bf16;
        if (vec) bias_grad_partial_kernel<bf16, true><<<grid, kNT, 0, s>>>((const bf16*)gy, spatial, nsplit, partial);
        else bias_grad_partial_kernel<bf16, false><<<grid, kNT, 0, s>>>((const bf16*)gy, spatial, nsplit, partial);
    }
    bias_grad_final_kernel<<<(channels + 127) / 128, 128, 0, s>>>(partial, batch, channels, nsplit, gbias);
    ndc::launched(2);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return bias_fail(NDC_ERR_CUDA, "bias gradient: %s", cudaGetErrorString(e));
    return NDC_OK;
}

int ndc_bias_gelu_fwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void* h,
                      const float* bias, void* out, void* stream) {
    if (!h || !out) return bias_fail(NDC_ERR_INVALID, "bias gelu: h and out must not be NULL");
    int st = check(batch, channels, spatial, dtype);
    if (st != NDC_OK) return st;
    const long long slabs = (long long)batch * channels;
    const int nsplit = choose_split(slabs, spatial);
    const bool vec = spatial % (dtype == NDC_BF16 ? 8 : 4) == 0 && ((uintptr_t)h % 16) == 0 &&
                     ((uintptr_t)out % 16) == 0;
    const unsigned grid = (unsigned)(slabs * nsplit);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == NDC_F32) {
        if (vec) bias_gelu_fwd_kernel<float, true><<<grid, kNT, 0, s>>>((const float*)h, (float*)out, spatial, channels, nsplit, bias);
        else bias_gelu_fwd_kernel<float, false><<<grid, kNT, 0, s>>>((const float*)h, (float*)out, spatial, channels, nsplit, bias);
    } else {
        typedef __nv_bfloat16 bf16;
        if (vec) bias_gelu_fwd_kernel<bf16, true><<<grid, kNT, 0, s>>>((const bf16*)h, (bf16*)out, spatial, channels, nsplit, bias);
        else bias_gelu_fwd_kernel<bf16, false><<<grid, kNT, 0, s>>>((const bf16*)h, (bf16*)out, spatial, channels, nsplit, bias);
    }
    ndc::launched();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return bias_fail(NDC_ERR_CUDA, "bias gelu: %s", cudaGetErrorString(e));
    return NDC_OK;
}

int ndc_bias_gelu_bwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void* ga,
                      const void* h, const float* bias, void* gh, float* gbias, void* workspace,
                      size_t workspace_bytes, void* stream) {
    if (!ga || !h || !gh) return bias_fail(NDC_ERR_INVALID, "bias gelu gradient: ga, h and gh must not be NULL");
    int st = check(batch, channels, spatial, dtype);
    if (st != NDC_OK) return st;
    if (gbias && (!workspace || workspace_bytes < ndc_bias_grad_workspace_bytes(batch, channels)))
        return bias_fail(NDC_ERR_WORKSPACE, "bias gelu gradient: workspace of %zu bytes needed",
                         ndc_bias_grad_workspace_bytes(batch, channels));
    const long long slabs = (long long)batch * channels;
    const int nsplit = choose_split(slabs, spatial);
    const bool vec = spatial % (dtype == NDC_BF16 ? 8 : 4) == 0 && ((uintptr_t)ga % 16) == 0 &&
                     ((uintptr_t)h % 16) == 0 && ((uintptr_t)gh % 16) == 0;
    const unsigned grid = (unsigned)(slabs * nsplit);
    cudaStream_t s = (cudaStream_t)stream;
    float* partial = gbias ? (float*)workspace : nullptr;
    if (dtype == NDC_F32) {
        if (vec) bias_gelu_bwd_kernel<float, true><<<grid, kNT, 0, s>>>((const float*)ga, (const float*)h, (float*)gh, spatial, channels, nsplit, bias, partial);
        else bias_gelu_bwd_kernel<float, false><<<grid, kNT, 0, s>>>((const float*)ga, (const float*)h, (float*)gh, spatial, channels, nsplit, bias, partial);
    } else {
        typedef __nv_bfloat16 bf16;
        if (vec) bias_gelu_bwd_kernel<bf16, true><<<grid, kNT, 0, s>>>((const bf16*)ga, (const bf16*)h, (bf16*)gh, spatial, channels, nsplit, bias, partial);
        else bias_gelu_bwd_kernel<bf16, false><<<grid, kNT, 0, s>>>((const bf16*)ga, (const bf16*)h, (bf16*)gh, spatial, channels, nsplit, bias, partial);
    }
    ndc::launched();
    if (gbias) {
        bias_grad_final_kernel<<<(channels + 127) / 128, 128, 0, s>>>(partial, batch, channels, nsplit, gbias);
        ndc::launched();
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return bias_fail(NDC_ERR_CUDA, "bias gelu gradient: %s", cudaGetErrorString(e));
    return NDC_OK;
}

}  // extern "C"
