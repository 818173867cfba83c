// Instance normalisation, forward and backward, for the blocks around the NDC layer.
//
//     y = (x - mean) * rstd [* weight + bias],   mean and biased variance over the spatial
//     positions of each (sample, channel) slab,  rstd = 1 / sqrt(var + eps)
//
// The work is bound by HBM traffic.  A (sample, channel) slab is cut into `nsplit` parts so that
// the grid fills the GPU even when batch x channels is small (a per-GPU batch of 2 with 64
// channels has only 128 slabs for 148 multiprocessors):
//
//   stats kernel   one CTA per (slab, part): shifted sums  sum(x - k), sum((x - k)^2)  of one part,
//                  k = the slab's first element (keeps the variance free of cancellation);
//                  16-byte loads, warp shuffles, a fixed-order combine per CTA
//   apply kernel   one CTA per (slab, part): adds the slab's partial sums in part order (every CTA of
//                  a slab repeats these few additions, so no third launch is needed), writes y
//                  and, from part 0, (mean, rstd) for backward
//   backward       the same two-step shape: partial sums of gy and gy * xhat, then
//                  gx = rstd * w * (gy - mean(gy) - xhat * mean(gy * xhat)); the partial sums
//                  also give the gradients of weight and bias (reduced per channel over the
//                  samples in a fixed order by a small third kernel)
//
// No atomics: results are bitwise reproducible.
#include <cstdarg>
#include <cstdio>

#include "ndc_b200.h"
#include "ndc_common.cuh"
#include "ndc_slab.cuh"

namespace {

thread_local char g_inorm_err[256] = "";

using namespace ndc::slab;

// ---- forward ------------------------------------------------------------------------------
// partial[(slab * nsplit + part) * 2 + {0, 1}] = sum(x - k), sum((x - k)^2) over the part
template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) inorm_stats_kernel(const T* __restrict__ x, long long sp,
                                                          int nsplit, float* __restrict__ partial) {
    __shared__ float scratch[2 * kNT / 32];
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    const T* xs = x + slab * sp;
    const float k = ndc::to_f32(xs[0]);
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    float s1 = 0.0f, s2 = 0.0f;
    if (VEC) {
        for (long long i = begin + (long long)threadIdx.x * N; i < end; i += (long long)kNT * N) {
            float v[N];
            Vec16<T>::unpack(__ldg(reinterpret_cast<const typename Vec16<T>::raw*>(xs + i)), v);
#pragma unroll
            for (int j = 0; j < N; ++j) { const float d = v[j] - k; s1 += d; s2 = fmaf(d, d, s2); }
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT) {
            const float d = ndc::to_f32(xs[i]) - k;
            s1 += d; s2 = fmaf(d, d, s2);
        }
    }
    cta_sum2(s1, s2, scratch);
    if (threadIdx.x == 0) {
        partial[(slab * nsplit + part) * 2] = s1;
        partial[(slab * nsplit + part) * 2 + 1] = s2;
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) inorm_apply_kernel(const T* __restrict__ x, long long sp, int channels,
                                                          int nsplit, const float* __restrict__ partial,
                                                          const float* __restrict__ weight,
                                                          const float* __restrict__ bias, float eps,
                                                          T* __restrict__ y, float* __restrict__ mean_rstd) {
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    const T* xs = x + slab * sp;
    T* ys = y + slab * sp;
    float s1 = 0.0f, s2 = 0.0f;
    for (int i = 0; i < nsplit; ++i) {          // same order in every CTA of the slab
        s1 += partial[(slab * nsplit + i) * 2];
        s2 += partial[(slab * nsplit + i) * 2 + 1];
    }
    const float inv_n = 1.0f / (float)sp;
    const float dm = s1 * inv_n;                                   // mean - k
    const float var = fmaxf(s2 * inv_n - dm * dm, 0.0f);
    const float mean = ndc::to_f32(xs[0]) + dm;
    const float rstd = rsqrtf(var + eps);
    if (part == 0 && threadIdx.x == 0 && mean_rstd) {
        mean_rstd[2 * slab] = mean;
        mean_rstd[2 * slab + 1] = rstd;
    }
    const int c = (int)(slab % channels);
    const float w = weight ? weight[c] : 1.0f, b = bias ? bias[c] : 0.0f;
    const float scale = rstd * w;
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    if (VEC) {
        for (long long i = begin + (long long)threadIdx.x * N; i < end; i += (long long)kNT * N) {
            float v[N];
            Vec16<T>::unpack(__ldg(reinterpret_cast<const typename Vec16<T>::raw*>(xs + i)), v);
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] = fmaf(v[j] - mean, scale, b);
            *reinterpret_cast<typename Vec16<T>::raw*>(ys + i) = Vec16<T>::pack(v);
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT)
            ys[i] = ndc::from_f32<T>(fmaf(ndc::to_f32(xs[i]) - mean, scale, b));
    }
}

// ---- backward -----------------------------------------------------------------------------
// partial[(slab * nsplit + part) * 2 + {0, 1}] = sum(gy), sum(gy * xhat) over the part
template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) inorm_bwd_stats_kernel(const T* __restrict__ x, const T* __restrict__ gy,
                                                              long long sp, int nsplit,
                                                              const float* __restrict__ mean_rstd,
                                                              float* __restrict__ partial) {
    __shared__ float scratch[2 * kNT / 32];
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    const T* xs = x + slab * sp;
    const T* gs = gy + slab * sp;
    const float mean = mean_rstd[2 * slab], rstd = mean_rstd[2 * slab + 1];
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    float s1 = 0.0f, s2 = 0.0f;
    if (VEC) {
        for (long long i = begin + (long long)threadIdx.x * N; i < end; i += (long long)kNT * N) {
            float xv[N], gv[N];
            Vec16<T>::unpack(__ldg(reinterpret_cast<const typename Vec16<T>::raw*>(xs + i)), xv);
            Vec16<T>::unpack(__ldg(reinterpret_cast<const typename Vec16<T>::raw*>(gs + i)), gv);
#pragma unroll
            for (int j = 0; j < N; ++j) { s1 += gv[j]; s2 = fmaf(gv[j], (xv[j] - mean) * rstd, s2); }
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT) {
            const float g = ndc::to_f32(gs[i]);
            s1 += g; s2 = fmaf(g, (ndc::to_f32(xs[i]) - mean) * rstd, s2);
        }
    }
    cta_sum2(s1, s2, scratch);
    if (threadIdx.x == 0) {
        partial[(slab * nsplit + part) * 2] = s1;
        partial[(slab * nsplit + part) * 2 + 1] = s2;
    }
}

template <typename T, bool VEC>
__global__ void __launch_bounds__(kNT) inorm_bwd_apply_kernel(const T* __restrict__ x, const T* __restrict__ gy,
                                                              long long sp, int channels, int nsplit,
                                                              const float* __restrict__ mean_rstd,
                                                              const float* __restrict__ partial,
                                                              const float* __restrict__ weight,
                                                              T* __restrict__ gx) {
    const long long slab = blockIdx.x / nsplit;
    const int part = blockIdx.x % nsplit;
    const T* xs = x + slab * sp;
    const T* gs = gy + slab * sp;
    T* os = gx + slab * sp;
    float s1 = 0.0f, s2 = 0.0f;
    for (int i = 0; i < nsplit; ++i) {
        s1 += partial[(slab * nsplit + i) * 2];
        s2 += partial[(slab * nsplit + i) * 2 + 1];
    }
    const float mean = mean_rstd[2 * slab], rstd = mean_rstd[2 * slab + 1];
    const float inv_n = 1.0f / (float)sp;
    const float w = weight ? weight[slab % channels] : 1.0f;
    // gx = rstd * w * (gy - mean(gy) - xhat * mean(gy * xhat))
    const float a = rstd * w, m1 = s1 * inv_n, m2 = s2 * inv_n;
    long long begin, end;
    part_range(sp, nsplit, part, Vec16<T>::N, begin, end);
    constexpr int N = Vec16<T>::N;
    if (VEC) {
        for (long long i = begin + (long long)threadIdx.x * N; i < end; i += (long long)kNT * N) {
            float xv[N], gv[N];
            Vec16<T>::unpack(__ldg(reinterpret_cast<const typename Vec16<T>::raw*>(xs + i)), xv);
            Vec16<T>::unpack(__ldg(reinterpret_cast<const typename Vec16<T>::raw*>(gs + i)), gv);
#pragma unroll
            for (int j = 0; j < N; ++j) gv[j] = a * (gv[j] - m1 - (xv[j] - mean) * rstd * m2);
            *reinterpret_cast<typename Vec16<T>::raw*>(os + i) = Vec16<T>::pack(gv);
        }
    } else {
        for (long long i = begin + threadIdx.x; i < end; i += kNT)
            os[i] = ndc::from_f32<T>(a * (ndc::to_f32(gs[i]) - m1 - (ndc::to_f32(xs[i]) - mean) * rstd * m2));
    }
}

// gweight[c] = sum over samples and parts of sum(gy * xhat), gbias[c] = ... of sum(gy); fixed order
__global__ void inorm_param_grad_kernel(const float* __restrict__ partial, int batch, int channels,
                                        int nsplit, float* __restrict__ gweight, float* __restrict__ gbias) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= channels) return;
    float s1 = 0.0f, s2 = 0.0f;
    for (int b = 0; b < batch; ++b)
        for (int i = 0; i < nsplit; ++i) {
            const long long k = (((long long)b * channels + c) * nsplit + i) * 2;
            s1 += partial[k]; s2 += partial[k + 1];
        }
    if (gbias) gbias[c] = s1;
    if (gweight) gweight[c] = s2;
}

int inorm_fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_inorm_err, sizeof(g_inorm_err), fmt, ap);
    va_end(ap);
    return status;
}

struct Problem {
    long long slabs, sp;
    int channels, nsplit;
    bool vec;
};

int make_problem(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void* a,
                 const void* b, const void* c, Problem& p) {
    if (batch <= 0 || channels <= 0 || spatial <= 0)
        return inorm_fail(NDC_ERR_INVALID, "instance norm: batch, channels and spatial size must be positive");
    if (dtype != NDC_F32 && dtype != NDC_BF16)
        return inorm_fail(NDC_ERR_INVALID, "instance norm: dtype must be NDC_F32 or NDC_BF16");
    p.slabs = (long long)batch * channels;
    if (p.slabs * kMaxSplit > 0x7fffffffLL)
        return inorm_fail(NDC_ERR_UNSUPPORTED, "instance norm: batch * channels is too large");
    p.sp = spatial;
    p.channels = channels;
    p.nsplit = choose_split(p.slabs, spatial);
    const int n = dtype == NDC_BF16 ? 8 : 4;
    auto ok = [](const void* q) { return q == nullptr || ((uintptr_t)q % 16) == 0; };
    p.vec = spatial % n == 0 && ok(a) && ok(b) && ok(c);
    return NDC_OK;
}

}  // namespace

extern "C" {

const char* ndc_inorm_last_error(void) { return g_inorm_err; }

size_t ndc_inorm_workspace_bytes(int32_t batch, int32_t channels) {
    if (batch <= 0 || channels <= 0) return 0;
    return (size_t)batch * channels * kMaxSplit * 2 * sizeof(float);
}

int ndc_inorm_fwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void* x,
                  const float* weight, const float* bias, float eps, void* y, float* mean_rstd,
                  void* workspace, size_t workspace_bytes, void* stream) {
    if (!x || !y) return inorm_fail(NDC_ERR_INVALID, "instance norm: x and y must not be NULL");
    Problem p;
    int st = make_problem(batch, channels, spatial, dtype, x, y, nullptr, p);
    if (st != NDC_OK) return st;
    if (!workspace || workspace_bytes < ndc_inorm_workspace_bytes(batch, channels))
        return inorm_fail(NDC_ERR_WORKSPACE, "instance norm: workspace of %zu bytes needed",
                          ndc_inorm_workspace_bytes(batch, channels));
    cudaStream_t s = (cudaStream_t)stream;
    float* partial = (float*)workspace;
    const unsigned grid = (unsigned)(p.slabs * p.nsplit);
#define NDC_INORM_FWD(T, V)                                                                       \
    do {                                                                                          \
        inorm_stats_kernel<T, V><<<grid, kNT, 0, s>>>((const T*)x, p.sp, p.nsplit, partial);      \
        inorm_apply_kernel<T, V><<<grid, kNT, 0, s>>>((const T*)x, p.sp, p.channels, p.nsplit,    \
                                                      partial, weight, bias, eps, (T*)y, mean_rstd); \
    } while (0)
    if (dtype == NDC_F32) { if (p.vec) NDC_INORM_FWD(float, true); else NDC_INORM_FWD(float, false); }
    else { if (p.vec) NDC_INORM_FWD(__nv_bfloat16, true); else NDC_INORM_FWD(__nv_bfloat16, false); }
#undef NDC_INORM_FWD
    ndc::launched(2);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return inorm_fail(NDC_ERR_CUDA, "instance norm forward: %s", cudaGetErrorString(e));
    return NDC_OK;
}

int ndc_inorm_bwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void* x,
                  const void* gy, const float* weight, const float* mean_rstd, void* gx,
                  float* gweight, float* gbias, void* workspace, size_t workspace_bytes, void* stream) {
    if (!x || !gy || !gx || !mean_rstd)
        return inorm_fail(NDC_ERR_INVALID, "instance norm: x, gy, gx and mean_rstd must not be NULL");
    Problem p;
    int st = make_problem(batch, channels, spatial, dtype, x, gy, gx, p);
    if (st != NDC_OK) return st;
    if (!workspace || workspace_bytes < ndc_inorm_workspace_bytes(batch, channels))
        return inorm_fail(NDC_ERR_WORKSPACE, "instance norm: workspace of %zu bytes needed",
                          ndc_inorm_workspace_bytes(batch, channels));
    cudaStream_t s = (cudaStream_t)stream;
    float* partial = (float*)workspace;
    const unsigned grid = (unsigned)(p.slabs * p.nsplit);
#define NDC_INORM_BWD(T, V)                                                                       \
    do {                                                                                          \
        inorm_bwd_stats_kernel<T, V><<<grid, kNT, 0, s>>>((const T*)x, (const T*)gy, p.sp, p.nsplit, \
                                                          mean_rstd, partial);                    \
        inorm_bwd_apply_kernel<T, V><<<grid, kNT, 0, s>>>((const T*)x, (const T*)gy, p.sp, p.channels, \
                                                          p.nsplit, mean_rstd, partial, weight, (T*)gx); \
    } while (0)
    if (dtype == NDC_F32) { if (p.vec) NDC_INORM_BWD(float, true); else NDC_INORM_BWD(float, false); }
    else { if (p.vec) NDC_INORM_BWD(__nv_bfloat16, true); else NDC_INORM_BWD(__nv_bfloat16, false); }
#undef NDC_INORM_BWD
    ndc::launched(2);
    if (gweight || gbias) {
        inorm_param_grad_kernel<<<(channels + 127) / 128, 128, 0, s>>>(partial, batch, channels, p.nsplit,
                                                                      gweight, gbias);
        ndc::launched();
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return inorm_fail(NDC_ERR_CUDA, "instance norm backward: %s", cudaGetErrorString(e));
    return NDC_OK;
}

}  // extern "C"
