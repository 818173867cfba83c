// Generic NDC kernels: any m, sc, odd kernel, 1-D/2-D/3-D, float32 or bfloat16 storage.
//
// One thread per output element, taps looped at run time, operands read through L1/L2.
// These cover every filter geometry; the depthwise ratio-4 geometries of the published
// configurations run on the tiled kernels in ndc_dw4_*.cuh instead.
#pragma once

#include "ndc_common.cuh"

namespace ndc {
namespace generic {

constexpr int kThreads = 256;

__device__ __forceinline__ void decode(long long idx, long long SP, int C, const Geo& g,
                                       long long& bg, int& c, int& d, int& y, int& x) {
    long long p = idx % SP;
    long long r = idx / SP;
    c = (int)(r % C);
    bg = r / C;
    x = (int)(p % g.W);
    long long q = p / g.W;
    y = (int)(q % g.H);
    d = (int)(q / g.H);
}

// out[bg, co, p] = K or A applied to `in`, optionally with bias/ReLU folded into the read.
template <typename TI, typename TO, bool ADJ>
__global__ void __launch_bounds__(kThreads)
gconv_kernel(Geo g, const TI* __restrict__ in, const float* __restrict__ h,
             const float* __restrict__ bias, int relu_in, TO* __restrict__ out) {
    const int cin = ADJ ? g.m : g.sc, cout = ADJ ? g.sc : g.m;
    const long long total = (long long)g.B * g.G * cout * g.SP;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long bg; int co, d, y, x;
        decode(idx, g.SP, cout, g, bg, co, d, y, x);
        const int gi = (int)(bg % g.G);
        const TI* inb = in + bg * cin * g.SP;
        const float* hg = h + (long long)gi * g.m * g.sc * g.KT;
        float acc = 0.0f;
        for (int a = 0; a < g.kD; ++a) {
            const int dd = ADJ ? d + g.pD - a : d + a - g.pD;
            if (dd < 0 || dd >= g.D) continue;
            for (int b = 0; b < g.kH; ++b) {
                const int yy = ADJ ? y + g.pH - b : y + b - g.pH;
                if (yy < 0 || yy >= g.H) continue;
                for (int c = 0; c < g.kW; ++c) {
                    const int xx = ADJ ? x + g.pW - c : x + c - g.pW;
                    if (xx < 0 || xx >= g.W) continue;
                    const int tau = (a * g.kH + b) * g.kW + c;
                    const long long q = ((long long)dd * g.H + yy) * g.W + xx;
                    for (int ci = 0; ci < cin; ++ci) {
                        float v = to_f32(inb[ci * g.SP + q]);
                        if (bias) v += bias[gi * cin + ci];
                        if (relu_in) v = fmaxf(v, 0.0f);
                        const float w = ADJ ? hg[((long long)ci * g.sc + co) * g.KT + tau]
                                            : hg[((long long)co * g.sc + ci) * g.KT + tau];
                        acc = fmaf(v, w, acc);
                    }
                }
            }
        }
        out[idx] = from_f32<TO>(acc);
    }
}

// n = A(x)[i,p], d = A(t1)[i,p] for one source element.
template <typename T>
__device__ __forceinline__ void adjoint_pair(const Geo& g, const T* __restrict__ xb,
                                             const T* __restrict__ tb, const float* __restrict__ hg,
                                             int i, int d, int y, int x, float& n, float& dn) {
    n = 0.0f; dn = 0.0f;
    for (int a = 0; a < g.kD; ++a) {
        const int dd = d + g.pD - a;
        if (dd < 0 || dd >= g.D) continue;
        for (int b = 0; b < g.kH; ++b) {
            const int yy = y + g.pH - b;
            if (yy < 0 || yy >= g.H) continue;
            for (int c = 0; c < g.kW; ++c) {
                const int xx = x + g.pW - c;
                if (xx < 0 || xx >= g.W) continue;
                const int tau = (a * g.kH + b) * g.kW + c;
                const long long q = ((long long)dd * g.H + yy) * g.W + xx;
                for (int o = 0; o < g.m; ++o) {
                    const float w = hg[((long long)o * g.sc + i) * g.KT + tau];
                    n = fmaf(to_f32(xb[o * g.SP + q]), w, n);
                    dn = fmaf(to_f32(tb[o * g.SP + q]), w, dn);
                }
            }
        }
    }
}

template <typename T>
__device__ __forceinline__ float source_value(const Geo& g, const T* z, long long e,
                                              const float* bias, int ch, float& pre) {
    float v = to_f32(z[e]);
    if (bias) v += bias[ch];
    pre = v;
    return g.relu ? fmaxf(v, 0.0f) : v;
}

// out = (s * (A(x) + eps)) / (A(t1) + eps)
template <typename T>
__global__ void __launch_bounds__(kThreads)
fwd_out_kernel(Geo g, const T* __restrict__ x, const T* __restrict__ t1, const T* __restrict__ z,
               const float* __restrict__ h, const float* __restrict__ bias, T* __restrict__ out) {
    const long long total = (long long)g.B * g.G * g.sc * g.SP;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long bg; int i, d, y, xx;
        decode(idx, g.SP, g.sc, g, bg, i, d, y, xx);
        const int gi = (int)(bg % g.G);
        float n, dn, pre;
        adjoint_pair(g, x + bg * g.m * g.SP, t1 + bg * g.m * g.SP,
                     h + (long long)gi * g.m * g.sc * g.KT, i, d, y, xx, n, dn);
        const float s = source_value(g, z, idx, bias, gi * g.sc + i, pre);
        out[idx] = from_f32<T>(__fdiv_rn(s * (n + g.eps), dn + g.eps));
    }
}

// gnum = g*s/d, gden = -(gnum*n)/d into float32 scratch; the direct term (g*n)/d into gz.
template <typename T>
__global__ void __launch_bounds__(kThreads)
bwd_ratio_kernel(Geo g, const T* __restrict__ x, const T* __restrict__ t1, const T* __restrict__ z,
                 const T* __restrict__ gout, const float* __restrict__ h,
                 const float* __restrict__ bias, float* __restrict__ gnum, float* __restrict__ gden,
                 T* __restrict__ gz_direct) {
    const long long total = (long long)g.B * g.G * g.sc * g.SP;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long bg; int i, d, y, xx;
        decode(idx, g.SP, g.sc, g, bg, i, d, y, xx);
        const int gi = (int)(bg % g.G);
        float n, dn, pre;
        adjoint_pair(g, x + bg * g.m * g.SP, t1 + bg * g.m * g.SP,
                     h + (long long)gi * g.m * g.sc * g.KT, i, d, y, xx, n, dn);
        n += g.eps; dn += g.eps;
        const float s = source_value(g, z, idx, bias, gi * g.sc + i, pre);
        const float gv = to_f32(gout[idx]);
        const float gn = __fdiv_rn(gv * s, dn);
        gnum[idx] = gn;
        gden[idx] = -__fdiv_rn(gn * n, dn);
        if (gz_direct) gz_direct[idx] = from_f32<T>(__fdiv_rn(gv * n, dn));
    }
}

// gz = [z + b > 0] * (direct + A(gt1)), in place over the direct term.
template <typename T>
__global__ void __launch_bounds__(kThreads)
gz_kernel(Geo g, const float* __restrict__ gt1, const T* __restrict__ z,
          const float* __restrict__ h, const float* __restrict__ bias, T* __restrict__ gz) {
    const long long total = (long long)g.B * g.G * g.sc * g.SP;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        long long bg; int i, d, y, xx;
        decode(idx, g.SP, g.sc, g, bg, i, d, y, xx);
        const int gi = (int)(bg % g.G);
        const float* gb = gt1 + bg * g.m * g.SP;
        const float* hg = h + (long long)gi * g.m * g.sc * g.KT;
        float acc = 0.0f;
        for (int a = 0; a < g.kD; ++a) {
            const int dd = d + g.pD - a;
            if (dd < 0 || dd >= g.D) continue;
            for (int b = 0; b < g.kH; ++b) {
                const int yy = y + g.pH - b;
                if (yy < 0 || yy >= g.H) continue;
                for (int c = 0; c < g.kW; ++c) {
                    const int x2 = xx + g.pW - c;
                    if (x2 < 0 || x2 >= g.W) continue;
                    const int tau = (a * g.kH + b) * g.kW + c;
                    const long long q = ((long long)dd * g.H + yy) * g.W + x2;
                    for (int o = 0; o < g.m; ++o)
                        acc = fmaf(gb[o * g.SP + q], hg[((long long)o * g.sc + i) * g.KT + tau], acc);
                }
            }
        }
        float r = to_f32(gz[idx]) + acc;
        if (g.relu) {
            float pre;
            (void)source_value(g, z, idx, bias, gi * g.sc + i, pre);
            if (!(pre > 0.0f)) r = 0.0f;
        }
        gz[idx] = from_f32<T>(r);
    }
}

// gh[g,o,i,tau] = sum_{b,p} gden[i,p] t1[o,q] + gnum[i,p] x[o,q] + s[i,p] gt1[o,q],
// q = p + pad - tau.  One block per filter element; fixed strided partition over (b,p),
// fixed reduction tree.
template <typename T>
__global__ void __launch_bounds__(kThreads)
wgrad_kernel(Geo g, const T* __restrict__ x, const T* __restrict__ t1, const T* __restrict__ z,
             const float* __restrict__ bias, const float* __restrict__ gnum,
             const float* __restrict__ gden, const float* __restrict__ gt1,
             float* __restrict__ gh) {
    __shared__ float scratch[kThreads / 32];
    long long e = blockIdx.x;  // ((gi*m + o)*sc + i)*KT + tau
    const int tau = (int)(e % g.KT); e /= g.KT;
    const int i = (int)(e % g.sc); e /= g.sc;
    const int o = (int)(e % g.m);
    const int gi = (int)(e / g.m);
    const int c = tau % g.kW, b = (tau / g.kW) % g.kH, a = tau / (g.kW * g.kH);
    const int sd = g.pD - a, sh = g.pH - b, sw = g.pW - c;
    float acc = 0.0f;
    for (int bi = 0; bi < g.B; ++bi) {
        const long long bg = (long long)bi * g.G + gi;
        const long long sb = (bg * g.sc + i) * g.SP, ob = (bg * g.m + o) * g.SP;
        for (long long p = threadIdx.x; p < g.SP; p += blockDim.x) {
            const int xw = (int)(p % g.W);
            const long long r = p / g.W;
            const int y = (int)(r % g.H), d = (int)(r / g.H);
            const int d2 = d + sd, y2 = y + sh, x2 = xw + sw;
            if (d2 < 0 || d2 >= g.D || y2 < 0 || y2 >= g.H || x2 < 0 || x2 >= g.W) continue;
            const long long q = ((long long)d2 * g.H + y2) * g.W + x2;
            float pre;
            const float s = source_value(g, z, sb + p, bias, gi * g.sc + i, pre);
            acc = fmaf(gden[sb + p], to_f32(t1[ob + q]), acc);
            acc = fmaf(gnum[sb + p], to_f32(x[ob + q]), acc);
            acc = fmaf(s, gt1[ob + q], acc);
        }
    }
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) gh[blockIdx.x] = acc;
}

// gb[c] = sum_{b,p} gz[b,c,p]; one block per channel, fixed order.
template <typename T>
__global__ void __launch_bounds__(kThreads)
gb_kernel(Geo g, const T* __restrict__ gz, float* __restrict__ gb) {
    __shared__ float scratch[kThreads / 32];
    const int ch = blockIdx.x, C = g.G * g.sc;
    float acc = 0.0f;
    for (int bi = 0; bi < g.B; ++bi) {
        const T* base = gz + ((long long)bi * C + ch) * g.SP;
        for (long long p = threadIdx.x; p < g.SP; p += blockDim.x) acc += to_f32(base[p]);
    }
    acc = block_sum(acc, scratch);
    if (threadIdx.x == 0) gb[ch] = acc;
}

inline int grid_for(long long total) {
    long long blocks = (total + kThreads - 1) / kThreads;
    const long long cap = 148LL * 64;  // grid-stride beyond 64 blocks per SM
    return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// Scratch layout of the generic backward: gnum | gden | gt1, each float32, 256-B aligned.
struct BwdScratch {
    size_t off_gnum, off_gden, off_gt1, bytes;
};
inline BwdScratch bwd_scratch(const Geo& g) {
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    BwdScratch s;
    const size_t src = (size_t)g.B * g.G * g.sc * g.SP * sizeof(float);
    const size_t flt = (size_t)g.B * g.G * g.m * g.SP * sizeof(float);
    s.off_gnum = 0;
    s.off_gden = up(src);
    s.off_gt1 = s.off_gden + up(src);
    s.bytes = s.off_gt1 + up(flt);
    return s;
}

template <typename T>
cudaError_t forward(const Geo& g, const T* x, const T* z, const float* h, const float* bias,
                    T* out, T* t1, cudaStream_t st) {
    const long long n_flt = (long long)g.B * g.G * g.m * g.SP;
    const long long n_src = (long long)g.B * g.G * g.sc * g.SP;
    gconv_kernel<T, T, false><<<grid_for(n_flt), kThreads, 0, st>>>(g, z, h, bias, g.relu, t1);
    fwd_out_kernel<T><<<grid_for(n_src), kThreads, 0, st>>>(g, x, t1, z, h, bias, out);
    launched(2);
    return cudaGetLastError();
}

template <typename T>
cudaError_t backward(const Geo& g, const T* x, const T* z, const T* t1, const float* h,
                     const float* bias, const T* gout, T* gx, T* gz, float* gh, float* gb,
                     void* ws, cudaStream_t st) {
    const BwdScratch sc = bwd_scratch(g);
    float* gnum = (float*)((char*)ws + sc.off_gnum);
    float* gden = (float*)((char*)ws + sc.off_gden);
    float* gt1 = (float*)((char*)ws + sc.off_gt1);
    const long long n_flt = (long long)g.B * g.G * g.m * g.SP;
    const long long n_src = (long long)g.B * g.G * g.sc * g.SP;
    bwd_ratio_kernel<T><<<grid_for(n_src), kThreads, 0, st>>>(g, x, t1, z, gout, h, bias, gnum,
                                                             gden, gz);
    launched();
    if (gz || gh) {
        gconv_kernel<float, float, false><<<grid_for(n_flt), kThreads, 0, st>>>(g, gden, h, nullptr,
                                                                               0, gt1);
        launched();
    }
    if (gx) {
        gconv_kernel<float, T, false><<<grid_for(n_flt), kThreads, 0, st>>>(g, gnum, h, nullptr, 0,
                                                                           gx);
        launched();
    }
    if (gh) {
        wgrad_kernel<T><<<g.G * g.m * g.sc * g.KT, kThreads, 0, st>>>(g, x, t1, z, bias, gnum,
                                                                     gden, gt1, gh);
        launched();
    }
    if (gz) {
        gz_kernel<T><<<grid_for(n_src), kThreads, 0, st>>>(g, gt1, z, h, bias, gz);
        launched();
        if (gb) {
            gb_kernel<T><<<g.G * g.sc, kThreads, 0, st>>>(g, gz, gb);
            launched();
        }
    }
    return cudaGetLastError();
}

template <typename T>
cudaError_t gconv(const Geo& g, const T* in, const float* h, const float* bias, bool adjoint,
                  T* out, cudaStream_t st) {
    if (adjoint) {
        const long long n = (long long)g.B * g.G * g.sc * g.SP;
        gconv_kernel<T, T, true><<<grid_for(n), kThreads, 0, st>>>(g, in, h, nullptr, 0, out);
    } else {
        const long long n = (long long)g.B * g.G * g.m * g.SP;
        gconv_kernel<T, T, false><<<grid_for(n), kThreads, 0, st>>>(g, in, h, bias, g.relu, out);
    }
    launched();
    return cudaGetLastError();
}

}  // namespace generic
}  // namespace ndc
