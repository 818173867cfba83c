// Host side of the tiled depthwise kernels: tiling decisions and launches.
#pragma once

#include <algorithm>

#include "ndc_dw4_fwd.cuh"
#include "ndc_dw4_bwd.cuh"

namespace ndc {
namespace dw4 {

constexpr int kNumSMs = 148;
constexpr size_t kSmemTwoPerSM = 112 * 1024;   // lets two CTAs share an SM
constexpr size_t kSmemMax = 227 * 1024;

// Launch shape per kernel geometry.
template <int KD, int KH, int KW> struct FwdShape;
template <> struct FwdShape<3, 3, 3> { static constexpr int NT = 256, MAXZ = 5, MAXX = 1, MINB = 2; };
template <> struct FwdShape<1, 5, 5> { static constexpr int NT = 256, MAXZ = 1, MAXX = 1, MINB = 2; };
template <> struct FwdShape<1, 3, 3> { static constexpr int NT = 256, MAXZ = 1, MAXX = 1, MINB = 2; };

inline bool shape_supported(int kD, int kH, int kW) {
    return (kD == 3 && kH == 3 && kW == 3) || (kD == 1 && kH == 5 && kW == 5) ||
           (kD == 1 && kH == 3 && kW == 3);
}

// Chunks along depth: enough CTAs for about `waves` rounds of two CTAs per SM, but chunks of
// at least 16 planes (every chunk recomputes 2*PD planes of its neighbours).
inline void plan_depth(int KD, int D, long long ctas_per_chunk, int waves, Tiling& t) {
    if (KD == 1) {
        t.DC = 1;
    } else {
        const long long target = (long long)waves * 2 * kNumSMs;
        long long ndc = target / std::max(1LL, ctas_per_chunk);
        ndc = std::max(1LL, std::min(ndc, (long long)std::max(1, D / 16)));
        t.DC = (int)((D + ndc - 1) / ndc);
    }
    t.ndc = (D + t.DC - 1) / t.DC;
}

template <int KD, int KH, int KW>
inline bool plan_fwd(int D, int H, int W, long long BC, Tiling& t, size_t& smem_bytes) {
    using S = FwdShape<KD, KH, KW>;
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29)) return false;  // 32-bit offsets inside a slab
    if (W > 256) return false;
    t.NQ = (W + 3) / 4;
    t.pitch = row_pitch(W);
    const int NS8 = (t.NQ + 1) / 2;
    int TH = H;
    if (KD > 1) {
        TH = std::min(TH, (S::NT / 2) / NS8 - 2 * PH);                   // one K strip per thread pair
        TH = std::min(TH, S::NT * S::MAXZ / (SCH * t.NQ) - 4 * PH);      // z prefetch registers
        TH = std::min(TH, S::NT * S::MAXX / t.NQ - 2 * PH);              // x prefetch registers
    }
    auto bytes = [&](int th) {
        Tiling q = t; q.TH = th;
        return (size_t)FwdSmem<KD, KH, KW>(q).total_floats * sizeof(float);
    };
    while (TH > 1 && (bytes(TH) > kSmemTwoPerSM || SCH * (TH + 4 * PH) * t.pitch > 65535)) --TH;
    if (TH < 1 || bytes(TH) > kSmemMax || SCH * (TH + 4 * PH) * t.pitch > 65535) return false;
    t.nth = (H + TH - 1) / TH;
    t.TH = (H + t.nth - 1) / t.nth;
    plan_depth(KD, D, BC * t.nth, 5, t);
    smem_bytes = bytes(t.TH);
    return true;
}

inline bool aligned_for_vec(const void* p, int dtype) {
    return ((uintptr_t)p % (dtype == NDC_BF16 ? 8 : 16)) == 0;
}

template <typename T, int KD, int KH, int KW, bool VEC, int WQ>
cudaError_t launch_fwd(const FwdParams& P, size_t smem_bytes, long long BC, cudaStream_t st) {
    using S = FwdShape<KD, KH, KW>;
    auto kern = fwd_kernel<T, KD, KH, KW, S::NT, S::MAXZ, S::MAXX, S::MINB, VEC, WQ>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem_bytes);
    if (e != cudaSuccess) return e;
    const long long grid = BC * P.t.ndc * P.t.nth;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    kern<<<(unsigned)grid, S::NT, smem_bytes, st>>>(P);
    launched();
    return cudaGetLastError();
}

template <typename T, int KD, int KH, int KW>
cudaError_t forward_shape(const Geo& g, const T* x, const T* z, const float* h, const float* bias,
                          T* out, T* t1, int dtype, cudaStream_t st, bool& handled) {
    FwdParams P;
    size_t smem = 0;
    const long long BC = (long long)g.B * g.G;
    handled = plan_fwd<KD, KH, KW>(g.D, g.H, g.W, BC, P.t, smem);
    if (!handled) return cudaSuccess;
    P.x = x; P.z = z; P.h = h; P.bias = bias; P.out = out; P.t1 = t1;
    P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W;
    P.eps = g.eps; P.relu = g.relu;
    const bool vec = g.W % 4 == 0 && aligned_for_vec(x, dtype) && aligned_for_vec(z, dtype) &&
                     aligned_for_vec(out, dtype) && aligned_for_vec(t1, dtype);
    // widths that occur in the published configurations get kernels with a compile-time width
    if constexpr (KD > 1) {
        if (vec && g.W == 64) return launch_fwd<T, KD, KH, KW, true, 16>(P, smem, BC, st);
        if (vec && g.W == 128) return launch_fwd<T, KD, KH, KW, true, 32>(P, smem, BC, st);
    }
    return vec ? launch_fwd<T, KD, KH, KW, true, 0>(P, smem, BC, st)
               : launch_fwd<T, KD, KH, KW, false, 0>(P, smem, BC, st);
}

// ---------------------------------------------------------------------------- backward

constexpr int kRatioNT = 128;   // ratio_kernel threads
constexpr int kRatioMAXX = 2;   // its prefetch registers (quads) per tensor
constexpr int kRingNT = 128;    // gz_kernel threads
constexpr int kRingMAXX = 4;
constexpr int kKconvNT = 192;   // 48 strip slots x 4 channel lanes

// Band height for the kernels that only hold single-channel rings (ratio: 2 tensors, gz: 1).
template <int KD, int KH, int KW>
inline bool plan_ring(int D, int H, int W, long long BC, int ntensors, int nt, int maxx,
                      int red_threads, size_t extra_bytes, size_t smem_target, Tiling& t,
                      size_t& smem_bytes) {
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29) || W > 256) return false;
    t.NQ = (W + 3) / 4;
    t.pitch = row_pitch(W);
    int TH = H;
    if (KD > 1) TH = std::min(TH, nt * maxx / t.NQ - 2 * PH);
    auto bytes = [&](int th) {
        Tiling q = t; q.TH = th;
        return (size_t)RingSmem<KD, KH, KW>(q, ntensors, red_threads).total_floats * sizeof(float) +
               extra_bytes;
    };
    while (TH > 1 && (bytes(TH) > smem_target || (TH + 2 * PH) * t.pitch > 65535)) --TH;
    if (TH < 1 || bytes(TH) > kSmemMax) return false;
    t.nth = (H + TH - 1) / TH;
    t.TH = (H + t.nth - 1) / t.nth;
    plan_depth(KD, D, BC * t.nth, 6, t);
    smem_bytes = bytes(t.TH);
    return true;
}

template <int KD, int KH, int KW>
inline bool plan_kconv(int D, int H, int W, long long BC, Tiling& t, size_t& smem_bytes) {
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29) || W > 256) return false;
    t.NQ = (W + 3) / 4;
    t.pitch = row_pitch(W);
    const int NS8 = (t.NQ + 1) / 2;
    int TH = H;
    if (KD > 1) {
        TH = std::min(TH, (kKconvNT / SCH) / NS8);
    }
    auto bytes = [&](int th) {
        Tiling q = t; q.TH = th;
        return (size_t)KconvSmem<KD, KH, KW>(q, kKconvNT).total_floats * sizeof(float);
    };
    while (TH > 1 && (bytes(TH) > 72 * 1024 || SCH * (TH + 2 * PH) * t.pitch > 65535)) --TH;
    if (TH < 1 || bytes(TH) > kSmemMax) return false;
    t.nth = (H + TH - 1) / TH;
    t.TH = (H + t.nth - 1) / t.nth;
    plan_depth(KD, D, 2 * BC * t.nth, 6, t);
    smem_bytes = bytes(t.TH);
    return true;
}

struct BwdPlan {
    Tiling ratio, kconv, gz;
    size_t smem_ratio, smem_kconv, smem_gz;
    size_t off_gnum, off_gden, off_gt1, off_gxtmp, off_pa, off_pa2, off_pb, bytes;
    long long n_ratio, n_kconv, n_gz;   // CTAs (kconv: per tensor; = partial records)
};

template <int KD, int KH, int KW>
inline bool plan_bwd(const Geo& g, BwdPlan& p) {
    const long long BC = (long long)g.B * g.G;
    if (!plan_ring<KD, KH, KW>(g.D, g.H, g.W, BC, 2, kRatioNT, kRatioMAXX, 0, 0, 56 * 1024, p.ratio, p.smem_ratio))
        return false;
    if (!plan_kconv<KD, KH, KW>(g.D, g.H, g.W, BC, p.kconv, p.smem_kconv)) return false;
    // gz_kernel also stages two sets of 8 strips per thread (z and the direct term)
    if (!plan_ring<KD, KH, KW>(g.D, g.H, g.W, BC, 1, kRingNT, kRingMAXX, kRingNT,
                               (size_t)2 * 2 * SCH * kRingNT * 16, kSmemTwoPerSM, p.gz, p.smem_gz))
        return false;
    auto up = [](size_t v) { return (v + 255) & ~(size_t)255; };
    const size_t src = (size_t)BC * SCH * g.SP * sizeof(float);
    const size_t flt = (size_t)BC * g.SP * sizeof(float);
    p.n_ratio = BC * p.ratio.ndc * p.ratio.nth;
    p.n_kconv = BC * p.kconv.ndc * p.kconv.nth;
    p.n_gz = BC * p.gz.ndc * p.gz.nth;
    const size_t rec = (size_t)kPartialStride * sizeof(float);
    p.off_gnum = 0;
    p.off_gden = up(src);
    p.off_gt1 = p.off_gden + up(src);
    p.off_gxtmp = p.off_gt1 + up(flt);      // K(gnum) when the caller does not want gx
    p.off_pa = p.off_gxtmp + up(flt);
    p.off_pa2 = p.off_pa + up((size_t)p.n_kconv * rec);
    p.off_pb = p.off_pa2 + up((size_t)p.n_kconv * rec);
    p.bytes = p.off_pb + up((size_t)p.n_gz * rec);
    return true;
}

inline bool plan_bwd_any(const Geo& g, BwdPlan& p) {
    if (g.m != 1 || g.sc != SCH) return false;
    if (g.kD == 3 && g.kH == 3 && g.kW == 3) return plan_bwd<3, 3, 3>(g, p);
    if (g.kD == 1 && g.kH == 5 && g.kW == 5) return plan_bwd<1, 5, 5>(g, p);
    if (g.kD == 1 && g.kH == 3 && g.kW == 3) return plan_bwd<1, 3, 3>(g, p);
    return false;
}

template <typename K>
inline cudaError_t set_smem(K kern, size_t bytes) {
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

#define NDC_CUDA_TRY(expr)                      \
    do {                                        \
        cudaError_t _e = (expr);                \
        if (_e != cudaSuccess) return _e;       \
    } while (0)

template <typename T, int KD, int KH, int KW, bool VEC, int WQ>
cudaError_t backward_launch(const Geo& g, const BwdPlan& p, const T* x, const T* z, const T* t1,
                            const float* h, const float* bias, const T* gout, T* gx, T* gz,
                            float* gh, float* gb, void* ws, cudaStream_t st) {
    float* gnum = (float*)((char*)ws + p.off_gnum);
    float* gden = (float*)((char*)ws + p.off_gden);
    float* gt1 = (float*)((char*)ws + p.off_gt1);
    float* pa = (float*)((char*)ws + p.off_pa);
    float* pa2 = (float*)((char*)ws + p.off_pa2);
    float* pb = (float*)((char*)ws + p.off_pb);
    {
        RatioParams P;
        P.x = x; P.t1 = t1; P.z = z; P.gout = gout; P.h = h; P.bias = bias;
        P.gnum = gnum; P.gden = gden; P.gz = gz;
        P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W; P.t = p.ratio; P.eps = g.eps; P.relu = g.relu;
        auto kern = ratio_kernel<T, KD, KH, KW, kRatioNT, kRatioMAXX, VEC, WQ>;
        NDC_CUDA_TRY(set_smem(kern, p.smem_ratio));
        kern<<<(unsigned)p.n_ratio, kRatioNT, p.smem_ratio, st>>>(P);
        launched();
    }
    {
        KconvParams P;
        int n = 0;
        if (gz || gh) {
            P.in[n] = gden; P.out[n] = gt1; P.out_is_f32[n] = 1; P.aux[n] = t1; P.partial[n] = gh ? pa : nullptr;
            ++n;
        }
        if (gx || gh) {
            // without gx the convolution result goes to scratch; the pass is still needed for
            // its correlation
            P.in[n] = gnum; P.out[n] = gx ? (void*)gx : (void*)((char*)ws + p.off_gxtmp);
            P.out_is_f32[n] = 0; P.aux[n] = x; P.partial[n] = gh ? pa2 : nullptr;
            ++n;
        }
        for (int i = n; i < 2; ++i) {
            P.in[i] = nullptr; P.out[i] = nullptr; P.out_is_f32[i] = 0; P.aux[i] = nullptr; P.partial[i] = nullptr;
        }
        P.h = h; P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W; P.t = p.kconv;
        if (n > 0) {
            dim3 grid((unsigned)p.n_kconv, n);
            if (gh) {
                auto kern = kconv_kernel<T, KD, KH, KW, kKconvNT, VEC, true, WQ>;
                NDC_CUDA_TRY(set_smem(kern, p.smem_kconv));
                kern<<<grid, kKconvNT, p.smem_kconv, st>>>(P);
            } else {
                auto kern = kconv_kernel<T, KD, KH, KW, kKconvNT, VEC, false, WQ>;
                NDC_CUDA_TRY(set_smem(kern, p.smem_kconv));
                kern<<<grid, kKconvNT, p.smem_kconv, st>>>(P);
            }
            launched();
        }
    }
    if (gz || gh) {
        GzParams P;
        P.gt1 = gt1; P.z = z; P.gz = gz; P.h = h; P.bias = bias; P.partial = pb;
        P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W; P.t = p.gz; P.relu = g.relu;
        if (gh) {
            auto kern = gz_kernel<T, KD, KH, KW, kRingNT, kRingMAXX, VEC, true, WQ>;
            NDC_CUDA_TRY(set_smem(kern, p.smem_gz));
            kern<<<(unsigned)p.n_gz, kRingNT, p.smem_gz, st>>>(P);
        } else {
            auto kern = gz_kernel<T, KD, KH, KW, kRingNT, kRingMAXX, VEC, false, WQ>;
            NDC_CUDA_TRY(set_smem(kern, p.smem_gz));
            kern<<<(unsigned)p.n_gz, kRingNT, p.smem_gz, st>>>(P);
        }
        launched();
    }
    if (gh || gb) {
        ReduceParams P;
        P.partial_a = gh ? pa : nullptr;
        P.partial_a2 = gh ? pa2 : nullptr;
        P.partial_b = pb;
        P.ctas_per_bc_a = (long long)p.kconv.ndc * p.kconv.nth;
        P.ctas_per_bc_b = (long long)p.gz.ndc * p.gz.nth;
        P.b_has_w = gh ? 1 : 0;
        P.B = g.B; P.C = g.G; P.KT = g.KT; P.gh = gh; P.gb = gb;
        reduce_kernel<<<g.G, 128, 0, st>>>(P);
        launched();
    }
    return cudaGetLastError();
}

template <typename T, int KD, int KH, int KW>
cudaError_t backward_shape(const Geo& g, const BwdPlan& p, const T* x, const T* z, const T* t1,
                           const float* h, const float* bias, const T* gout, T* gx, T* gz,
                           float* gh, float* gb, void* ws, int dtype, cudaStream_t st) {
    bool vec = g.W % 4 == 0 && aligned_for_vec(x, dtype) && aligned_for_vec(z, dtype) &&
               aligned_for_vec(t1, dtype) && aligned_for_vec(gout, dtype);
    if (gx) vec = vec && aligned_for_vec(gx, dtype);
    if (gz) vec = vec && aligned_for_vec(gz, dtype);
    if constexpr (KD > 1) {
        if (vec && g.W == 64)
            return backward_launch<T, KD, KH, KW, true, 16>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
        if (vec && g.W == 128)
            return backward_launch<T, KD, KH, KW, true, 32>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
    }
    return vec ? backward_launch<T, KD, KH, KW, true, 0>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st)
               : backward_launch<T, KD, KH, KW, false, 0>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
}

template <typename T>
cudaError_t backward(const Geo& g, const BwdPlan& p, const T* x, const T* z, const T* t1,
                     const float* h, const float* bias, const T* gout, T* gx, T* gz, float* gh,
                     float* gb, void* ws, int dtype, cudaStream_t st) {
    if (g.kD == 3)
        return backward_shape<T, 3, 3, 3>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
    if (g.kH == 5)
        return backward_shape<T, 1, 5, 5>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
    return backward_shape<T, 1, 3, 3>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
}

// Whether the tiled kernels take this geometry (pointer alignment only affects vector width).
inline bool covers(const Geo& g) {
    if (g.m != 1 || g.sc != SCH || !shape_supported(g.kD, g.kH, g.kW)) return false;
    Tiling t; size_t smem;
    const long long BC = (long long)g.B * g.G;
    BwdPlan bp;
    if (!plan_bwd_any(g, bp)) return false;
    if (g.kD == 3) return plan_fwd<3, 3, 3>(g.D, g.H, g.W, BC, t, smem);
    if (g.kH == 5) return plan_fwd<1, 5, 5>(g.D, g.H, g.W, BC, t, smem);
    return plan_fwd<1, 3, 3>(g.D, g.H, g.W, BC, t, smem);
}

template <typename T>
cudaError_t forward(const Geo& g, const T* x, const T* z, const float* h, const float* bias,
                    T* out, T* t1, int dtype, cudaStream_t st, bool& handled) {
    handled = false;
    if (g.m != 1 || g.sc != SCH) return cudaSuccess;
    if (g.kD == 3 && g.kH == 3 && g.kW == 3)
        return forward_shape<T, 3, 3, 3>(g, x, z, h, bias, out, t1, dtype, st, handled);
    if (g.kD == 1 && g.kH == 5 && g.kW == 5)
        return forward_shape<T, 1, 5, 5>(g, x, z, h, bias, out, t1, dtype, st, handled);
    if (g.kD == 1 && g.kH == 3 && g.kW == 3)
        return forward_shape<T, 1, 3, 3>(g, x, z, h, bias, out, t1, dtype, st, handled);
    return cudaSuccess;
}

}  // namespace dw4
}  // namespace ndc
