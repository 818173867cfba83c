// Host side of the tiled depthwise kernels: tiling decisions and launches.
#pragma once

#include <algorithm>

#include "ndc_dw4_fwd.cuh"

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
        TH = std::min(TH, S::NT / NS8 - 2 * PH);                         // one K strip per thread
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

template <typename T, int KD, int KH, int KW, bool VEC>
cudaError_t launch_fwd(const FwdParams& P, size_t smem_bytes, long long BC, cudaStream_t st) {
    using S = FwdShape<KD, KH, KW>;
    auto kern = fwd_kernel<T, KD, KH, KW, S::NT, S::MAXZ, S::MAXX, S::MINB, VEC>;
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
    return vec ? launch_fwd<T, KD, KH, KW, true>(P, smem, BC, st)
               : launch_fwd<T, KD, KH, KW, false>(P, smem, BC, st);
}

// Whether the tiled kernels take this geometry (pointer alignment only affects vector width).
inline bool covers(const Geo& g) {
    if (g.m != 1 || g.sc != SCH || !shape_supported(g.kD, g.kH, g.kW)) return false;
    Tiling t; size_t smem;
    const long long BC = (long long)g.B * g.G;
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
