// Host side of the tiled depthwise kernels: tiling decisions and launches.
#pragma once

#include <algorithm>

#include "ndc_dw4_fwd.cuh"
#include "ndc_dw4_ksrc.cuh"
#include "ndc_dw4_bwd.cuh"

namespace ndc {
namespace dw4 {

// Multiprocessors of the current device (148 on B200), asked once per process; 148 where no
// device answers (planning on a host without a GPU).
inline int num_sms() {
    static const int n = [] {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
            (void)cudaGetLastError();   // planning must not leave an error behind
            v = 148;
        }
        return v;
    }();
    return n;
}
constexpr size_t kSmemTwoPerSM = 112 * 1024;   // lets two CTAs share an SM
constexpr size_t kSmemMax = 227 * 1024;

// Launch shape per kernel geometry.
template <int KD, int KH, int KW> struct FwdShape;
template <> struct FwdShape<1, 5, 5> { static constexpr int NT = 256, MAXZ = 1, MAXX = 1, MINB = 2; };
template <> struct FwdShape<1, 3, 3> { static constexpr int NT = 256, MAXZ = 1, MAXX = 1, MINB = 2; };
// 2-D image batches run as volumes of one-row planes: rows become the marching axis,
// so nothing is recomputed between row bands and the loads of the next row overlap the work
// on this one.  A CTA is as wide as one row has 4-voxel strips.
template <int NT_> struct FwdRows { static constexpr int NT = NT_, MAXZ = 4, MAXX = 1, MINB = 384 / NT_; };
inline bool shape_supported(int kD, int kH, int kW) {
    return (kD == 3 && kH == 3 && kW == 3) || (kD == 1 && kH == 5 && kW == 5) ||
           (kD == 1 && kH == 3 && kW == 3);
}

// Chunks along depth: enough CTAs for about `waves` rounds of `ctas_per_sm` CTAs per SM, but
// chunks of at least 16*PD planes (every chunk recomputes 2*PD planes of its neighbours); only
// a grid that would not even fill the GPU once is cut finer, down to 4*PD planes.
inline void plan_depth(int KD, int D, long long ctas_per_chunk, int waves, Tiling& t,
                       int ctas_per_sm = 2) {
    if (KD == 1) {
        t.DC = 1;
    } else {
        const int PD = KD / 2;
        const long long per = std::max(1LL, ctas_per_chunk);
        const long long one_wave = (long long)ctas_per_sm * num_sms();
        long long ndc = std::min(waves * one_wave / per, (long long)std::max(1, D / (16 * PD)));
        if (ndc * per < one_wave)
            ndc = std::min((one_wave + per - 1) / per, (long long)std::max(1, D / (4 * PD)));
        ndc = std::max(1LL, ndc);
        t.DC = (int)((D + ndc - 1) / ndc);
    }
    t.ndc = (D + t.DC - 1) / t.DC;
}

template <int KD, int KH, int KW, typename S = FwdShape<KD, KH, KW>>
inline bool plan_fwd(int D, int H, int W, long long BC, Tiling& t, size_t& smem_bytes) {
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29)) return false;  // 32-bit offsets inside a slab
    if (W > ((KD > 1 && KH == 1) ? 512 : 256)) return false;   // row kernels: up to 128 strips
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
    plan_depth(KD, D, BC * t.nth, 5, t, S::MINB);
    smem_bytes = bytes(t.TH);
    return true;
}

inline bool aligned_for_vec(const void* p, int dtype) {
    return ((uintptr_t)p % (dtype == NDC_BF16 ? 8 : 16)) == 0;
}

template <typename T, int KD, int KH, int KW, typename S, bool VEC, int WQ>
cudaError_t launch_fwd(const FwdParams& P, size_t smem_bytes, long long BC, cudaStream_t st) {
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

template <typename T, int KD, int KH, int KW, typename S = FwdShape<KD, KH, KW>>
cudaError_t forward_shape(const Geo& g, const T* x, const T* z, const float* h, const float* bias,
                          T* out, T* t1, int dtype, cudaStream_t st, bool& handled) {
    FwdParams P;
    size_t smem = 0;
    const long long BC = (long long)g.B * g.G;
    handled = plan_fwd<KD, KH, KW, S>(g.D, g.H, g.W, BC, P.t, smem);
    if (!handled) return cudaSuccess;
    P.x = x; P.z = z; P.h = h; P.bias = bias; P.out = out; P.t1 = t1;
    P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W;
    P.eps = g.eps; P.relu = g.relu;
    const bool vec = g.W % 4 == 0 && aligned_for_vec(x, dtype) && aligned_for_vec(z, dtype) &&
                     aligned_for_vec(out, dtype) && aligned_for_vec(t1, dtype);
    // widths that occur in the published configurations get kernels with a compile-time width
    if constexpr (KD > 1 && KH > 1 && S::NT == 256) {
        if (vec && g.W == 64) return launch_fwd<T, KD, KH, KW, S, true, 16>(P, smem, BC, st);
        if (vec && g.W == 128) return launch_fwd<T, KD, KH, KW, S, true, 32>(P, smem, BC, st);
    }
    if constexpr (KD > 1 && KH == 1) {   // rows kernels: 256, 128 and 64 columns
        if (vec && g.W == 4 * S::NT) return launch_fwd<T, KD, KH, KW, S, true, S::NT>(P, smem, BC, st);
        if (vec && S::NT == 64 && g.W == 128) return launch_fwd<T, KD, KH, KW, S, true, 32>(P, smem, BC, st);
        if (vec && S::NT == 64 && g.W == 64) return launch_fwd<T, KD, KH, KW, S, true, 16>(P, smem, BC, st);
    }
    return vec ? launch_fwd<T, KD, KH, KW, S, true, 0>(P, smem, BC, st)
               : launch_fwd<T, KD, KH, KW, S, false, 0>(P, smem, BC, st);
}

// ---------------------------------------------------------------------------- backward

// Threads (and prefetch registers, in quads per thread) of the three backward kernels.
// Bands: a CTA owns a band of rows of every plane.  kconv: 48 strip slots x 4 channel lanes.
// Kconv2NT / Kconv2VK: threads and strip length of the packed K kernel (3x3x3 volumes): a strip
// of VK voxels per group of 4 channel lanes.  Kconv2WideNT: the CTA used instead for rows of more
// than 64 voxels (0: none), where the narrow one would be left with bands of one or two rows.
// Kconv2MAXC: 16-byte source chunks a thread copies per plane, at most (bands shrink to fit).
struct BwdBands {
    static constexpr int RatioNT = 128, RatioMAXX = 2, KconvNT = 192, GzNT = 128, GzMAXX = 4;
    static constexpr int Kconv2NT = 128, Kconv2VK = 8, Kconv2MAXC = 6, Kconv2WideNT = 256, Kconv2WideMAXC = 6;
};
// Rows: one-row planes of NQ 4-voxel strips (2-D images run as volumes, see FwdRows).
template <int NQ_> struct BwdRows {
    static constexpr int RatioNT = NQ_, RatioMAXX = 1, KconvNT = 2 * NQ_, GzNT = NQ_, GzMAXX = 1;
    // (not used: the row kernels keep two K passes)
    static constexpr int Kconv2NT = 4 * NQ_, Kconv2VK = 4, Kconv2MAXC = 4, Kconv2WideNT = 0, Kconv2WideMAXC = 0;
};
// Small volumes (3x3x3): narrower CTAs where they cover the same bands as the default ones
// (a wide CTA would mostly idle on a band of 16 or 8 short rows).
struct BwdSmall16 {   // bands of up to 64 strips of 4 (16 x 16 rows)
    static constexpr int RatioNT = 64, RatioMAXX = 2, KconvNT = 128, GzNT = 64, GzMAXX = 2;
    static constexpr int Kconv2NT = 128, Kconv2VK = 8, Kconv2MAXC = 6, Kconv2WideNT = 0, Kconv2WideMAXC = 0;
};
struct BwdSmall8 {    // bands of up to 32 strips of 4 (8 x 8 rows)
    static constexpr int RatioNT = 32, RatioMAXX = 1, KconvNT = 32, GzNT = 32, GzMAXX = 1;
    static constexpr int Kconv2NT = 32, Kconv2VK = 8, Kconv2MAXC = 5, Kconv2WideNT = 0, Kconv2WideMAXC = 0;
};
constexpr int kGzCS = 1;        // channel split of gz_kernel (2 was measured no faster)

// Band height for the kernels that only hold single-channel rings (ratio: 2 tensors, gz: 1).
template <int KD, int KH, int KW>
inline bool plan_ring(int D, int H, int W, long long BC, int ntensors, int nt, int maxx,
                      int red_floats, size_t extra_bytes, size_t smem_target, int ctas_per_sm,
                      Tiling& t, size_t& smem_bytes) {
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29) || W > ((KD > 1 && KH == 1) ? 512 : 256)) return false;
    t.NQ = (W + 3) / 4;
    t.pitch = row_pitch(W);
    int TH = H;
    if (KD > 1) TH = std::min(TH, nt * maxx / t.NQ - 2 * PH);
    auto bytes = [&](int th) {
        Tiling q = t; q.TH = th;
        return (size_t)RingSmem<KD, KH, KW>(q, ntensors, red_floats).total_floats * sizeof(float) +
               extra_bytes;
    };
    while (TH > 1 && (bytes(TH) > smem_target || (TH + 2 * PH) * t.pitch > 65535)) --TH;
    if (TH < 1 || bytes(TH) > kSmemMax) return false;
    t.nth = (H + TH - 1) / TH;
    if (KD > 1) {
        // A plane's strips are worked off in rounds of `nt` (one strip per thread): prefer the
        // band count whose bands fill their rounds (13 rows of 16 strips on 128 threads waste
        // 3/8 of every second round, 8 rows none), against the two halo rows a band reloads.
        double best = -1.0;
        int best_nth = t.nth;
        for (int nth = t.nth; nth <= std::min(H, 4 * t.nth); ++nth) {
            const int th = (H + nth - 1) / nth;
            if ((nth - 1) * th >= H) continue;                     // an empty last band
            const int last = H - (nth - 1) * th;
            const long long rounds = (long long)(nth - 1) * (((long long)th * t.NQ + nt - 1) / nt) +
                                     ((long long)last * t.NQ + nt - 1) / nt;
            const double fill = (double)H * t.NQ / ((double)rounds * nt);
            const double score = fill / (1.0 + 0.3 * PH * nth / H);
            if (score > best * 1.001) { best = score; best_nth = nth; }
        }
        t.nth = best_nth;
    }
    t.TH = (H + t.nth - 1) / t.nth;
    plan_depth(KD, D, BC * t.nth, 4, t, ctas_per_sm);
    smem_bytes = bytes(t.TH);
    return true;
}

template <int KD, int KH, int KW, int NT>
inline bool plan_kconv(int D, int H, int W, long long BC, Tiling& t, size_t& smem_bytes) {
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29) || W > ((KD > 1 && KH == 1) ? 512 : 256)) return false;
    t.NQ = (W + 3) / 4;
    t.pitch = row_pitch(W);
    const int NS8 = (t.NQ + 1) / 2;
    int TH = H;
    if (KD > 1) {
        TH = std::min(TH, (NT / SCH) / NS8);
    }
    auto bytes = [&](int th) {
        Tiling q = t; q.TH = th;
        return (size_t)KconvSmem<KD, KH, KW>(q, NT).total_floats * sizeof(float);
    };
    while (TH > 1 && (bytes(TH) > 72 * 1024 || SCH * (TH + 2 * PH) * t.pitch > 65535)) --TH;
    if (TH < 1 || bytes(TH) > kSmemMax) return false;
    t.nth = (H + TH - 1) / TH;
    t.TH = (H + t.nth - 1) / t.nth;
    plan_depth(KD, D, 2 * BC * t.nth, 6, t, 384 / NT);
    smem_bytes = bytes(t.TH);
    return true;
}

// The packed K kernel (both scratch tensors in one pass) serves the 3x3x3 volumes.
template <int KD, int KH, int KW>
constexpr bool packed_kconv() { return KD == 3 && KH == 3 && KW == 3; }

template <int KD, int KH, int KW, int NT, int VK, int MAXC>
inline bool plan_kconv2(int D, int H, int W, long long BC, Tiling& t, size_t& smem_bytes) {
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29) || W > 256) return false;
    t.NQ = (W + 3) / 4;
    t.pitch = row_pitch(W);
    const int NSV = (4 * t.NQ + VK - 1) / VK;
    int TH = std::min(H, (NT / SCH) / NSV);            // one strip per group of 4 channel lanes
    auto bytes = [&](int th) {
        Tiling q = t; q.TH = th;
        return (size_t)Kconv2Smem<KD, KH, KW>(q, NT).total_floats * sizeof(float);
    };
    auto chunks = [&](int th) { return SCH * (th + 2 * PH) * 2 * t.NQ; };
    constexpr int per_sm = kconv2_min_blocks<NT, VK>();
    const size_t target = (kSmemMax - 8 * 1024) / per_sm;
    while (TH > 1 && (bytes(TH) > target || chunks(TH) > MAXC * NT ||
                      SCH * (TH + 2 * PH) * 2 * t.pitch >= (1 << 26)))
        --TH;
    if (TH < 1 || bytes(TH) > target || chunks(TH) > MAXC * NT) return false;
    t.nth = (H + TH - 1) / TH;
    t.TH = (H + t.nth - 1) / t.nth;
    plan_depth(KD, D, BC * t.nth, 6, t, per_sm);
    smem_bytes = bytes(t.TH);
    return true;
}

struct BwdPlan {
    Tiling ratio, kconv, gz;
    size_t smem_ratio, smem_kconv, smem_gz;
    size_t off_gnum, off_gden, off_gt1, off_gxtmp, off_pa, off_pa2, off_pb, bytes;
    long long n_ratio, n_kconv, n_gz;   // CTAs (kconv: per tensor; = partial records)
    int kconv_wide;                     // packed K kernel: the wide CTA was planned
    int rows;                           // 0: band kernels; else the rows class planned
    int small;                          // 0, or the small-volume class planned (16 or 8)
};

template <int KD, int KH, int KW, typename S>
inline bool plan_bwd(const Geo& g, BwdPlan& p) {
    const long long BC = (long long)g.B * g.G;
    if (!plan_ring<KD, KH, KW>(g.D, g.H, g.W, BC, 2, S::RatioNT, S::RatioMAXX, 0, 0, 56 * 1024,
                               512 / S::RatioNT, p.ratio, p.smem_ratio))
        return false;
    p.kconv_wide = 0;
    if constexpr (packed_kconv<KD, KH, KW>()) {
        bool ok = false;
        if constexpr (S::Kconv2WideNT > 0) {
            if (g.W > 64) {
                ok = plan_kconv2<KD, KH, KW, S::Kconv2WideNT, S::Kconv2VK, S::Kconv2WideMAXC>(g.D, g.H, g.W, BC, p.kconv, p.smem_kconv);
                p.kconv_wide = ok ? 1 : 0;
            }
        }
        if (!ok && !plan_kconv2<KD, KH, KW, S::Kconv2NT, S::Kconv2VK, S::Kconv2MAXC>(g.D, g.H, g.W, BC, p.kconv, p.smem_kconv))
            return false;
    } else {
        if (!plan_kconv<KD, KH, KW, S::KconvNT>(g.D, g.H, g.W, BC, p.kconv, p.smem_kconv)) return false;
    }
    // gz_kernel also double-buffers its strips of z and of the direct term (16 bytes each)
    if (!plan_ring<KD, KH, KW>(g.D, g.H, g.W, BC, 1, S::GzNT, S::GzMAXX,
                               gz_combine_floats<KD, KH, KW, kGzCS>(S::GzNT),
                               (size_t)2 * 2 * (SCH / kGzCS) * S::GzNT * 16, kSmemTwoPerSM,
                               256 / S::GzNT, p.gz, p.smem_gz))
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

// 2-D batches (5x5 or 3x3 kernels, up to 512 columns, at least 8 rows) are run as ONE volume per
// group whose planes are the image rows and whose plane rows are the images of the batch (the
// same memory and the same filter layout; kernel K x 1 x K, so images never mix).  A CTA takes
// as many images as fill its threads (one image of 129..512 columns, four of 64, ...).  Returns
// the CTA size class (strips of 4 per CTA), or 0 where the band kernels stay: a batch too small
// to fill even the small CTA, or a band whose 32-bit offsets would overflow.
inline int rows_class(const Geo& g) {
    if (g.D != 1 || g.kD != 1 || g.kH != g.kW || (g.kH != 5 && g.kH != 3) || g.H < 8) return 0;
    const int NQ = (g.W + 3) / 4;
    if (NQ > 128) return 0;
    const int images = NQ > 64 ? 1 : std::min(g.B, 64 / NQ);   // per CTA
    const long long image = (long long)g.H * g.W;       // elements of one channel
    if ((images * (long long)g.G + 1) * SCH * image >= (1LL << 31)) return 0;
    const int strips = images * NQ;
    return strips > 64 ? 128 : strips > 32 ? 64 : strips >= 24 ? 32 : 0;
}
inline Geo as_rows(const Geo& g) {
    Geo v = g;
    v.B = 1; v.D = g.H; v.H = g.B;
    v.kD = g.kH; v.kH = 1; v.pD = g.pH; v.pH = 0;
    v.SP = (long long)v.D * v.H * v.W;
    return v;
}

// K x K images: row kernels where rows_class allows, else band kernels.
template <int K>
inline bool plan_bwd_image(const Geo& g, BwdPlan& p) {
    const int rc = rows_class(g);
    p.rows = rc;
    if (rc == 128 && plan_bwd<K, 1, K, BwdRows<128>>(as_rows(g), p)) return true;
    if (rc == 64 && plan_bwd<K, 1, K, BwdRows<64>>(as_rows(g), p)) return true;
    if (rc == 32 && plan_bwd<K, 1, K, BwdRows<32>>(as_rows(g), p)) return true;
    p.rows = 0;
    return plan_bwd<1, K, K, BwdBands>(g, p);
}

inline bool plan_bwd_any(const Geo& g, BwdPlan& p) {
    p.rows = 0; p.small = 0;
    if (g.m != 1 || g.sc != SCH) return false;
    if (g.kD == 3 && g.kH == 3 && g.kW == 3) {
        BwdPlan p0;
        if (!plan_bwd<3, 3, 3, BwdBands>(g, p0)) return false;
        auto same_bands = [&](const BwdPlan& q) {
            return q.ratio.nth == p0.ratio.nth && q.kconv.nth == p0.kconv.nth && q.gz.nth == p0.gz.nth;
        };
        p.small = 8;
        if (plan_bwd<3, 3, 3, BwdSmall8>(g, p) && same_bands(p)) return true;
        p.small = 16;
        if (plan_bwd<3, 3, 3, BwdSmall16>(g, p) && same_bands(p)) return true;
        p = p0;
        p.rows = 0; p.small = 0;
        return true;
    }
    if (g.kD == 1 && g.kH == 5 && g.kW == 5) return plan_bwd_image<5>(g, p);
    if (g.kD == 1 && g.kH == 3 && g.kW == 3) return plan_bwd_image<3>(g, p);
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

template <typename T, int KD, int KH, int KW, typename S, bool VEC, int WQ>
cudaError_t backward_launch(const Geo& g, const BwdPlan& p, const T* x, const T* z, const T* t1,
                            const float* h, const float* bias, const T* gout, T* gx, T* gz,
                            float* gh, float* gb, void* ws, cudaStream_t st) {
    float* gnum = (float*)((char*)ws + p.off_gnum);
    float* gden = (float*)((char*)ws + p.off_gden);
    float* gt1 = (float*)((char*)ws + p.off_gt1);
    float* pa = (float*)((char*)ws + p.off_pa);
    float* pa2 = (float*)((char*)ws + p.off_pa2);
    float* pb = (float*)((char*)ws + p.off_pb);
    if (p.n_ratio > 0x7fffffffLL || p.n_kconv > 0x7fffffffLL || p.n_gz > 0x7fffffffLL)
        return cudaErrorInvalidConfiguration;
    {
        RatioParams P;
        P.x = x; P.t1 = t1; P.z = z; P.gout = gout; P.h = h; P.bias = bias;
        P.gnum = gnum; P.gden = gden; P.gz = gz;
        P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W; P.t = p.ratio; P.eps = g.eps; P.relu = g.relu;
        auto kern = ratio_kernel<T, KD, KH, KW, S::RatioNT, S::RatioMAXX, VEC, WQ, packed_kconv<KD, KH, KW>() ? kRatioPairs : kRatioPlanar>;
        NDC_CUDA_TRY(set_smem(kern, p.smem_ratio));
        kern<<<(unsigned)p.n_ratio, S::RatioNT, p.smem_ratio, st>>>(P);
        launched();
    }
    if constexpr (packed_kconv<KD, KH, KW>()) {
        Kconv2Params P;
        P.in = gnum;                          // (gden, gnum) pairs fill the gnum | gden area
        P.gt1 = (gz || gh) ? gt1 : nullptr;
        P.gx = gx;
        P.t1 = t1; P.x = x;
        P.partial = gh ? pa : nullptr;
        P.h = h; P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W; P.t = p.kconv;
        auto run = [&](auto nt, auto maxc) -> cudaError_t {
            constexpr int NT = decltype(nt)::value, VK = S::Kconv2VK, MAXC = decltype(maxc)::value;
            if (gh) {
                auto kern = kconv2_kernel<T, KD, KH, KW, NT, VK, MAXC, VEC, true, WQ>;
                NDC_CUDA_TRY(set_smem(kern, p.smem_kconv));
                kern<<<(unsigned)p.n_kconv, NT, p.smem_kconv, st>>>(P);
            } else {
                auto kern = kconv2_kernel<T, KD, KH, KW, NT, VK, MAXC, VEC, false, WQ>;
                NDC_CUDA_TRY(set_smem(kern, p.smem_kconv));
                kern<<<(unsigned)p.n_kconv, NT, p.smem_kconv, st>>>(P);
            }
            return cudaSuccess;
        };
        if constexpr (S::Kconv2WideNT > 0) {
            if (p.kconv_wide)
                NDC_CUDA_TRY(run(std::integral_constant<int, S::Kconv2WideNT>{}, std::integral_constant<int, S::Kconv2WideMAXC>{}));
            else
                NDC_CUDA_TRY(run(std::integral_constant<int, S::Kconv2NT>{}, std::integral_constant<int, S::Kconv2MAXC>{}));
        } else {
            NDC_CUDA_TRY(run(std::integral_constant<int, S::Kconv2NT>{}, std::integral_constant<int, S::Kconv2MAXC>{}));
        }
        launched();
    } else {
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
                auto kern = kconv_kernel<T, KD, KH, KW, S::KconvNT, VEC, true, WQ>;
                NDC_CUDA_TRY(set_smem(kern, p.smem_kconv));
                kern<<<grid, S::KconvNT, p.smem_kconv, st>>>(P);
            } else {
                auto kern = kconv_kernel<T, KD, KH, KW, S::KconvNT, VEC, false, WQ>;
                NDC_CUDA_TRY(set_smem(kern, p.smem_kconv));
                kern<<<grid, S::KconvNT, p.smem_kconv, st>>>(P);
            }
            launched();
        }
    }
    if (gz || gh) {
        GzParams P;
        P.gt1 = gt1; P.z = z; P.gz = gz; P.h = h; P.bias = bias; P.partial = pb;
        P.C = g.G; P.D = g.D; P.H = g.H; P.W = g.W; P.t = p.gz; P.relu = g.relu;
        if (gh) {
            auto kern = gz_kernel<T, KD, KH, KW, S::GzNT, S::GzMAXX, VEC, true, WQ, kGzCS>;
            NDC_CUDA_TRY(set_smem(kern, p.smem_gz));
            kern<<<(unsigned)p.n_gz, S::GzNT, p.smem_gz, st>>>(P);
        } else {
            auto kern = gz_kernel<T, KD, KH, KW, S::GzNT, S::GzMAXX, VEC, false, WQ, kGzCS>;
            NDC_CUDA_TRY(set_smem(kern, p.smem_gz));
            kern<<<(unsigned)p.n_gz, S::GzNT, p.smem_gz, st>>>(P);
        }
        launched();
    }
    if (gh || gb) {
        ReduceParams P;
        P.partial_a = gh ? pa : nullptr;
        P.partial_a2 = (gh && !packed_kconv<KD, KH, KW>()) ? pa2 : nullptr;   // packed: one record set
        P.partial_b = pb;
        P.ctas_per_bc_a = (long long)p.kconv.ndc * p.kconv.nth;
        P.ctas_per_bc_b = (long long)p.gz.ndc * p.gz.nth;
        P.b_has_w = gh ? 1 : 0;
        P.B = g.B; P.C = g.G; P.KT = g.KT; P.gh = gh; P.gb = gb;
        reduce_kernel<kPartialStride><<<g.G, kPartialStride, 0, st>>>(P);
        launched();
    }
    return cudaGetLastError();
}

template <typename T, int KD, int KH, int KW, typename S>
cudaError_t backward_shape(const Geo& g, const BwdPlan& p, const T* x, const T* z, const T* t1,
                           const float* h, const float* bias, const T* gout, T* gx, T* gz,
                           float* gh, float* gb, void* ws, int dtype, cudaStream_t st) {
    bool vec = g.W % 4 == 0 && aligned_for_vec(x, dtype) && aligned_for_vec(z, dtype) &&
               aligned_for_vec(t1, dtype) && aligned_for_vec(gout, dtype);
    if (gx) vec = vec && aligned_for_vec(gx, dtype);
    if (gz) vec = vec && aligned_for_vec(gz, dtype);
    // widths that occur in the published configurations get kernels with a compile-time width
    if constexpr (KD > 1 && KH > 1 && S::RatioNT == 128) {
        if (vec && g.W == 64)
            return backward_launch<T, KD, KH, KW, S, true, 16>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
        if (vec && g.W == 128)
            return backward_launch<T, KD, KH, KW, S, true, 32>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
    }
    if constexpr (KD > 1 && KH == 1) {   // rows kernels: 256, 128 and 64 columns
        if (vec && g.W == 4 * S::RatioNT)
            return backward_launch<T, KD, KH, KW, S, true, S::RatioNT>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
        if (vec && S::RatioNT == 64 && g.W == 128)
            return backward_launch<T, KD, KH, KW, S, true, 32>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
        if (vec && S::RatioNT == 64 && g.W == 64)
            return backward_launch<T, KD, KH, KW, S, true, 16>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
    }
    return vec ? backward_launch<T, KD, KH, KW, S, true, 0>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st)
               : backward_launch<T, KD, KH, KW, S, false, 0>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, st);
}

template <typename T, int K>
cudaError_t backward_image(const Geo& g, const BwdPlan& p, const T* x, const T* z, const T* t1,
                           const float* h, const float* bias, const T* gout, T* gx, T* gz,
                           float* gh, float* gb, void* ws, int dtype, cudaStream_t st) {
    if (p.rows == 128)
        return backward_shape<T, K, 1, K, BwdRows<128>>(as_rows(g), p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
    if (p.rows == 64)
        return backward_shape<T, K, 1, K, BwdRows<64>>(as_rows(g), p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
    if (p.rows == 32)
        return backward_shape<T, K, 1, K, BwdRows<32>>(as_rows(g), p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
    return backward_shape<T, 1, K, K, BwdBands>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
}

// `p` must come from plan_bwd_any(g): the same rule picks the kernel family here.
template <typename T>
cudaError_t backward(const Geo& g, const BwdPlan& p, const T* x, const T* z, const T* t1,
                     const float* h, const float* bias, const T* gout, T* gx, T* gz, float* gh,
                     float* gb, void* ws, int dtype, cudaStream_t st) {
    if (g.kD == 3) {
        if (p.small == 8)
            return backward_shape<T, 3, 3, 3, BwdSmall8>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
        if (p.small == 16)
            return backward_shape<T, 3, 3, 3, BwdSmall16>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
        return backward_shape<T, 3, 3, 3, BwdBands>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
    }
    if (g.kH == 5) return backward_image<T, 5>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
    return backward_image<T, 3>(g, p, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws, dtype, st);
}

// ---------------------------------------------------------------- two-launch forward (3x3x3)
// t1 = K(relu(z + b)) by ksrc_kernel, then out by ratio_kernel<kRatioForward>.  Measured against
// the fused fwd_kernel on every stage geometry of the 3-D networks (64^3 x 64 channels ... 8^3 x
// 512, 128^3) it is 17-29 % faster: no row of t1 is computed twice, the K pass is packed, and
// both launches run four or more small CTAs per multiprocessor.  The price is traffic: t1 and z
// are read once more (15 instead of 10 tensor units), which this arithmetic-bound path can pay.
template <int NT_, int MINB_> struct KsrcShape { static constexpr int NT = NT_, MAXZP = 3, MINB = MINB_; };

template <int KD, int KH, int KW, typename S>
inline bool plan_ksrc(int D, int H, int W, long long BC, Tiling& t, size_t& smem_bytes) {
    constexpr int PH = KH / 2;
    if ((long long)D * H * W >= (1LL << 29) || W > 256) return false;
    t.NQ = (W + 3) / 4;
    t.pitch = row_pitch(W);
    const int NS8 = (t.NQ + 1) / 2;
    int TH = std::min(H, (S::NT / 2) / NS8);                           // one strip per thread pair
    TH = std::min(TH, S::NT * S::MAXZP / (2 * t.NQ) - 2 * PH);         // source prefetch registers
    auto bytes = [&](int th) {
        Tiling q = t; q.TH = th;
        return (size_t)KsrcSmem<KD, KH, KW>(q).total_floats * sizeof(float);
    };
    const size_t target = (kSmemMax - 8 * 1024) / S::MINB;
    while (TH > 1 && bytes(TH) > target) --TH;
    if (TH < 1 || bytes(TH) > target) return false;
    t.nth = (H + TH - 1) / TH;
    t.TH = (H + t.nth - 1) / t.nth;
    plan_depth(KD, D, BC * t.nth, 6, t, S::MINB);
    smem_bytes = bytes(t.TH);
    return true;
}

template <typename T, int KD, int KH, int KW, typename S>
cudaError_t launch_ksrc(const KsrcParams& P, size_t smem_bytes, long long BC, bool vec, cudaStream_t st) {
    const long long grid = BC * P.t.ndc * P.t.nth;
    if (grid > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    auto go = [&](auto kern) -> cudaError_t {
        NDC_CUDA_TRY(set_smem(kern, smem_bytes));
        kern<<<(unsigned)grid, S::NT, smem_bytes, st>>>(P);
        launched();
        return cudaSuccess;
    };
    if (vec && P.W == 64) return go(ksrc_kernel<T, KD, KH, KW, S::NT, S::MAXZP, S::MINB, true, 16>);
    if (vec && P.W == 128) return go(ksrc_kernel<T, KD, KH, KW, S::NT, S::MAXZP, S::MINB, true, 32>);
    return vec ? go(ksrc_kernel<T, KD, KH, KW, S::NT, S::MAXZP, S::MINB, true, 0>)
               : go(ksrc_kernel<T, KD, KH, KW, S::NT, S::MAXZP, S::MINB, false, 0>);
}

template <typename T, int KD, int KH, int KW, typename S>
cudaError_t launch_ratio_forward(const RatioParams& P, size_t smem_bytes, long long n_ctas, bool vec,
                                 cudaStream_t st) {
    if (n_ctas > 0x7fffffffLL) return cudaErrorInvalidConfiguration;
    auto go = [&](auto kern) -> cudaError_t {
        NDC_CUDA_TRY(set_smem(kern, smem_bytes));
        kern<<<(unsigned)n_ctas, S::RatioNT, smem_bytes, st>>>(P);
        launched();
        return cudaSuccess;
    };
    if (vec && P.W == 64) return go(ratio_kernel<T, KD, KH, KW, S::RatioNT, S::RatioMAXX, true, 16, kRatioForward>);
    if (vec && P.W == 128) return go(ratio_kernel<T, KD, KH, KW, S::RatioNT, S::RatioMAXX, true, 32, kRatioForward>);
    return vec ? go(ratio_kernel<T, KD, KH, KW, S::RatioNT, S::RatioMAXX, true, 0, kRatioForward>)
               : go(ratio_kernel<T, KD, KH, KW, S::RatioNT, S::RatioMAXX, false, 0, kRatioForward>);
}

template <typename T>
cudaError_t forward_split(const Geo& g, const T* x, const T* z, const float* h, const float* bias,
                          T* out, T* t1, int dtype, cudaStream_t st, bool& handled) {
    constexpr int KD = 3, KH = 3, KW = 3;
    const long long BC = (long long)g.B * g.G;
    const bool vec = g.W % 4 == 0 && aligned_for_vec(x, dtype) && aligned_for_vec(z, dtype) &&
                     aligned_for_vec(out, dtype) && aligned_for_vec(t1, dtype);
    handled = false;
    // ---- K: the narrowest CTA that covers the volume with as few bands as the widest
    KsrcParams K;
    K.z = z; K.h = h; K.bias = bias; K.t1 = t1;
    K.C = g.G; K.D = g.D; K.H = g.H; K.W = g.W; K.relu = g.relu;
    Tiling t0, tk; size_t sm0 = 0, smk = 0;
    typedef KsrcShape<128, 3> K128; typedef KsrcShape<64, 6> K64; typedef KsrcShape<32, 12> K32;
    if (!plan_ksrc<KD, KH, KW, K128>(g.D, g.H, g.W, BC, t0, sm0)) return cudaSuccess;
    // ---- A: the same classes as the backward's ratio kernel
    RatioParams R;
    R.x = x; R.t1 = t1; R.z = z; R.gout = nullptr; R.h = h; R.bias = bias;
    R.gnum = nullptr; R.gden = nullptr; R.gz = out;
    R.C = g.G; R.D = g.D; R.H = g.H; R.W = g.W; R.eps = g.eps; R.relu = g.relu;
    Tiling r0; size_t smr0 = 0;
    if (!plan_ring<KD, KH, KW>(g.D, g.H, g.W, BC, 2, BwdBands::RatioNT, BwdBands::RatioMAXX, 0, 0,
                               56 * 1024, 512 / BwdBands::RatioNT, r0, smr0))
        return cudaSuccess;
    handled = true;
    if (plan_ksrc<KD, KH, KW, K32>(g.D, g.H, g.W, BC, tk, smk) && tk.nth == t0.nth) {
        K.t = tk; NDC_CUDA_TRY((launch_ksrc<T, KD, KH, KW, K32>(K, smk, BC, vec, st)));
    } else if (plan_ksrc<KD, KH, KW, K64>(g.D, g.H, g.W, BC, tk, smk) && tk.nth == t0.nth) {
        K.t = tk; NDC_CUDA_TRY((launch_ksrc<T, KD, KH, KW, K64>(K, smk, BC, vec, st)));
    } else {
        K.t = t0; NDC_CUDA_TRY((launch_ksrc<T, KD, KH, KW, K128>(K, sm0, BC, vec, st)));
    }
    Tiling tr; size_t smr = 0;
    if (plan_ring<KD, KH, KW>(g.D, g.H, g.W, BC, 2, BwdSmall8::RatioNT, BwdSmall8::RatioMAXX, 0, 0,
                              56 * 1024, 512 / BwdSmall8::RatioNT, tr, smr) && tr.nth == r0.nth) {
        R.t = tr; NDC_CUDA_TRY((launch_ratio_forward<T, KD, KH, KW, BwdSmall8>(R, smr, BC * tr.ndc * tr.nth, vec, st)));
    } else if (plan_ring<KD, KH, KW>(g.D, g.H, g.W, BC, 2, BwdSmall16::RatioNT, BwdSmall16::RatioMAXX, 0, 0,
                                     56 * 1024, 512 / BwdSmall16::RatioNT, tr, smr) && tr.nth == r0.nth) {
        R.t = tr; NDC_CUDA_TRY((launch_ratio_forward<T, KD, KH, KW, BwdSmall16>(R, smr, BC * tr.ndc * tr.nth, vec, st)));
    } else {
        R.t = r0; NDC_CUDA_TRY((launch_ratio_forward<T, KD, KH, KW, BwdBands>(R, smr0, BC * r0.ndc * r0.nth, vec, st)));
    }
    return cudaGetLastError();
}

// Forward plan of a K x K image batch: the row kernels of its class, else the band kernels.
template <int K>
inline bool plan_fwd_image(const Geo& g) {
    Tiling t; size_t smem;
    const int rc = rows_class(g);
    if (rc) {
        const Geo v = as_rows(g);
        const long long BC = (long long)v.B * v.G;
        if (rc == 128 && plan_fwd<K, 1, K, FwdRows<128>>(v.D, v.H, v.W, BC, t, smem)) return true;
        if (rc == 64 && plan_fwd<K, 1, K, FwdRows<64>>(v.D, v.H, v.W, BC, t, smem)) return true;
        if (rc == 32 && plan_fwd<K, 1, K, FwdRows<32>>(v.D, v.H, v.W, BC, t, smem)) return true;
    }
    return plan_fwd<1, K, K>(g.D, g.H, g.W, (long long)g.B * g.G, t, smem);
}

// Whether the tiled kernels take this geometry (pointer alignment only affects vector width).
inline bool covers(const Geo& g) {
    if (g.m != 1 || g.sc != SCH || !shape_supported(g.kD, g.kH, g.kW)) return false;
    Tiling t; size_t smem;
    const long long BC = (long long)g.B * g.G;
    BwdPlan bp;
    if (!plan_bwd_any(g, bp)) return false;
    if (g.kD == 3)
        return plan_ksrc<3, 3, 3, KsrcShape<128, 3>>(g.D, g.H, g.W, BC, t, smem) &&
               plan_ring<3, 3, 3>(g.D, g.H, g.W, BC, 2, BwdBands::RatioNT, BwdBands::RatioMAXX, 0, 0,
                                  56 * 1024, 512 / BwdBands::RatioNT, t, smem);
    if (g.kH == 5) return plan_fwd_image<5>(g);
    return plan_fwd_image<3>(g);
}

template <typename T, int K>
cudaError_t forward_image(const Geo& g, const T* x, const T* z, const float* h, const float* bias,
                          T* out, T* t1, int dtype, cudaStream_t st, bool& handled) {
    const int rc = rows_class(g);
    if (rc) {
        const Geo v = as_rows(g);
        cudaError_t e = rc == 128
            ? forward_shape<T, K, 1, K, FwdRows<128>>(v, x, z, h, bias, out, t1, dtype, st, handled)
            : rc == 64
            ? forward_shape<T, K, 1, K, FwdRows<64>>(v, x, z, h, bias, out, t1, dtype, st, handled)
            : forward_shape<T, K, 1, K, FwdRows<32>>(v, x, z, h, bias, out, t1, dtype, st, handled);
        if (handled || e != cudaSuccess) return e;
    }
    return forward_shape<T, 1, K, K>(g, x, z, h, bias, out, t1, dtype, st, handled);
}

template <typename T>
cudaError_t forward(const Geo& g, const T* x, const T* z, const float* h, const float* bias,
                    T* out, T* t1, int dtype, cudaStream_t st, bool& handled) {
    handled = false;
    if (g.m != 1 || g.sc != SCH) return cudaSuccess;
    if (g.kD == 3 && g.kH == 3 && g.kW == 3)
        return forward_split<T>(g, x, z, h, bias, out, t1, dtype, st, handled);
    if (g.kD == 1 && g.kH == 5 && g.kW == 5)
        return forward_image<T, 5>(g, x, z, h, bias, out, t1, dtype, st, handled);
    if (g.kD == 1 && g.kH == 3 && g.kW == 3)
        return forward_image<T, 3>(g, x, z, h, bias, out, t1, dtype, st, handled);
    return cudaSuccess;
}

// ---------------------------------------------------------------------------------------
// The kernels are compiled in several translation units (ndc_dw4_inst.cu, once per part and
// storage type) so that the build can use several host cores.  NDC_DW4_INSTANCES(PREFIX, T)
// lists every heavy instantiation of part NDC_DW4_PART: PREFIX is `template` where they are
// compiled and `extern template` in the translation unit that only calls them.
#define NDC_DW4_FWD_INSTANCES(PREFIX, T)                                                      \
    PREFIX cudaError_t forward<T>(const Geo&, const T*, const T*, const float*, const float*, \
                                  T*, T*, int, cudaStream_t, bool&);
#define NDC_DW4_BWD_ARGS(T)                                                                   \
    (const Geo&, const BwdPlan&, const T*, const T*, const T*, const float*, const float*,    \
     const T*, T*, T*, float*, float*, void*, int, cudaStream_t)
#define NDC_DW4_BWD3D_INSTANCES(PREFIX, T)                                                    \
    PREFIX cudaError_t backward_shape<T, 3, 3, 3, BwdBands> NDC_DW4_BWD_ARGS(T);              \
    PREFIX cudaError_t backward_shape<T, 3, 3, 3, BwdSmall16> NDC_DW4_BWD_ARGS(T);            \
    PREFIX cudaError_t backward_shape<T, 3, 3, 3, BwdSmall8> NDC_DW4_BWD_ARGS(T);
#define NDC_DW4_BWD2D_INSTANCES(PREFIX, T)                                                    \
    PREFIX cudaError_t backward_shape<T, 1, 5, 5, BwdBands> NDC_DW4_BWD_ARGS(T);              \
    PREFIX cudaError_t backward_shape<T, 1, 3, 3, BwdBands> NDC_DW4_BWD_ARGS(T);              \
    PREFIX cudaError_t backward_shape<T, 5, 1, 5, BwdRows<128>> NDC_DW4_BWD_ARGS(T);          \
    PREFIX cudaError_t backward_shape<T, 3, 1, 3, BwdRows<128>> NDC_DW4_BWD_ARGS(T);          \
    PREFIX cudaError_t backward_shape<T, 5, 1, 5, BwdRows<64>> NDC_DW4_BWD_ARGS(T);           \
    PREFIX cudaError_t backward_shape<T, 5, 1, 5, BwdRows<32>> NDC_DW4_BWD_ARGS(T);           \
    PREFIX cudaError_t backward_shape<T, 3, 1, 3, BwdRows<64>> NDC_DW4_BWD_ARGS(T);           \
    PREFIX cudaError_t backward_shape<T, 3, 1, 3, BwdRows<32>> NDC_DW4_BWD_ARGS(T);

#ifdef NDC_DW4_EXTERN
NDC_DW4_FWD_INSTANCES(extern template, float)
NDC_DW4_FWD_INSTANCES(extern template, __nv_bfloat16)
NDC_DW4_BWD3D_INSTANCES(extern template, float)
NDC_DW4_BWD3D_INSTANCES(extern template, __nv_bfloat16)
NDC_DW4_BWD2D_INSTANCES(extern template, float)
NDC_DW4_BWD2D_INSTANCES(extern template, __nv_bfloat16)
#endif

}  // namespace dw4
}  // namespace ndc
