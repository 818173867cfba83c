// First half of the two-launch forward of 3-D kernels:  t1 = K(relu(z + b)).
//
// (The second half is ratio_kernel<kRatioForward>: out = (s * (A(x) + eps)) / (A(t1) + eps).)
// One CTA owns a (sample, group) pair, a band of TH rows and a chunk of planes and marches through
// the chunk.  A source plane is fetched into registers one step ahead, biased and rectified ONCE,
// and written to shared memory as rows of (s[2c], s[2c+1]) PAIRS, c = channel pair 0 or 1.  A
// thread convolves one channel pair of an 8-voxel strip with two-lane `fma.rn.f32x2`: lane 0 of
// its KD running sums collects channel 2c, lane 1 channel 2c+1 (the filter is staged as
// (h[2c], h[2c+1]) pairs), so a 64-bit shared-memory element is a ready operand.  When a plane
// completes, the two lanes and the two channel pairs (one shuffle) are added and the strip goes
// to HBM.  Unlike the fused kernel, no row of t1 is computed twice: neighbouring bands only
// re-read source rows.
#pragma once

#include "ndc_dw4_common.cuh"

namespace ndc {
namespace dw4 {

struct KsrcParams {
    const void* z; const float* h; const float* bias;
    void* t1;
    int C, D, H, W;
    Tiling t;
    int relu;
};

template <int KD, int KH, int KW>
struct KsrcSmem {
    static constexpr int PD = KD / 2, PH = KH / 2;
    static constexpr int NTK = (KD * KW + 1) / 2 * 2;  // taps per (kh, channel pair), even
    static constexpr int NSB = 2;                      // source buffers
    int wK, sbuf, total_floats, RS, plane_s, pitch2;
    __host__ __device__ KsrcSmem(const Tiling& t) {
        RS = t.TH + 2 * PH;
        pitch2 = 2 * t.pitch;
        plane_s = 2 * RS * pitch2;                     // two channel pairs
        int o = 0;
        wK = o; o += KH * 2 * NTK * 2;                 // [kh][pair][kd*KW + kw] -> (h[2c], h[2c+1])
        o = (o + 3) / 4 * 4;
        sbuf = o; o += NSB * plane_s;
        total_floats = o;
    }
};

// Place of 16-byte chunk `c` (two pairs) in a row of pairs read by 8-voxel strips: neighbouring
// lanes are 4 chunks apart, so bits 3-4 of the chunk index are folded into bits 0-1 and the eight
// lanes of a quarter-warp hit eight different 16-byte bank groups.
__device__ __forceinline__ int swz_strip8(int chunk) { return chunk ^ ((chunk >> 3) & 3); }

template <typename T, int KD, int KH, int KW, int NT, int MAXZP, int MINB, bool VEC, int WQ>
__global__ void __launch_bounds__(NT, MINB) ksrc_kernel(const KsrcParams P) {
    constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2, KT = KD * KH * KW;
    using L = KsrcSmem<KD, KH, KW>;
    constexpr int NTK = L::NTK, NSB = L::NSB;
    static_assert(KD > 1 && PW == 1, "ksrc_kernel: marching kernels, 3 columns");
    extern __shared__ __align__(16) float smem[];
    const L lay(P.t);
    const int tid = threadIdx.x;
    const int NQ = WQ ? WQ : P.t.NQ, NS8 = (NQ + 1) / 2,
              pitch2 = 2 * (WQ ? row_pitch(4 * WQ) : P.t.pitch),
              W = WQ ? 4 * WQ : P.W, D = P.D;   // WQ > 0: the width is a compile-time constant
    const long long HW = (long long)P.H * W, SP = HW * D;

    int blk = blockIdx.x;
    const int th = blk % P.t.nth; blk /= P.t.nth;
    const int dch = blk % P.t.ndc; blk /= P.t.ndc;
    const int bc = blk;
    const int c = bc % P.C;
    const int h0 = th * P.t.TH, H = P.H;
    const int TH = min(P.t.TH, H - h0);
    const int d0 = dch * P.t.DC, d1 = min(D, d0 + P.t.DC);
    const int RS = lay.RS;

    const T* zg = reinterpret_cast<const T*>(P.z) + (long long)bc * SCH * SP;
    T* tg = reinterpret_cast<T*>(P.t1) + (long long)bc * SP;
    float* wK = smem + lay.wK;
    float* sbuf = smem + lay.sbuf;

    for (int i = tid; i < NSB * lay.plane_s / 4; i += NT)
        reinterpret_cast<float4*>(sbuf)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    {
        const float* hc = P.h + (long long)c * SCH * KT;
        for (int i = tid; i < KH * 2 * NTK; i += NT) {       // wK[kh][pair][kd*KW + kw]
            const int e = i % NTK, cp = (i / NTK) % 2, kh = i / (2 * NTK);
            float a = 0.0f, b = 0.0f;
            if (e < KD * KW) {
                const int tap = ((e / KW) * KH + kh) * KW + e % KW;
                a = hc[(2 * cp) * KT + tap];
                b = hc[(2 * cp + 1) * KT + tap];
            }
            wK[2 * i] = a; wK[2 * i + 1] = b;
        }
    }
    float bj[SCH];
#pragma unroll
    for (int j = 0; j < SCH; ++j) bj[j] = P.bias ? P.bias[c * SCH + j] : 0.0f;

    // this thread's chunks of a source plane (fixed for the CTA's lifetime): 4 voxels of BOTH
    // channels of a pair.  Element offset of the first channel in the plane (-1: nothing to
    // load), float offsets of the two destination chunks, valid count, the two biases.
    const int nzp = 2 * RS * NQ;
    int zg_off[MAXZP], zs0[MAXZP], zs1[MAXZP], zn[MAXZP];
    float zb0[MAXZP], zb1[MAXZP];
#pragma unroll
    for (int i = 0; i < MAXZP; ++i) {
        const int id = tid + i * NT;
        zg_off[i] = -1; zs0[i] = 0; zs1[i] = 0; zn[i] = 0; zb0[i] = 0.0f; zb1[i] = 0.0f;
        if (id < nzp) {
            const int c4 = id % NQ, t = id / NQ, r = t % RS, cp = t / RS;
            const int h = h0 - PH + r, w = 4 * c4;
            if (h >= 0 && h < H) zg_off[i] = (int)(2 * cp * SP + (long long)h * W) + w;
            // shared pair column = w + 4: chunks 2*c4 + 2 and 2*c4 + 3 of the row
            const int row = (cp * RS + r) * pitch2;
            zs0[i] = row + (swz_strip8(2 * c4 + 2) << 2);
            zs1[i] = row + (swz_strip8(2 * c4 + 3) << 2);
            zn[i] = min(4, W - w);
            zb0[i] = cp ? bj[2] : bj[0];
            zb1[i] = cp ? bj[3] : bj[1];
        }
    }

    // this thread's strip (8 voxels of one row of the band) and channel pair.  lane = pair*16 +
    // strip lane: a quarter-warp reads 8 consecutive strips of one pair.
    const int cpair = (tid >> 4) & 1;
    const int k_slot = (tid >> 5) * 16 + (tid & 15);
    const int n_kitems = TH * NS8;
    const bool k_ok = k_slot < n_kitems;
    const int k_row = k_ok ? k_slot / NS8 : 0, k_strip = k_ok ? k_slot % NS8 : 0;
    int kq[6];                           // window chunks 4*strip+1 .. +6: voxels w0-2 .. w0+9
#pragma unroll
    for (int q = 0; q < 6; ++q) kq[q] = swz_strip8(4 * k_strip + 1 + q) << 2;
    f32x2 kacc[KD][VK];
#pragma unroll
    for (int a = 0; a < KD; ++a)
#pragma unroll
        for (int v = 0; v < VK; ++v) kacc[a][v] = pack2(0.0f, 0.0f);
    __syncthreads();

    auto rectify = [&](float4 v, float b, int n) {
        v.x += b; v.y += b; v.z += b; v.w += b;
        if (P.relu) {
            v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f);
            v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
        }
        if (!VEC && n < 4) {  // elements past the end of the row stay zero
            if (n < 2) v.y = 0.f;
            if (n < 3) v.z = 0.f;
            v.w = 0.f;
        }
        return v;
    };
    auto fetch_z = [&](Raw4<T> (&reg)[MAXZP][2], int plane) {
        const T* src = zg + (long long)plane * HW;
#pragma unroll
        for (int i = 0; i < MAXZP; ++i)
            if (zg_off[i] >= 0) {
                reg[i][0] = load4_raw<T, VEC>(src + zg_off[i], zn[i]);
                reg[i][1] = load4_raw<T, VEC>(src + zg_off[i] + SP, zn[i]);
            }
    };
    auto stage_z = [&](const Raw4<T> (&reg)[MAXZP][2], int plane) {
        float* dst = sbuf + (plane & (NSB - 1)) * lay.plane_s;
#pragma unroll
        for (int i = 0; i < MAXZP; ++i)
            if (zg_off[i] >= 0) {
                const float4 a = rectify(to_float4(reg[i][0]), zb0[i], zn[i]);
                const float4 b = rectify(to_float4(reg[i][1]), zb1[i], zn[i]);
                *reinterpret_cast<float4*>(dst + zs0[i]) = make_float4(a.x, b.x, a.y, b.y);
                *reinterpret_cast<float4*>(dst + zs1[i]) = make_float4(a.z, b.z, a.w, b.w);
            }
    };

    const int p_first = d0 - PD, p_last = d1 - 1 + PD;
    if (p_first >= 0 && p_first < D) {
        Raw4<T> reg[MAXZP][2];
        fetch_z(reg, p_first);
        stage_z(reg, p_first);
    }
    __syncthreads();

    for (int p = p_first; p <= p_last; ++p) {
        Raw4<T> zr[MAXZP][2];
        const bool have_z = p + 1 <= p_last && p + 1 >= 0 && p + 1 < D;
        if (have_z) fetch_z(zr, p + 1);

        // source plane p feeds output planes p+PD-kd (slot kd); plane p-PD completes
        if (k_ok && p >= 0 && p < D) {
            const float* sp = sbuf + (p & (NSB - 1)) * lay.plane_s + (cpair * RS + k_row) * pitch2;
#pragma unroll
            for (int kh = 0; kh < KH; ++kh) {
                f32x2 sv[12], w[NTK];
#pragma unroll
                for (int q = 0; q < 6; ++q) {
                    const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(sp + kh * pitch2 + kq[q]);
                    sv[2 * q] = t.x; sv[2 * q + 1] = t.y;
                }
#pragma unroll
                for (int q = 0; q < NTK / 2; ++q) {
                    const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(
                        wK + 2 * ((kh * 2 + cpair) * NTK + 2 * q));
                    w[2 * q] = t.x; w[2 * q + 1] = t.y;
                }
#pragma unroll
                for (int kd = 0; kd < KD; ++kd)
#pragma unroll
                    for (int kw = 0; kw < KW; ++kw)
#pragma unroll
                        for (int v = 0; v < VK; ++v)
                            fma2(kacc[kd][v], sv[v + kw - PW + 2], w[kd * KW + kw]);
            }
        }
        const int qdone = p - PD;
        if (qdone >= d0 && qdone < d1) {
            // both channels of the pair, then the two pairs (one shuffle); each lane then owns
            // one quad of the strip
            float tv[VA];
#pragma unroll
            for (int i = 0; i < VA; ++i) {
                float a0, a1, b0, b1;
                unpack2(kacc[KD - 1][i], a0, a1);
                unpack2(kacc[KD - 1][VA + i], b0, b1);
                const float lo = a0 + a1, up = b0 + b1;
                const float send = cpair ? lo : up, keep = cpair ? up : lo;
                tv[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
            }
            if (k_ok)
                store_strip_global<T, VEC, VA>(tg + (long long)qdone * HW + (long long)(h0 + k_row) * W,
                                               VK * k_strip + VA * cpair, W, tv);
        }
        // rotate the running sums: slot kd now stands for plane (p+1)+PD-kd
#pragma unroll
        for (int kd = KD - 1; kd > 0; --kd)
#pragma unroll
            for (int v = 0; v < VK; ++v) kacc[kd][v] = kacc[kd - 1][v];
#pragma unroll
        for (int v = 0; v < VK; ++v) kacc[0][v] = pack2(0.0f, 0.0f);

        if (have_z) stage_z(zr, p + 1);
        __syncthreads();
    }
}

}  // namespace dw4
}  // namespace ndc
