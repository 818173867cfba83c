// Backward of the update for the depthwise ratio-4 geometry (m = 1, sc = 4), four kernels:
//
//   ratio_kernel    per voxel: n = A(x)+eps, d = A(t1)+eps recomputed from shared-memory rings,
//                   gnum = g*s/d, gden = -(gnum*n)/d (float32 scratch), the direct term
//                   (g*n)/d (into the gz buffer)
//   kconv_kernel    K applied to a 4-channel float32 tensor with running sums along depth:
//                   gt1 = K(gden) (scratch) and gx = K(gnum); the windows it loads for that
//                   also feed two of the three filter-gradient correlations,
//                   sum_q t1[q] gden[j, q+tau-pad]  and  sum_q x[q] gnum[j, q+tau-pad]
//   gz_kernel       gz = [z+b>0] * (direct + A(gt1)) in place, gb = sum gz, and the third
//                   correlation  sum_p s[j,p] gt1[p+pad-tau]
//   reduce_kernel   fixed-order sum of the per-CTA partial filter/bias gradients
//
// The correlations are accumulated in 27*4 (or 25*4, 9*4) registers per thread over all the
// strips a thread visits, then combined per CTA in a fixed order: no atomics anywhere, so the
// gradients are bitwise reproducible.
#pragma once

#include <type_traits>

#include "ndc_dw4_common.cuh"

namespace ndc {
namespace dw4 {

constexpr int kPartialStride = 128;  // floats per CTA partial record (taps*4 + 4 bias sums, padded)

// ------------------------------------------------------------------------------------------
// Rings of single-channel planes, shifted layout, read by 4-voxel strips.
template <int KD, int KH, int KW>
struct RingSmem {
    static constexpr int PD = KD / 2, PH = KH / 2;
    static constexpr int RING = KD > 1 ? KD + 1 : 1;
    int wA, ring0, desc, total_floats, RT, plane_t;
    __host__ __device__ RingSmem(const Tiling& t, int ntensors, int red_floats) {
        RT = t.TH + 2 * PH;
        plane_t = RT * t.pitch;
        int o = 0;
        wA = o; o += KD * KH * KW * SCH;
        o = (o + 3) / 4 * 4;
        ring0 = o; o += ntensors * RING * plane_t;
        desc = o; o += KD > 1 ? 2 * (RT * t.NQ) : 0;
        // the end-of-kernel reduction reuses the ring area and needs red_floats of it
        if (o - ring0 < red_floats) o = ring0 + red_floats;
        total_floats = (o + 3) / 4 * 4;
    }
};

struct RatioParams {
    const void* x; const void* t1; const void* z; const void* gout;
    const float* h; const float* bias;
    float* gnum; float* gden;   // float32 scratch, source-sized
    void* gz;                   // direct term goes here (storage dtype), or NULL
    int C, D, H, W;
    Tiling t;
    float eps;
    int relu;
};

// Deterministic per-CTA combine of per-thread accumulators: every thread writes its NACC values
// to a padded row of shared memory, then thread k sums column k over the threads in order.
template <int NACC, int NT>
__device__ __forceinline__ void cta_combine(float* scratch, const float (&acc)[NACC], float* out) {
    constexpr int LD = NACC + 1;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NACC; ++k) scratch[threadIdx.x * LD + k] = acc[k];
    __syncthreads();
    for (int k = threadIdx.x; k < NACC; k += NT) {
        float s = 0.0f;
        for (int i = 0; i < NT; ++i) s += scratch[i * LD + k];
        out[k] = s;
    }
}

// MODE says what the per-voxel epilogue after the two adjoint sweeps produces:
//   kRatioPlanar   backward: gnum, gden as two planar float32 scratch tensors, direct term
//   kRatioPairs    backward: ONE scratch tensor of (gden, gnum) pairs per voxel at P.gnum (the
//                  layout the packed K kernel reads), direct term
//   kRatioForward  forward:  out = (s * n) / d into P.gz (storage type); P.gout is not read.
//                  This is the second half of the two-launch forward (t1 = K(s) comes from
//                  ksrc_kernel), used where it is faster than the fused fwd_kernel.
enum RatioMode { kRatioPlanar = 0, kRatioPairs = 1, kRatioForward = 2 };

template <typename T, int KD, int KH, int KW, int NT, int MAXX, bool VEC, int WQ, int MODE = kRatioPlanar>
__global__ void __launch_bounds__(NT, 512 / NT) ratio_kernel(const RatioParams P) {
    constexpr bool PAIRS = MODE == kRatioPairs, FWD = MODE == kRatioForward;
    constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2, KT = KD * KH * KW;
    using L = RingSmem<KD, KH, KW>;
    constexpr int RING = L::RING;
    constexpr int NQA = 1 + (2 * PW + 3) / 4;
    extern __shared__ __align__(16) float smem[];
    const L lay(P.t, 2, 0);
    const int tid = threadIdx.x;
    constexpr bool ROWS = KD > 1 && KH == 1;   // images of a batch as the rows of one volume
    const int NQ = WQ ? WQ : P.t.NQ, pitch = WQ ? row_pitch(4 * WQ) : P.t.pitch,
              W = WQ ? 4 * WQ : P.W, D = P.D;   // WQ > 0: the width is a compile-time constant
    const SlabAddr<ROWS> addr(P.C, D, P.H, W);
    const long long HW = addr.plane, SP = addr.chan;
    const long long RWX = ROWS ? addr.row_x : W, RWZ = ROWS ? addr.row_z : W;

    int blk = blockIdx.x;
    const int th = blk % P.t.nth; blk /= P.t.nth;
    const int dch = blk % P.t.ndc; blk /= P.t.ndc;
    const int bc = blk;
    const int c = bc % P.C;
    const int h_band = th * P.t.TH;
    const int TH = min(P.t.TH, P.H - h_band);
    const int d0 = dch * P.t.DC, d1 = min(D, d0 + P.t.DC);
    const int RT = lay.RT;
    // rows mode: the band is folded into the base pointers and rows are counted from it
    const int h0 = ROWS ? 0 : h_band, H = ROWS ? P.H - h_band : P.H;
    const long long bx = (long long)bc * SP + (ROWS ? h_band * RWX : 0);
    const long long bz = (long long)bc * SCH * SP + (ROWS ? h_band * RWZ : 0);

    const T* xg = reinterpret_cast<const T*>(P.x) + bx;
    const T* tg = reinterpret_cast<const T*>(P.t1) + bx;
    const T* zg = reinterpret_cast<const T*>(P.z) + bz;
    const T* gg = FWD ? nullptr : reinterpret_cast<const T*>(P.gout) + bz;
    float* gng = FWD ? nullptr : P.gnum + (PAIRS ? 2 * bz : bz);
    float* gdg = (PAIRS || FWD) ? nullptr : P.gden + bz;
    T* dirg = P.gz ? reinterpret_cast<T*>(P.gz) + bz : nullptr;

    float* wA = smem + lay.wA;
    float* xring = smem + lay.ring0;
    float* tring = xring + RING * lay.plane_t;
    ChunkDesc* desc = reinterpret_cast<ChunkDesc*>(smem + lay.desc);

    for (int i = tid; i < 2 * RING * lay.plane_t; i += NT) xring[i] = 0.0f;
    {
        const float* hc = P.h + (long long)c * SCH * KT;
        for (int i = tid; i < KT * SCH; i += NT) wA[i] = hc[(i % SCH) * KT + i / SCH];  // [tau][j]
    }
    const int nx = RT * NQ;
    if (KD > 1) build_descs(desc, 1, RT, NQ, pitch, h0 - PH, H, W, SP, RWX, NT);
    float bj[SCH];
#pragma unroll
    for (int j = 0; j < SCH; ++j) bj[j] = P.bias ? P.bias[c * SCH + j] : 0.0f;
    __syncthreads();

    const int qbase = d0 - PD - 1;
    auto slot_of = [&](int q) { return (q - qbase) % RING; };
    auto load_now = [&](const T* src_t, float* ring, int plane) {
        const T* src = src_t + (long long)plane * HW;
        float* dst = ring + slot_of(plane) * lay.plane_t;
        for (int id = tid; id < nx; id += NT) {
            const int c4 = id % NQ, r = id / NQ;
            const int h = h0 - PH + r, w = 4 * c4, n = min(4, W - w);
            if (h < 0 || h >= H) continue;
            stage_chunk<PW, false>(dst, (r * pitch) | (w << 16) | (n << 26),
                                   load4<T, VEC>(src + h * RWX + w, n));
        }
    };
    // prologue: planes d0-PD .. d0+PD
    for (int q = d0 - PD; q <= d0 + PD; ++q)
        if (q >= 0 && q < D) { load_now(xg, xring, q); load_now(tg, tring, q); }
    __syncthreads();

    const int items = TH * NQ;
    for (int d = d0; d < d1; ++d) {
        // prefetch the plane the next step needs
        Raw4<T> xr[MAXX], tr[MAXX];
        const int qn = d + PD + 1;
        const bool have = KD > 1 && d + 1 < d1 && qn < D;
        if (have) {
#pragma unroll
            for (int i = 0; i < MAXX; ++i) {
                const int id = tid + i * NT;
                if (id < nx) {
                    const ChunkDesc dsc = desc[id];
                    if (dsc.goff >= 0) {
                        xr[i] = load4_raw<T, VEC>(xg + (long long)qn * HW + dsc.goff, desc_n(dsc.soff));
                        tr[i] = load4_raw<T, VEC>(tg + (long long)qn * HW + dsc.goff, desc_n(dsc.soff));
                    }
                }
            }
        }
#pragma unroll 1
        for (int item = tid; item < items; item += NT) {
            const int a_row = item / NQ, a_q = item % NQ;
            const int hrow = h0 + a_row, w0 = VA * a_q;
            const long long off = (long long)d * HW + hrow * RWZ;
            // global strips first: their latency hides behind the tap sweep
            Raw4<T> zraw[SCH], graw[FWD ? 1 : SCH];   // converted in the epilogue
#pragma unroll
            for (int j = 0; j < SCH; ++j) {
                zraw[j] = load_strip_raw<T, VEC>(zg + j * SP + off, w0, W);
                if (!FWD) graw[FWD ? 0 : j] = load_strip_raw<T, VEC>(gg + j * SP + off, w0, W);
            }
            // accumulators hold channel pairs (2jp, 2jp+1) of one voxel
            f32x2 an2[SCH / 2][VA], ad2[SCH / 2][VA];
            {
                const f32x2 e2 = pack2(P.eps, P.eps);
#pragma unroll
                for (int jp = 0; jp < SCH / 2; ++jp)
#pragma unroll
                    for (int v = 0; v < VA; ++v) { an2[jp][v] = e2; ad2[jp][v] = e2; }
            }
#pragma unroll 1
            for (int kd = 0; kd < KD; ++kd) {
                const int q = d + PD - kd;
                if (q < 0 || q >= D) continue;
                const int slot = slot_of(q);
#pragma unroll
                for (int kh = 0; kh < KH; ++kh) {
                    const int rr = a_row + PH + PH - kh;
                    adjoint_row2<KW, NQA>(xring + slot * lay.plane_t + rr * pitch,
                                          tring + slot * lay.plane_t + rr * pitch, a_q + 1,
                                          wA + (kd * KH + kh) * KW * SCH, an2, ad2);
                }
            }
            // epilogue: gnum, gden, direct term
#pragma unroll
            for (int j = 0; j < SCH; ++j) {
                float dv[VA], zj[VA], gj[VA], gnv[VA], gdv[VA];
                raw_to_array(zraw[j], zj);
                if (FWD) {
#pragma unroll
                    for (int v = 0; v < VA; ++v) {
                        float s = zj[v] + bj[j];
                        if (P.relu) s = fmaxf(s, 0.0f);
                        dv[v] = fast_div(s * lane_of(an2[j / 2][v], j & 1), lane_of(ad2[j / 2][v], j & 1));
                    }
                    store_strip_global<T, VEC, VA>(dirg + j * SP + off, w0, W, dv);
                    continue;
                }
                raw_to_array(graw[FWD ? 0 : j], gj);
#pragma unroll
                for (int v = 0; v < VA; ++v) {
                    float s = zj[v] + bj[j];
                    if (P.relu) s = fmaxf(s, 0.0f);
                    const float n = lane_of(an2[j / 2][v], j & 1);
                    const float r = fast_div(1.0f, lane_of(ad2[j / 2][v], j & 1));
                    const float gr = gj[v] * r;
                    const float gn = gr * s;
                    dv[v] = gr * n;
                    gdv[v] = -(gn * n) * r;
                    gnv[v] = gn;
                    if (w0 + v >= W) { gnv[v] = 0.0f; gdv[v] = 0.0f; }
                }
                if (PAIRS) {
                    float* dst = gng + 2 * (j * SP + off + w0);
                    if (VEC) {
                        reinterpret_cast<float4*>(dst)[0] = make_float4(gdv[0], gnv[0], gdv[1], gnv[1]);
                        reinterpret_cast<float4*>(dst)[1] = make_float4(gdv[2], gnv[2], gdv[3], gnv[3]);
                    } else {
#pragma unroll
                        for (int v = 0; v < VA; ++v)
                            if (w0 + v < W) { dst[2 * v] = gdv[v]; dst[2 * v + 1] = gnv[v]; }
                    }
                } else {
                    store_strip_global<float, VEC, VA>(gng + j * SP + off, w0, W, gnv);
                    store_strip_global<float, VEC, VA>(gdg + j * SP + off, w0, W, gdv);
                }
                if (dirg) store_strip_global<T, VEC, VA>(dirg + j * SP + off, w0, W, dv);
            }
        }
        if (have) {
#pragma unroll
            for (int i = 0; i < MAXX; ++i) {
                const int id = tid + i * NT;
                if (id < nx) {
                    const ChunkDesc dsc = desc[id];
                    if (dsc.goff >= 0) {
                        stage_chunk<PW, false>(xring + slot_of(qn) * lay.plane_t, dsc.soff, to_float4(xr[i]));
                        stage_chunk<PW, false>(tring + slot_of(qn) * lay.plane_t, dsc.soff, to_float4(tr[i]));
                    }
                }
            }
        }
        __syncthreads();
    }
}

// ------------------------------------------------------------------------------------------
// K applied to a 4-channel float32 tensor (gnum or gden) with running sums along depth.
struct KconvParams {
    const float* in[2];     // gridDim.y selects: [0] gden -> gt1 (float32), [1] gnum -> gx (T)
    void* out[2];
    int out_is_f32[2];
    const void* aux[2];     // single-channel tensor correlated with in[]: t1 for gden, x for gnum
    float* partial[2];      // [cta][kPartialStride] records of the correlations, or NULL
    const float* h;
    int C, D, H, W;
    Tiling t;
};

template <int KD, int KH, int KW>
struct KconvSmem {
    static constexpr int PD = KD / 2, PH = KH / 2;
    static constexpr int WKP = (KD * KW + 3) / 4 * 4;
    static constexpr int NSB = KD > 1 ? 3 : 1;   // planes p, p+1 (landed) and p+2 (in flight)
    int wK, sbuf, desc, total_floats, RS, plane_s;
    __host__ __device__ KconvSmem(const Tiling& t) {
        RS = t.TH + 2 * PH;
        plane_s = SCH * RS * t.pitch;
        int o = 0;
        wK = o; o += KH * SCH * WKP;
        o = (o + 3) / 4 * 4;
        sbuf = o; o += NSB * plane_s;
        desc = o; o += 2 * (SCH * RS * t.NQ);
        total_floats = o;
    }
    // with the correlations: room for the end-of-kernel combine (nthreads/4 rows of taps*4+1)
    __host__ __device__ KconvSmem(const Tiling& t, int nthreads) : KconvSmem(t) {
        const int red = (nthreads / SCH) * (KD * KH * KW * SCH + 1);
        if (total_floats - sbuf < red) total_floats = sbuf + red;
    }
};

// Thread layout: a warp covers 8 strips x 4 input channels (lane = channel*8 + strip lane), so a
// thread convolves ONE channel: its running sums are partial and are added across the four
// channel lanes when a plane completes, and its correlation accumulators are the taps of its
// own channel only (27 instead of 108 registers).
//
// Source planes are float32 already, so they go from HBM to shared memory with cp.async
// (no registers, no staging pass): rows are UNshifted here (shared column c holds w = c - 4),
// 16-byte chunks land on 16-byte quads, and an 8-voxel strip reads a 4-quad window.
// The KD running sums and their aux strips never move between registers: plane q lives in
// slot q mod KD, and the step body exists in KD rotated copies.
template <typename T, int KD, int KH, int KW, int NT, bool VEC, bool WGRAD, int WQ>
__global__ void __launch_bounds__(NT, 384 / NT) kconv_kernel(const KconvParams P) {
    constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2;
    using L = KconvSmem<KD, KH, KW>;
    constexpr int WKP = L::WKP, NSB = L::NSB, KT = KD * KH * KW;
    constexpr int NG = NT / SCH;                 // strip slots per CTA
    constexpr int NW = WGRAD ? KT : 1;           // correlation accumulators per thread
    extern __shared__ __align__(16) float smem[];
    const L lay(P.t);
    const int tid = threadIdx.x;
    constexpr bool ROWS = KD > 1 && KH == 1;   // images of a batch as the rows of one volume
    const int NQ = WQ ? WQ : P.t.NQ, NS8 = (NQ + 1) / 2, pitch = WQ ? row_pitch(4 * WQ) : P.t.pitch,
              W = WQ ? 4 * WQ : P.W, D = P.D;   // WQ > 0: the width is a compile-time constant
    const SlabAddr<ROWS> addr(P.C, D, P.H, W);
    const long long HW = addr.plane, SP = addr.chan;
    const long long RWX = ROWS ? addr.row_x : W, RWZ = ROWS ? addr.row_z : W;
    const int which = blockIdx.y;

    int blk = blockIdx.x;
    const int th = blk % P.t.nth; blk /= P.t.nth;
    const int dch = blk % P.t.ndc; blk /= P.t.ndc;
    const int bc = blk;
    const int c = bc % P.C;
    const int h_band = th * P.t.TH;
    const int TH = min(P.t.TH, P.H - h_band);
    const int d0 = dch * P.t.DC, d1 = min(D, d0 + P.t.DC);
    const int RS = lay.RS;
    // rows mode: the band is folded into the base pointers and rows are counted from it
    const int h0 = ROWS ? 0 : h_band, H = ROWS ? P.H - h_band : P.H;
    const long long bx = (long long)bc * SP + (ROWS ? h_band * RWX : 0);
    const long long bz = (long long)bc * SCH * SP + (ROWS ? h_band * RWZ : 0);

    const float* ing = P.in[which] + bz;
    float* outf = P.out_is_f32[which] ? reinterpret_cast<float*>(P.out[which]) + bx : nullptr;
    T* outt = P.out_is_f32[which] ? nullptr : reinterpret_cast<T*>(P.out[which]) + bx;
    const T* auxg = WGRAD ? reinterpret_cast<const T*>(P.aux[which]) + bx : nullptr;

    float* wK = smem + lay.wK;
    float* sbuf = smem + lay.sbuf;
    ChunkDesc* desc = reinterpret_cast<ChunkDesc*>(smem + lay.desc);
    for (int i = tid; i < NSB * lay.plane_s; i += NT) sbuf[i] = 0.0f;
    {
        const float* hc = P.h + (long long)c * SCH * KT;
        for (int i = tid; i < KH * SCH * WKP; i += NT) {   // wK[kh][j][kd*KW + kw]
            const int e = i % WKP, j = (i / WKP) % SCH, kh = i / (WKP * SCH);
            float v = 0.0f;
            if (e < KD * KW) v = hc[j * KT + ((e / KW) * KH + kh) * KW + e % KW];
            wK[i] = v;
        }
    }
    // loader table: .goff = element offset in the plane (-1: row outside the volume),
    // .soff = float offset of the destination quad in a plane buffer | (valid elements << 26)
    const int nz = SCH * RS * NQ;
    for (int id = tid; id < nz; id += NT) {
        const int c4 = id % NQ, t = id / NQ, r = t % RS, ch = t / RS;
        const int h = h0 - PH + r, w = 4 * c4, n = min(4, W - w);
        ChunkDesc dsc;
        dsc.goff = (h < 0 || h >= H) ? -1 : (int)(ch * SP + h * RWZ) + w;
        dsc.soff = ((ch * RS + r) * pitch + (phys_quad<true>(c4 + 1) << 2)) | (n << 26);
        desc[id] = dsc;
    }
    const int lane = tid & 31;
    const int jch = (lane >> 3) & 3;                       // this thread's input channel
    const int slot = (tid >> 5) * 8 + (lane & 7);          // strip slot inside the CTA
    const int n_items = TH * NS8;
    float accw[NW];
#pragma unroll
    for (int k = 0; k < NW; ++k) accw[k] = 0.0f;
    __syncthreads();

    const int p_first = d0 - PD, p_last = d1 - 1 + PD;
    // plane -> shared buffer: asynchronous 16-byte copies where rows allow, else through registers
    auto copy_plane = [&](int plane) {
        const float* src = ing + (long long)plane * HW;
        float* dst = sbuf + ((plane - p_first) % NSB) * lay.plane_s;
        for (int id = tid; id < nz; id += NT) {
            const ChunkDesc dsc = desc[id];
            if (dsc.goff < 0) continue;
            float* q = dst + (dsc.soff & 0x3ffffff);
            if (VEC) {
                const unsigned sa = (unsigned)__cvta_generic_to_shared(q);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(src + dsc.goff) : "memory");
            } else {
                *reinterpret_cast<float4*>(q) = load4<float, false>(src + dsc.goff, (dsc.soff >> 26) & 7);
            }
        }
        if (VEC) cp_async_commit();
    };
    auto wait_but_newest = [&]() { if (VEC) asm volatile("cp.async.wait_group 1;\n" ::: "memory"); };
    // one source row of this thread's channel feeds KD output planes (and their correlations);
    // output plane p+PD-kd lives in slot (R + PD - kd) mod KD, R = rotation of this step
    auto accumulate = [&](auto rot, int p, int row, int strip, float (&acc)[KD][VK],
                          const float (&aux)[WGRAD ? KD : 1][VK]) {
        constexpr int R = decltype(rot)::value;
        const float* sp = sbuf + ((p - p_first) % NSB) * lay.plane_s + (jch * RS + row) * pitch;
        int qo[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) qo[q] = phys_quad<true>(2 * strip + q) << 2;
#pragma unroll
        for (int kh = 0; kh < KH; ++kh) {
            float sv[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 t = *reinterpret_cast<const float4*>(sp + kh * pitch + qo[q]);
                sv[4 * q] = t.x; sv[4 * q + 1] = t.y; sv[4 * q + 2] = t.z; sv[4 * q + 3] = t.w;
            }
            float w[WKP];
#pragma unroll
            for (int q4 = 0; q4 < WKP / 4; ++q4) {
                const float4 t = *reinterpret_cast<const float4*>(wK + (kh * SCH + jch) * WKP + 4 * q4);
                w[4 * q4] = t.x; w[4 * q4 + 1] = t.y; w[4 * q4 + 2] = t.z; w[4 * q4 + 3] = t.w;
            }
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) {
                constexpr int dummy = 0; (void)dummy;
                const int sl = (R + PD - kd + 2 * KD) % KD;
#pragma unroll
                for (int kw = 0; kw < KW; ++kw) {
                    float a = WGRAD ? accw[WGRAD ? (kd * KH + kh) * KW + kw : 0] : 0.0f;
#pragma unroll
                    for (int v = 0; v < VK; ++v) {
                        acc[sl][v] = fmaf(sv[4 - PW + v + kw], w[kd * KW + kw], acc[sl][v]);
                        if (WGRAD) a = fmaf(aux[WGRAD ? sl : 0][v], sv[4 - PW + v + kw], a);
                    }
                    if (WGRAD) accw[WGRAD ? (kd * KH + kh) * KW + kw : 0] = a;
                }
            }
        }
    };
    // add the four channel lanes' partial sums; every lane ends up owning two voxels of the strip
    auto finish = [&](int q, int row, int strip, const float (&part)[VK]) {
        float h4[4];
        const bool hi = jch & 2;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float send = hi ? part[i] : part[4 + i];
            const float keep = hi ? part[4 + i] : part[i];
            h4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
        const bool odd = jch & 1;
        float o2[2];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const float send = odd ? h4[i] : h4[2 + i];
            const float keep = odd ? h4[2 + i] : h4[i];
            o2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
        if (row >= 0) {
            const int w0 = VK * strip + (hi ? 4 : 0) + (odd ? 2 : 0);
            const long long off = (long long)q * HW + (h0 + row) * RWX + w0;
            if (VEC) {
                if (w0 < W) {
                    if (outf) *reinterpret_cast<float2*>(outf + off) = make_float2(o2[0], o2[1]);
                    else if (sizeof(T) == 4) *reinterpret_cast<float2*>(outt + off) = make_float2(o2[0], o2[1]);
                    else *reinterpret_cast<__nv_bfloat162*>(outt + off) = __floats2bfloat162_rn(o2[0], o2[1]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 2; ++i)
                    if (w0 + i < W) {
                        if (outf) outf[off + i] = o2[i];
                        else outt[off + i] = from_f32<T>(o2[i]);
                    }
            }
        }
    };

    // planes are requested two steps ahead of their use: a step is shorter than the memory
    // latency under load
    auto plane_ok = [&](int q) { return q >= 0 && q < D && q <= p_last; };
    if (plane_ok(p_first)) copy_plane(p_first); else if (VEC) cp_async_commit();
    if (KD > 1) { if (plane_ok(p_first + 1)) copy_plane(p_first + 1); else if (VEC) cp_async_commit(); }
    if (KD > 1) wait_but_newest(); else if (VEC) cp_async_wait_all();
    __syncthreads();

    if (KD > 1) {
        // ---- marching: one strip per thread group, running sums along depth
        const bool k_ok = slot < n_items;
        const int k_row = k_ok ? slot / NS8 : 0, k_strip = k_ok ? slot % NS8 : 0;
        float kacc[KD][VK], auxs[WGRAD ? KD : 1][VK];
#pragma unroll
        for (int a = 0; a < KD; ++a)
#pragma unroll
            for (int v = 0; v < VK; ++v) kacc[a][v] = 0.0f;
        // strip of plane q of the aux tensor, zero outside the chunk; the row/column part of the
        // address is fixed per thread
        const T* aux_row = WGRAD ? auxg + (h0 + k_row) * RWX : nullptr;
        auto aux_raw = [&](int q, Raw4<T> (&dst)[2]) {
            if (k_ok && q >= d0 && q < d1) {
                dst[0] = load_strip_raw<T, VEC>(aux_row + (long long)q * HW, VK * k_strip, W);
                dst[1] = load_strip_raw<T, VEC>(aux_row + (long long)q * HW, VK * k_strip + 4, W);
            } else {
                dst[0].v = {}; dst[1].v = {};
            }
        };
        auto aux_strip = [&](int q, float (&dst)[VK]) {
            Raw4<T> raw[2];
            aux_raw(q, raw);
            const float4 a = to_float4(raw[0]), b = to_float4(raw[1]);
            dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
            dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
        };
        // plane q lives in slot (q - p_first) mod KD: at the first step (rotation 0) output plane
        // p_first + PD - kd is slot (PD - kd) mod KD
        if (WGRAD) {
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) aux_strip(p_first + PD - kd, auxs[WGRAD ? (PD - kd + KD) % KD : 0]);
        }
        Raw4<T> aux_near[2];
        if (WGRAD) aux_raw(p_first + 1 + PD, aux_near); else { aux_near[0].v = {}; aux_near[1].v = {}; }
        auto step = [&](auto rot, int p) {
            constexpr int R = decltype(rot)::value;
            constexpr int DONE = (R - PD + 2 * KD) % KD;     // slot of plane p-PD, reused for p+1+PD
            Raw4<T> aux_far[2];   // aux strip two steps ahead (raw); aux_near is next step's
            if (WGRAD) aux_raw(p + 2 + PD, aux_far);
            if (plane_ok(p + 2)) copy_plane(p + 2); else if (VEC) cp_async_commit();
            const int qdone = p - PD;
            if (k_ok && p >= 0 && p < D) accumulate(rot, p, k_row, k_strip, kacc, auxs);
            if (qdone >= d0 && qdone < d1) finish(qdone, k_ok ? k_row : -1, k_strip, kacc[DONE]);
#pragma unroll
            for (int v = 0; v < VK; ++v) kacc[DONE][v] = 0.0f;
            if (WGRAD) {
                const float4 a = to_float4(aux_near[0]), b = to_float4(aux_near[1]);
                float (&dst)[VK] = auxs[WGRAD ? DONE : 0];
                dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w;
                dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
                aux_near[0] = aux_far[0]; aux_near[1] = aux_far[1];
            }
            wait_but_newest();   // plane p+1 has landed; p+2 may still be in flight
            __syncthreads();
        };
        int p = p_first;
        while (p <= p_last) {
            step(std::integral_constant<int, 0>{}, p++);
            if (p > p_last) break;
            if (KD > 1) step(std::integral_constant<int, 1 % KD>{}, p++);
            if (p > p_last) break;
            if (KD > 2) step(std::integral_constant<int, 2 % KD>{}, p++);
            if (KD > 3) {   // wider depth kernels: remaining rotations
                if (p > p_last) break;
                step(std::integral_constant<int, 3 % KD>{}, p++);
                if (p > p_last) break;
                if (KD > 4) step(std::integral_constant<int, 4 % KD>{}, p++);
            }
        }
    } else {
        // ---- no depth taps: every plane is its own chunk, strips are looped over.  All lanes of
        // a warp run the same number of rounds (the channel lanes exchange partial sums).
        const int p = p_first;
        if (p >= 0 && p < D) {
            const int rounds = (n_items + NG - 1) / NG;
            for (int r = 0; r < rounds; ++r) {
                const int item = slot + r * NG;
                const bool ok = item < n_items;
                const int row = ok ? item / NS8 : 0, strip = ok ? item % NS8 : 0;
                float acc[KD][VK], aux[WGRAD ? KD : 1][VK];
#pragma unroll
                for (int v = 0; v < VK; ++v) { acc[0][v] = 0.0f; aux[0][v] = 0.0f; }
                if (WGRAD && ok)
                    load_strip_global<T, VEC, VK>(auxg + (long long)p * HW + (h0 + row) * RWX,
                                                  VK * strip, W, aux[0]);
                if (ok) accumulate(std::integral_constant<int, 0>{}, p, row, strip, acc, aux);
                finish(p, ok ? row : -1, strip, acc[0]);
            }
        }
    }
    if (WGRAD && P.partial[which]) {
        // per-CTA combine in a fixed order: slot-major scratch rows of taps*4 (+1 pad) floats
        constexpr int LD = KT * SCH + 1;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < NW; ++k) sbuf[slot * LD + k * SCH + jch] = accw[k];
        __syncthreads();
        float* out = P.partial[which] + (long long)blockIdx.x * kPartialStride;
        for (int k = tid; k < KT * SCH; k += NT) {
            float s = 0.0f;
            for (int i = 0; i < NG; ++i) s += sbuf[i * LD + k];
            out[k] = s;
        }
    }
}

// ------------------------------------------------------------------------------------------
// K applied to BOTH scratch tensors at once, packed.  The source is the tensor of (gden, gnum)
// pairs ratio_kernel<PAIRS> writes; every multiply-add is a two-lane `fma.rn.f32x2` whose low
// lane works on gden and whose high lane works on gnum:
//
//     running sums    (gt1, gx)[q]      += (gden, gnum)[j, q + tau - pad] * (h, h)[j, tau]
//     correlations    (cD, cN)[j, tau]  += (t1, x)[q] * (gden, gnum)[j, q + tau - pad]
//
// so the source window is used as loaded (a 64-bit shared-memory element is a ready pair), the
// filter is staged duplicated, and the saved (t1, x) strips are paired once per plane.  Half
// the multiply-add instructions of two separate passes; the filter gradient needs cD + cN.
struct Kconv2Params {
    const float* in;        // (gden, gnum) pairs: [(b*C + c)*4 + j][voxel][2]
    float* gt1;             // K(gden), float32 scratch, or NULL
    void* gx;               // K(gnum), storage type, or NULL
    const void* t1;         // saved t1 and x: the strips the correlations pair with
    const void* x;
    float* partial;         // [cta][kPartialStride] records of cD + cN, or NULL
    const float* h;
    int C, D, H, W;
    Tiling t;
};

template <int KD, int KH, int KW>
struct Kconv2Smem {
    static constexpr int PD = KD / 2, PH = KH / 2;
    static constexpr int KWP = (KW + 1) / 2 * 2;   // taps per (kh, j, kd), padded to an even count
    static constexpr int NSB = KD > 1 ? 3 : 1;     // planes p, p+1 (landed) and p+2 (in flight)
    int wK, sbuf, total_floats, RS, plane_s, pitch2, NC2;
    __host__ __device__ Kconv2Smem(const Tiling& t, int nthreads) {
        RS = t.TH + 2 * PH;
        pitch2 = 2 * t.pitch;                      // a row of pairs
        plane_s = SCH * RS * pitch2;
        NC2 = 2 * t.NQ;                            // 16-byte chunks (two voxels) per row
        int o = 0;
        wK = o; o += KH * SCH * KD * KWP * 2;      // [kh][j][kd][tap] duplicated weights
        o = (o + 3) / 4 * 4;
        sbuf = o; o += NSB * plane_s;
        total_floats = o;
        // room for the end-of-kernel combine (nthreads/4 rows of taps*4 + 1 floats)
        const int red = (nthreads / SCH) * (KD * KH * KW * SCH + 1);
        if (total_floats - sbuf < red) total_floats = sbuf + red;
    }
};

// 16-byte chunk c of a row of pairs -> its place in shared memory.  The eight lanes of a
// quarter-warp read chunks VK/2 apart (strips of VK voxels); folding bits 3.. of the chunk index
// into the low bits sends them to eight different 16-byte bank groups.
template <int VK> __device__ __forceinline__ int swz2(int chunk) {
    return chunk ^ ((chunk >> 3) & (VK == 8 ? 3 : 1));
}

// Threads per SM the packed K kernel is built for, by CTA size and strip length.
template <int NT, int VK> constexpr int kconv2_min_blocks() {
    return VK == 8 ? (NT >= 256 ? 1 : NT >= 128 ? 2 : NT >= 64 ? 4 : 8)
                   : (NT >= 256 ? 1 : NT >= 192 ? 2 : NT >= 128 ? 3 : 4);
}

template <typename T, int KD, int KH, int KW, int NT, int VK, int MAXC, bool VEC, bool WGRAD, int WQ>
__global__ void __launch_bounds__(NT, kconv2_min_blocks<NT, VK>()) kconv2_kernel(const Kconv2Params P) {
    constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2, KT = KD * KH * KW;
    using L = Kconv2Smem<KD, KH, KW>;
    constexpr int KWP = L::KWP, NSB = L::NSB;
    constexpr int NG = NT / SCH;                 // strip slots per CTA
    constexpr int NW = WGRAD ? KT : 1;           // correlation accumulators (pairs) per thread
    constexpr int NWIN = VK + 4;                 // window pairs held: voxels w0-2 .. w0+VK+1
    constexpr int VO = VK / 4;                   // voxels a lane owns after the channel lanes add up
    static_assert(KD > 1 && PW <= 2 && (VK == 4 || VK == 8), "packed K kernel: marching kernels with up to 5 columns");
    extern __shared__ __align__(16) float smem[];
    const L lay(P.t, NT);
    const int tid = threadIdx.x;
    const int NQ = WQ ? WQ : P.t.NQ, pitch2 = 2 * (WQ ? row_pitch(4 * WQ) : P.t.pitch),
              W = WQ ? 4 * WQ : P.W, D = P.D;   // WQ > 0: the width is a compile-time constant
    const int NSV = (4 * NQ + VK - 1) / VK;      // strips per row
    const long long HW = (long long)P.H * W, SP = HW * D;
    const int NC2 = 2 * NQ;

    int blk = blockIdx.x;
    const int th = blk % P.t.nth; blk /= P.t.nth;
    const int dch = blk % P.t.ndc; blk /= P.t.ndc;
    const int bc = blk;
    const int c = bc % P.C;
    const int h0 = th * P.t.TH, H = P.H;
    const int TH = min(P.t.TH, H - h0);
    const int d0 = dch * P.t.DC, d1 = min(D, d0 + P.t.DC);
    const int RS = lay.RS;
    const long long bx = (long long)bc * SP;

    const float* ing = P.in + 2 * (long long)bc * SCH * SP;
    float* gt1g = P.gt1 ? P.gt1 + bx : nullptr;
    T* gxg = P.gx ? reinterpret_cast<T*>(P.gx) + bx : nullptr;
    const T* t1g = reinterpret_cast<const T*>(P.t1) + bx;
    const T* xg = reinterpret_cast<const T*>(P.x) + bx;

    float* wK = smem + lay.wK;
    float* sbuf = smem + lay.sbuf;
    for (int i = tid; i < NSB * lay.plane_s; i += NT) sbuf[i] = 0.0f;
    {
        const float* hc = P.h + (long long)c * SCH * KT;
        for (int i = tid; i < KH * SCH * KD * KWP; i += NT) {   // wK[kh][j][kd][kw] = (w, w)
            const int kw = i % KWP, kd = (i / KWP) % KD, j = (i / (KWP * KD)) % SCH, kh = i / (KWP * KD * SCH);
            const float v = kw < KW ? hc[j * KT + (kd * KH + kh) * KW + kw] : 0.0f;
            wK[2 * i] = v; wK[2 * i + 1] = v;
        }
    }
    // this thread's chunks of a source plane (fixed for the CTA's lifetime): voxel offset in the
    // plane (-1: nothing to load) and float offset of the destination chunk | (valid voxels << 26)
    const int nz = SCH * RS * NC2;
    int cg_off[MAXC], cs_off[MAXC];
#pragma unroll
    for (int i = 0; i < MAXC; ++i) {
        const int id = tid + i * NT;
        cg_off[i] = -1; cs_off[i] = 0;
        if (id < nz) {
            const int c2 = id % NC2, t = id / NC2, r = t % RS, ch = t / RS;
            const int h = h0 - PH + r, w = 2 * c2, n = min(2, W - w);
            if (h >= 0 && h < H && n > 0) cg_off[i] = (int)(ch * SP + (long long)h * W) + w;
            cs_off[i] = ((ch * RS + r) * pitch2 + (swz2<VK>(c2 + 2) << 2)) | (max(n, 0) << 26);
        }
    }
    const int lane = tid & 31;
    const int jch = (lane >> 3) & 3;                       // this thread's source channel
    const int slot = (tid >> 5) * 8 + (lane & 7);          // strip slot inside the CTA
    const int n_items = TH * NSV;
    f32x2 accw[NW];
#pragma unroll
    for (int k = 0; k < NW; ++k) accw[k] = pack2(0.0f, 0.0f);
    __syncthreads();

    const int p_first = d0 - PD, p_last = d1 - 1 + PD;
    auto copy_plane = [&](int plane) {
        const float* src = ing + 2 * (long long)plane * HW;
        float* dst = sbuf + ((plane - p_first) % NSB) * lay.plane_s;
#pragma unroll
        for (int i = 0; i < MAXC; ++i) {
            if (cg_off[i] < 0) continue;
            float* q = dst + (cs_off[i] & 0x3ffffff);
            const float* g = src + 2 * (long long)cg_off[i];
            if (VEC) {
                const unsigned sa = (unsigned)__cvta_generic_to_shared(q);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(g) : "memory");
            } else {
                const bool two = ((cs_off[i] >> 26) & 3) > 1;
                *reinterpret_cast<float4*>(q) =
                    make_float4(__ldg(g), __ldg(g + 1), two ? __ldg(g + 2) : 0.0f, two ? __ldg(g + 3) : 0.0f);
            }
        }
        if (VEC) cp_async_commit();
    };
    auto wait_but_newest = [&]() { if (VEC) asm volatile("cp.async.wait_group 1;\n" ::: "memory"); };

    const bool k_ok = slot < n_items;
    const int k_row = k_ok ? slot / NSV : 0, k_strip = k_ok ? slot % NSV : 0;
    // shared-memory offsets (floats) of the window chunks of this strip: chunks
    // (VK/2)*strip + 1 .. + VK/2 + 2 of a row hold voxels w0-2 .. w0+VK+1
    int qo[NWIN / 2];
#pragma unroll
    for (int q = 0; q < NWIN / 2; ++q) qo[q] = swz2<VK>((VK / 2) * k_strip + 1 + q) << 2;

    f32x2 kacc[KD][VK], auxs[WGRAD ? KD : 1][VK];
#pragma unroll
    for (int a = 0; a < KD; ++a)
#pragma unroll
        for (int v = 0; v < VK; ++v) kacc[a][v] = pack2(0.0f, 0.0f);

    // one source row of this thread's channel feeds KD output planes (and their correlations);
    // output plane p+PD-kd lives in slot (R + PD - kd) mod KD, R = rotation of this step
    auto accumulate = [&](auto rot, int p) {
        constexpr int R = decltype(rot)::value;
        const float* sp = sbuf + ((p - p_first) % NSB) * lay.plane_s + (jch * RS + k_row) * pitch2;
#pragma unroll
        for (int kh = 0; kh < KH; ++kh) {
            f32x2 sv[NWIN];
#pragma unroll
            for (int q = 0; q < NWIN / 2; ++q) {
                const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(sp + kh * pitch2 + qo[q]);
                sv[2 * q] = t.x; sv[2 * q + 1] = t.y;
            }
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) {
                f32x2 w[KWP];
#pragma unroll
                for (int q = 0; q < KWP / 2; ++q) {
                    const ulonglong2 t = *reinterpret_cast<const ulonglong2*>(
                        wK + 2 * (((kh * SCH + jch) * KD + kd) * KWP + 2 * q));
                    w[2 * q] = t.x; w[2 * q + 1] = t.y;
                }
                const int sl = (R + PD - kd + 2 * KD) % KD;
#pragma unroll
                for (int kw = 0; kw < KW; ++kw) {
                    f32x2 a = accw[WGRAD ? (kd * KH + kh) * KW + kw : 0];
#pragma unroll
                    for (int v = 0; v < VK; ++v) {
                        fma2(kacc[sl][v], sv[v + kw - PW + 2], w[kw]);
                        if (WGRAD) fma2(a, auxs[WGRAD ? sl : 0][v], sv[v + kw - PW + 2]);
                    }
                    if (WGRAD) accw[WGRAD ? (kd * KH + kh) * KW + kw : 0] = a;
                }
            }
        }
    };
    // add the four channel lanes' partial sums; every lane ends up owning VO voxels of the strip
    auto finish = [&](int q, bool store, const f32x2 (&part)[VK]) {
        const bool hi = jch & 2, odd = jch & 1;
        f32x2 h2[VK / 2];
#pragma unroll
        for (int i = 0; i < VK / 2; ++i) {
            float s_lo, s_up, k_lo, k_up;
            unpack2(hi ? part[i] : part[VK / 2 + i], s_lo, s_up);
            unpack2(hi ? part[VK / 2 + i] : part[i], k_lo, k_up);
            k_lo += __shfl_xor_sync(0xffffffffu, s_lo, 16);
            k_up += __shfl_xor_sync(0xffffffffu, s_up, 16);
            h2[i] = pack2(k_lo, k_up);
        }
        float o_t[VO], o_x[VO];
#pragma unroll
        for (int i = 0; i < VO; ++i) {
            float s_lo, s_up;
            unpack2(odd ? h2[i] : h2[VO + i], s_lo, s_up);
            unpack2(odd ? h2[VO + i] : h2[i], o_t[i], o_x[i]);
            o_t[i] += __shfl_xor_sync(0xffffffffu, s_lo, 8);
            o_x[i] += __shfl_xor_sync(0xffffffffu, s_up, 8);
        }
        if (store) {
            const int w = VK * k_strip + (hi ? VK / 2 : 0) + (odd ? VO : 0);
            const long long off = (long long)q * HW + (long long)(h0 + k_row) * W + w;
            if (VEC && VO == 2) {
                if (w < W) {
                    if (gt1g) *reinterpret_cast<float2*>(gt1g + off) = make_float2(o_t[0], o_t[VO - 1]);
                    if (gxg) {
                        if (sizeof(T) == 4) *reinterpret_cast<float2*>(gxg + off) = make_float2(o_x[0], o_x[VO - 1]);
                        else *reinterpret_cast<__nv_bfloat162*>(gxg + off) = __floats2bfloat162_rn(o_x[0], o_x[VO - 1]);
                    }
                }
            } else {
#pragma unroll
                for (int i = 0; i < VO; ++i)
                    if (w + i < W) {
                        if (gt1g) gt1g[off + i] = o_t[i];
                        if (gxg) gxg[off + i] = from_f32<T>(o_x[i]);
                    }
            }
        }
    };
    // (t1, x) strips of plane q, raw; zero outside the chunk
    const T* t1_row = t1g + (long long)(h0 + k_row) * W;
    const T* x_row = xg + (long long)(h0 + k_row) * W;
    auto aux_raw = [&](int q, Raw4<T> (&dst)[2 * VO]) {
        if (WGRAD && k_ok && q >= d0 && q < d1) {
#pragma unroll
            for (int i = 0; i < VO; ++i) {
                dst[i] = load_strip_raw<T, VEC>(t1_row + (long long)q * HW, VK * k_strip + 4 * i, W);
                dst[VO + i] = load_strip_raw<T, VEC>(x_row + (long long)q * HW, VK * k_strip + 4 * i, W);
            }
        } else {
#pragma unroll
            for (int i = 0; i < 2 * VO; ++i) dst[i].v = {};
        }
    };
    auto aux_pairs = [&](const Raw4<T> (&raw)[2 * VO], f32x2 (&dst)[VK]) {
#pragma unroll
        for (int i = 0; i < VO; ++i) {
            const float4 a = to_float4(raw[i]), b = to_float4(raw[VO + i]);
            dst[4 * i] = pack2(a.x, b.x); dst[4 * i + 1] = pack2(a.y, b.y);
            dst[4 * i + 2] = pack2(a.z, b.z); dst[4 * i + 3] = pack2(a.w, b.w);
        }
    };

    // planes are requested two steps ahead of their use
    auto plane_ok = [&](int q) { return q >= 0 && q < D && q <= p_last; };
    if (plane_ok(p_first)) copy_plane(p_first); else if (VEC) cp_async_commit();
    if (plane_ok(p_first + 1)) copy_plane(p_first + 1); else if (VEC) cp_async_commit();
    // plane q lives in slot (q - p_first) mod KD: at the first step (rotation 0) output plane
    // p_first + PD - kd is slot (PD - kd) mod KD
    if (WGRAD) {
#pragma unroll
        for (int kd = 0; kd < KD; ++kd) {
            Raw4<T> raw[2 * VO];
            aux_raw(p_first + PD - kd, raw);
            aux_pairs(raw, auxs[WGRAD ? (PD - kd + KD) % KD : 0]);
        }
    }
    wait_but_newest();
    __syncthreads();

    auto step = [&](auto rot, int p) {
        constexpr int R = decltype(rot)::value;
        constexpr int DONE = (R - PD + 2 * KD) % KD;     // slot of plane p-PD, reused for p+1+PD
        Raw4<T> aux_next[2 * VO];                          // strips of plane p+1+PD, in flight
        aux_raw(p + 1 + PD, aux_next);
        if (plane_ok(p + 2)) copy_plane(p + 2); else if (VEC) cp_async_commit();
        const int qdone = p - PD;
        if (k_ok && p >= 0 && p < D) accumulate(rot, p);
        if (qdone >= d0 && qdone < d1) finish(qdone, k_ok, kacc[DONE]);
#pragma unroll
        for (int v = 0; v < VK; ++v) kacc[DONE][v] = pack2(0.0f, 0.0f);
        if (WGRAD) {
            // keep the conversion of the raw strips here, after the step's arithmetic: done
            // right after the loads it would make the warp wait for them at the top of the step
            if (sizeof(T) == 2) {
#pragma unroll
                for (int i = 0; i < 2 * VO; ++i) hold_raw(aux_next[i]);
            }
            aux_pairs(aux_next, auxs[WGRAD ? DONE : 0]);
        }
        wait_but_newest();   // plane p+1 has landed; p+2 may still be in flight
        __syncthreads();
    };
    int p = p_first;
    while (p <= p_last) {
        step(std::integral_constant<int, 0>{}, p++);
        if (p > p_last) break;
        step(std::integral_constant<int, 1 % KD>{}, p++);
        if (p > p_last) break;
        if (KD > 2) step(std::integral_constant<int, 2 % KD>{}, p++);
        if (KD > 3) {
            if (p > p_last) break;
            step(std::integral_constant<int, 3 % KD>{}, p++);
            if (p > p_last) break;
            if (KD > 4) step(std::integral_constant<int, 4 % KD>{}, p++);
        }
    }
    if (WGRAD && P.partial) {
        // per-CTA combine in a fixed order: slot-major scratch rows of taps*4 (+1 pad) floats
        constexpr int LD = KT * SCH + 1;
        if (VEC) cp_async_wait_all();
        __syncthreads();
#pragma unroll
        for (int k = 0; k < NW; ++k) {
            float lo, up;
            unpack2(accw[k], lo, up);
            sbuf[slot * LD + k * SCH + jch] = lo + up;
        }
        __syncthreads();
        float* out = P.partial + (long long)blockIdx.x * kPartialStride;
        for (int k = tid; k < KT * SCH; k += NT) {
            float s = 0.0f;
            for (int i = 0; i < NG; ++i) s += sbuf[i * LD + k];
            out[k] = s;
        }
    }
}

// ------------------------------------------------------------------------------------------
struct GzParams {
    const float* gt1;           // float32 scratch
    const void* z;
    void* gz;                   // holds the direct term on entry, gz on exit (or NULL)
    const float* h; const float* bias;
    float* partial;             // [cta][kPartialStride]
    int C, D, H, W;
    Tiling t;
    int relu;
};

// Floats of shared memory the end-of-kernel combine of gz_kernel needs: one row of sums (+1 pad)
// per thread.
template <int KD, int KH, int KW, int CS>
__host__ __device__ constexpr int gz_combine_floats(int nthreads) {
    return nthreads * ((KD * KH * KW + 1) * (SCH / CS) + 1);
}

// CS = channel split: CS threads share one 4-voxel strip and each takes SCH/CS channels (a
// whole number of pairs).  The correlation sums are per channel, so CS = 2 halves the registers
// a thread needs (54 + 2 sums instead of 108 + 4) and twice as many warps fit on an SM; the two
// threads sit in adjacent lanes and read the same window quads.
template <typename T, int KD, int KH, int KW, int NT, int MAXX, bool VEC, bool WGRAD, int WQ, int CS>
__global__ void __launch_bounds__(NT, CS == 2 ? 512 / NT : 256 / NT) gz_kernel(const GzParams P) {
    constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2, KT = KD * KH * KW;
    using L = RingSmem<KD, KH, KW>;
    constexpr int RING = L::RING;
    constexpr int NQA = 1 + (2 * PW + 3) / 4;
    constexpr int CH = SCH / CS;          // channels per thread
    constexpr int NP = CH / 2;            // channel pairs per thread
    constexpr int NACC = (WGRAD ? KT * SCH : 0) + SCH;      // sums per CTA record
    constexpr int NLOC = (WGRAD ? KT * CH : 0) + CH;        // sums per thread
    static_assert(CS == 1 || CS == 2, "channel split");
    extern __shared__ __align__(16) float smem[];
    const L lay(P.t, 1, gz_combine_floats<KD, KH, KW, CS>(NT));
    const int tid = threadIdx.x;
    const int part = tid % CS;            // which channels: part*CH .. part*CH + CH-1
    constexpr bool ROWS = KD > 1 && KH == 1;   // images of a batch as the rows of one volume
    const int NQ = WQ ? WQ : P.t.NQ, pitch = WQ ? row_pitch(4 * WQ) : P.t.pitch,
              W = WQ ? 4 * WQ : P.W, D = P.D;   // WQ > 0: the width is a compile-time constant
    const SlabAddr<ROWS> addr(P.C, D, P.H, W);
    const long long HW = addr.plane, SP = addr.chan;
    const long long RWX = ROWS ? addr.row_x : W, RWZ = ROWS ? addr.row_z : W;

    int blk = blockIdx.x;
    const int th = blk % P.t.nth; blk /= P.t.nth;
    const int dch = blk % P.t.ndc; blk /= P.t.ndc;
    const int bc = blk;
    const int c = bc % P.C;
    const int h_band = th * P.t.TH;
    const int TH = min(P.t.TH, P.H - h_band);
    const int d0 = dch * P.t.DC, d1 = min(D, d0 + P.t.DC);
    const int RT = lay.RT;
    // rows mode: the band is folded into the base pointers and rows are counted from it
    const int h0 = ROWS ? 0 : h_band, H = ROWS ? P.H - h_band : P.H;
    const long long bx = (long long)bc * SP + (ROWS ? h_band * RWX : 0);
    const long long bz = ((long long)bc * SCH + part * CH) * SP + (ROWS ? h_band * RWZ : 0);

    const float* tg = P.gt1 + bx;
    const T* zg = reinterpret_cast<const T*>(P.z) + bz;
    T* gzg = P.gz ? reinterpret_cast<T*>(P.gz) + bz : nullptr;

    float* wA = smem + lay.wA;
    float* ring = smem + lay.ring0;
    ChunkDesc* desc = reinterpret_cast<ChunkDesc*>(smem + lay.desc);
    for (int i = tid; i < RING * lay.plane_t; i += NT) ring[i] = 0.0f;
    {
        const float* hc = P.h + (long long)c * SCH * KT;
        for (int i = tid; i < KT * SCH; i += NT) wA[i] = hc[(i % SCH) * KT + i / SCH];
    }
    const int nx = RT * NQ;
    if (KD > 1) build_descs(desc, 1, RT, NQ, pitch, h0 - PH, H, W, SP, RWX, NT);
    float bj[CH];
#pragma unroll
    for (int j = 0; j < CH; ++j) bj[j] = P.bias ? P.bias[c * SCH + part * CH + j] : 0.0f;
    // filter-gradient sums [tap][channel pair] (if WGRAD), and the bias sums
    constexpr int NW2 = WGRAD ? KT * NP : 1;
    f32x2 acc2[NW2];
    float gbs[CH];
#pragma unroll
    for (int k = 0; k < NW2; ++k) acc2[k] = pack2(0.0f, 0.0f);
#pragma unroll
    for (int j = 0; j < CH; ++j) gbs[j] = 0.0f;
    __syncthreads();

    const int qbase = d0 - PD - 1;
    auto slot_of = [&](int q) { return (q - qbase) % RING; };
    auto load_now = [&](int plane) {
        const float* src = tg + (long long)plane * HW;
        float* dst = ring + slot_of(plane) * lay.plane_t;
        for (int id = tid; id < nx; id += NT) {
            const int c4 = id % NQ, r = id / NQ;
            const int h = h0 - PH + r, w = 4 * c4, n = min(4, W - w);
            if (h < 0 || h >= H) continue;
            stage_chunk<PW, false>(dst, (r * pitch) | (w << 16) | (n << 26),
                                   load4<float, VEC>(src + h * RWX + w, n));
        }
    };
    for (int q = d0 - PD; q <= d0 + PD; ++q)
        if (q >= 0 && q < D) load_now(q);
    __syncthreads();

    const int items = TH * NQ;
    constexpr int NSLOT = NT / CS;        // strips in flight per CTA
    const int slot0 = tid / CS;
    // z (and the direct term) of the next item are fetched while the current one is computed
    constexpr int NSTR = 2 * CH;
    StripFetcher<T, VEC, NSTR, NT> fetch(smem + lay.total_floats);
    auto strip_ptrs = [&](int d, int item, const T* (&ptr)[NSTR]) {
        const long long off = (long long)d * HW + (h0 + item / NQ) * RWZ + VA * (item % NQ);
#pragma unroll
        for (int j = 0; j < CH; ++j) {
            ptr[j] = zg + j * SP + off;
            ptr[CH + j] = (gzg ? gzg : zg) + j * SP + off;
        }
    };
    if (slot0 < items && d0 < d1) {
        const T* ptr[NSTR];
        strip_ptrs(d0, slot0, ptr);
        fetch.request(ptr);
    }
    for (int d = d0; d < d1; ++d) {
        float4 tr[MAXX];
        const int qn = d + PD + 1;
        const bool have = KD > 1 && d + 1 < d1 && qn < D;
        if (have) {
#pragma unroll
            for (int i = 0; i < MAXX; ++i) {
                const int id = tid + i * NT;
                if (id < nx) {
                    const ChunkDesc dsc = desc[id];
                    if (dsc.goff >= 0)
                        tr[i] = load4<float, VEC>(tg + (long long)qn * HW + dsc.goff, desc_n(dsc.soff));
                }
            }
        }
#pragma unroll 1
        for (int item = slot0; item < items; item += NSLOT) {
            const int a_row = item / NQ, a_q = item % NQ;
            const int hrow = h0 + a_row, w0 = VA * a_q;
            const long long off = (long long)d * HW + hrow * RWZ;
            float strips[NSTR][VA];
            {
                const T* ptr[NSTR];
                strip_ptrs(d, item, ptr);
                fetch.receive(ptr, w0, W, strips);
                int nd = d, nitem = item + NSLOT;
                if (nitem >= items) { nitem = slot0; nd = d + 1; }
                if (nd < d1 && nitem < items) {
                    strip_ptrs(nd, nitem, ptr);
                    fetch.request(ptr);
                }
            }
            float sv[CH][VA], pre[CH][VA];
#pragma unroll
            for (int j = 0; j < CH; ++j) {
#pragma unroll
                for (int v = 0; v < VA; ++v) {
                    pre[j][v] = strips[j][v] + bj[j];
                    sv[j][v] = P.relu ? fmaxf(pre[j][v], 0.0f) : pre[j][v];
                    if (w0 + v >= W) sv[j][v] = 0.0f;
                }
            }
            // channel pairs (2jp, 2jp+1) of one voxel share a register pair; the accumulators
            // start from the direct term
            f32x2 ag[NP][VA], s2[NP][VA];
#pragma unroll
            for (int jp = 0; jp < NP; ++jp)
#pragma unroll
                for (int v = 0; v < VA; ++v) {
                    ag[jp][v] = gzg ? pack2(strips[CH + 2 * jp][v], strips[CH + 2 * jp + 1][v])
                                    : pack2(0.0f, 0.0f);
                    s2[jp][v] = pack2(sv[2 * jp][v], sv[2 * jp + 1][v]);
                }
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) {
                const int q = d + PD - kd;
                if (q < 0 || q >= D) continue;
                const int slot = slot_of(q);
#pragma unroll
                for (int kh = 0; kh < KH; ++kh) {
                    const int rr = a_row + PH + PH - kh;
                    float tv[4 * NQA];
                    load_window<NQA, false>(ring + slot * lay.plane_t + rr * pitch, a_q + 1, tv);
                    f32x2 t2[VA + KW - 1];
#pragma unroll
                    for (int i = 0; i < VA + KW - 1; ++i) t2[i] = pack2(tv[i], tv[i]);
#pragma unroll
                    for (int kw = 0; kw < KW; ++kw) {
                        const float* wp4 = wA + ((kd * KH + kh) * KW + kw) * SCH + part * CH;
                        f32x2 wp[NP];
                        if (CS == 1) {
                            const float4 w4 = *reinterpret_cast<const float4*>(wp4);
                            wp[0] = pack2(w4.x, w4.y);
                            wp[NP - 1] = pack2(w4.z, w4.w);
                        } else {
                            const float2 w2 = *reinterpret_cast<const float2*>(wp4);
                            wp[0] = pack2(w2.x, w2.y);
                        }
#pragma unroll
                        for (int jp = 0; jp < NP; ++jp) {
                            const int k2 = WGRAD ? ((kd * KH + kh) * KW + kw) * NP + jp : 0;
                            f32x2 a = acc2[k2];
#pragma unroll
                            for (int v = 0; v < VA; ++v) {
                                fma2(ag[jp][v], t2[v + 2 * PW - kw], wp[jp]);
                                if (WGRAD) fma2(a, s2[jp][v], t2[v + 2 * PW - kw]);
                            }
                            if (WGRAD) acc2[k2] = a;
                        }
                    }
                }
            }
            if (gzg) {
#pragma unroll
                for (int j = 0; j < CH; ++j) {
                    float dv[VA];
#pragma unroll
                    for (int v = 0; v < VA; ++v) {
                        float r = lane_of(ag[j / 2][v], j & 1);
                        if (P.relu && !(pre[j][v] > 0.0f)) r = 0.0f;
                        if (w0 + v >= W) r = 0.0f;
                        dv[v] = r;
                        // the bias gradient sums the values as stored (rounded to the storage type)
                        gbs[j] += to_f32(from_f32<T>(r));
                    }
                    store_strip_global<T, VEC, VA>(gzg + j * SP + off, w0, W, dv);
                }
            }
        }
        if (have) {
#pragma unroll
            for (int i = 0; i < MAXX; ++i) {
                const int id = tid + i * NT;
                if (id < nx) {
                    const ChunkDesc dsc = desc[id];
                    if (dsc.goff >= 0) stage_chunk<PW, false>(ring + slot_of(qn) * lay.plane_t, dsc.soff, tr[i]);
                }
            }
        }
        __syncthreads();
    }
    float* out = P.partial + (long long)blockIdx.x * kPartialStride;
    // Per-CTA combine in a fixed order.  Thread rows hold [tap][own channel] filter sums, then
    // the own bias sums; record layout: [0, taps*4) filter sums [tap][channel] (zero if not
    // WGRAD), [124, 128) bias sums.
    constexpr int LD = NLOC + 1;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NLOC - CH; ++k) ring[tid * LD + k] = lane_of(acc2[k / 2], k & 1);
#pragma unroll
    for (int j = 0; j < CH; ++j) ring[tid * LD + NLOC - CH + j] = gbs[j];
    __syncthreads();
    for (int k = tid; k < NACC; k += NT) {
        const bool is_bias = k >= NACC - SCH;
        const int j = is_bias ? k - (NACC - SCH) : k % SCH;          // channel of this sum
        const int loc = is_bias ? NLOC - CH + j % CH : (k / SCH) * CH + j % CH;
        float s = 0.0f;
        for (int i = j / CH; i < NT; i += CS) s += ring[i * LD + loc];
        out[is_bias ? kPartialStride - SCH + j : k] = s;
    }
}

// ------------------------------------------------------------------------------------------
// gh[c][j][tau] = sum over CTAs of group c, in launch order, of both partial sets; gb likewise.
struct ReduceParams {
    const float* partial_a;   // kconv records, gden half (or NULL)
    const float* partial_a2;  // kconv records, gnum half (or NULL)
    const float* partial_b;   // gz kernel records (or NULL)
    long long ctas_per_bc_a, ctas_per_bc_b;  // records per (sample, group) pair
    int b_has_w;              // the gz records carry filter sums
    int B, C, KT;
    float* gh;    // (C, 4, KT) or NULL
    float* gb;    // (C*4) or NULL
};

template <int NT>
__global__ void __launch_bounds__(NT) reduce_kernel(const ReduceParams P) {
    const int c = blockIdx.x;
    const int k = threadIdx.x;       // record slot
    const bool is_w = k < P.KT * SCH, is_b = k >= kPartialStride - SCH;
    if (!is_w && !is_b) return;
    float s = 0.0f;
    for (int b = 0; b < P.B; ++b) {
        const long long bc = (long long)b * P.C + c;
        if (P.partial_a && is_w)
            for (long long i = 0; i < P.ctas_per_bc_a; ++i)
                s += P.partial_a[(bc * P.ctas_per_bc_a + i) * kPartialStride + k];
        if (P.partial_a2 && is_w)
            for (long long i = 0; i < P.ctas_per_bc_a; ++i)
                s += P.partial_a2[(bc * P.ctas_per_bc_a + i) * kPartialStride + k];
        if (P.partial_b && (is_b || P.b_has_w))
            for (long long i = 0; i < P.ctas_per_bc_b; ++i)
                s += P.partial_b[(bc * P.ctas_per_bc_b + i) * kPartialStride + k];
    }
    if (is_w && P.gh) {
        const int j = k % SCH, tau = k / SCH;     // records are [tau][j]; gh is (c, j, tau)
        P.gh[((long long)c * SCH + j) * P.KT + tau] = s;
    }
    if (is_b && P.gb) P.gb[c * SCH + (k - (kPartialStride - SCH))] = s;
}

}  // namespace dw4
}  // namespace ndc
