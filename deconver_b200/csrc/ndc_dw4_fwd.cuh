// Fused forward update for the depthwise ratio-4 geometry (m = 1, sc = 4):
//
//     s = relu(z + b);  t1 = K(s);  out = (s * (A(x) + eps)) / (A(t1) + eps)
//
// in ONE kernel.  This is the forward of 2-D image batches (5x5 and 3x3 kernels, marching down
// the image rows or band by band); 3x3x3 volumes take two launches instead (ksrc_kernel, then
// ratio_kernel in its forward mode), which was measured faster on every volume size.  t1 never makes a round trip through HBM: each CTA marches through its depth
// chunk and keeps the planes it needs in shared-memory rings.  Per step p (a source plane):
//
//   prefetch   z plane p+1 and x plane p-PD into registers, raw (global loads in flight;
//              converted, biased and rectified only when they are staged)
//   K phase    an 8-voxel strip of the t1 band (TH + 2*PH rows) is shared by two threads, each
//              convolving two of the four source channels; each keeps KD partial running
//              sums, one per t1 plane that source plane p contributes to; plane p-PD is
//              complete after this step: the two halves are added (one shuffle) and go to
//              the t1 ring (and to HBM)
//   stage      the prefetched planes are rectified/biased and written to shared memory
//   barrier
//   A phase    output plane d = p-2*PD, 4-voxel strips: A(x) and A(t1) from the rings,
//              epilogue, store
//
// One barrier per step: the s buffer is double-buffered and both rings hold KD+1 planes, so
// whatever a fast thread writes in step p+1 is never what a slow thread still reads in p.
#pragma once

#include "ndc_dw4_common.cuh"

namespace ndc {
namespace dw4 {

struct FwdParams {
    const void* x; const void* z; const float* h; const float* bias;
    void* out; void* t1;
    int C, D, H, W;
    Tiling t;
    float eps;
    int relu;
};

template <int KD, int KH, int KW>
struct FwdSmem {
    static constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2;
    static constexpr int WKP = (KD * KW + 3) / 4 * 4;  // padded weights per (kh, j), K layout
    static constexpr int RING = KD > 1 ? KD + 1 : 1;   // planes per ring
    static constexpr int NSB = KD > 1 ? 2 : 1;         // source buffers
    int wA, wK, sbuf, t1ring, xring, zdesc, xdesc, total_floats;  // float offsets
    int RS, RT, plane_s, plane_t;
    __host__ __device__ FwdSmem(const Tiling& t) {
        RS = t.TH + 4 * PH;
        RT = t.TH + 2 * PH;
        plane_s = SCH * RS * t.pitch;
        plane_t = RT * t.pitch;
        int o = 0;
        wA = o; o += KD * KH * KW * SCH;
        wK = o; o += KH * SCH * WKP;
        o = (o + 3) / 4 * 4;
        sbuf = o; o += NSB * plane_s;
        t1ring = o; o += RING * plane_t;
        xring = o; o += RING * plane_t;
        zdesc = o;                                    // (end of the zero-initialised area)
        xdesc = o; o += KD > 1 ? 2 * (RT * t.NQ) : 0;  // x loader table: marching kernels only
        total_floats = o;
    }
};

template <typename T, int KD, int KH, int KW, int NT, int MAXZ, int MAXX, int MINB, bool VEC, int WQ>
__global__ void __launch_bounds__(NT, MINB) fwd_kernel(const FwdParams P) {
    constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2;
    using L = FwdSmem<KD, KH, KW>;
    constexpr int WKP = L::WKP, RING = L::RING, NSB = L::NSB;
    constexpr int NQA = 1 + (2 * PW + 3) / 4;   // quads in a 4-strip window (4 + 2*PW floats)
    extern __shared__ __align__(16) float smem[];
    const L lay(P.t);
    const int tid = threadIdx.x;
    constexpr bool ROWS = KD > 1 && KH == 1;   // images of a batch as the rows of one volume
    const int NQ = WQ ? WQ : P.t.NQ, NS8 = (NQ + 1) / 2, pitch = WQ ? row_pitch(4 * WQ) : P.t.pitch,
              W = WQ ? 4 * WQ : P.W, D = P.D;   // WQ > 0: the width is a compile-time constant
    const SlabAddr<ROWS> addr(P.C, D, P.H, W);
    const long long HW = addr.plane, SP = addr.chan;
    const long long RWX = ROWS ? addr.row_x : W, RWZ = ROWS ? addr.row_z : W;

    // ---- which work item
    int blk = blockIdx.x;
    const int th = blk % P.t.nth; blk /= P.t.nth;
    const int dch = blk % P.t.ndc; blk /= P.t.ndc;
    const int bc = blk;                 // b * C + c
    const int c = bc % P.C;
    const int h_band = th * P.t.TH;     // first row of this CTA's band
    const int TH = min(P.t.TH, P.H - h_band);
    const int d0 = dch * P.t.DC, d1 = min(D, d0 + P.t.DC);
    const int RS = lay.RS, RT = lay.RT;
    // rows mode: the band is folded into the base pointers and rows are counted from it
    const int h0 = ROWS ? 0 : h_band, H = ROWS ? P.H - h_band : P.H;
    const long long bx = (long long)bc * SP + (ROWS ? h_band * RWX : 0);
    const long long bz = (long long)bc * SCH * SP + (ROWS ? h_band * RWZ : 0);

    const T* xg = reinterpret_cast<const T*>(P.x) + bx;
    const T* zg = reinterpret_cast<const T*>(P.z) + bz;
    T* og = reinterpret_cast<T*>(P.out) + bz;
    T* tg = reinterpret_cast<T*>(P.t1) + bx;

    float* wA = smem + lay.wA;
    float* wK = smem + lay.wK;
    float* sbuf = smem + lay.sbuf;
    float* t1ring = smem + lay.t1ring;
    float* xring = smem + lay.xring;
    ChunkDesc* xdesc = reinterpret_cast<ChunkDesc*>(smem + lay.xdesc);

    // ---- one-time set-up: zero the planes, stage the filter, build the loader tables
    for (int i = tid; i < (lay.zdesc - lay.sbuf) / 4; i += NT)
        reinterpret_cast<float4*>(sbuf)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    {
        const float* hc = P.h + (long long)c * SCH * (KD * KH * KW);
        for (int i = tid; i < KD * KH * KW * SCH; i += NT) {
            const int j = i % SCH, tau = i / SCH;           // wA[tau][j]
            wA[i] = hc[j * (KD * KH * KW) + tau];
        }
        for (int i = tid; i < KH * SCH * WKP; i += NT) {    // wK[kh][j][kd*KW + kw]
            const int e = i % WKP, j = (i / WKP) % SCH, kh = i / (WKP * SCH);
            float v = 0.0f;
            if (e < KD * KW) {
                const int kd = e / KW, kw = e % KW;
                v = hc[j * (KD * KH * KW) + (kd * KH + kh) * KW + kw];
            }
            wK[i] = v;
        }
    }
    const int nz = SCH * RS * NQ, nx = RT * NQ;
    // The source buffer is UNshifted (shared column c holds w = c - 4) and swizzled: 16-byte
    // chunks of z land on whole quads, and an 8-voxel strip reads a 4-quad window.
    auto z_soff = [&](int ch, int r, int c4, int n) {
        return ((ch * RS + r) * pitch + (phys_quad<true>(c4 + 1) << 2)) | (n << 26) | (ch << 29);
    };
    if (KD > 1) build_descs(xdesc, 1, RT, NQ, pitch, h0 - PH, H, W, SP, RWX, NT);
    float bj[SCH];
#pragma unroll
    for (int j = 0; j < SCH; ++j) bj[j] = P.bias ? P.bias[c * SCH + j] : 0.0f;

    // ---- this thread's chunks of a z plane (fixed for the CTA's lifetime, kept in registers):
    // element offset in the plane (-1: nothing to load), shared offset | valid count, bias
    int zg_off[MAXZ], zs_off[MAXZ];
    float zb[MAXZ];
#pragma unroll
    for (int i = 0; i < MAXZ; ++i) {
        const int id = tid + i * NT;
        zg_off[i] = -1; zs_off[i] = 0; zb[i] = 0.0f;
        if (KD > 1 && id < nz) {
            const int c4 = id % NQ, t = id / NQ, r = t % RS, ch = t / RS;
            const int h = h0 - 2 * PH + r, w = 4 * c4;
            if (h >= 0 && h < H) zg_off[i] = (int)(ch * SP + h * RWZ) + w;
            zs_off[i] = z_soff(ch, r, c4, min(4, W - w));
            zb[i] = ch == 0 ? bj[0] : ch == 1 ? bj[1] : ch == 2 ? bj[2] : bj[3];
        }
    }

    // ---- this thread's K strip (8 voxels of one row of the t1 band), its channel pair and
    // its partial running sums.  lane = pair*16 + strip lane: a quarter-warp reads 8
    // consecutive strips of one channel.
    constexpr int NG = NT / 2;                              // strip slots per CTA
    const int cpair = (tid >> 4) & 1;
    const int k_slot = (tid >> 5) * 16 + (tid & 15);
    const int n_kitems = (TH + 2 * PH) * NS8;
    const int k_row = k_slot < n_kitems ? k_slot / NS8 : 0, k_strip = k_slot < n_kitems ? k_slot % NS8 : 0;
    const bool k_ok = k_slot < n_kitems && h0 - PH + k_row >= 0 && h0 - PH + k_row < H;
    float kacc[KD][VK];
#pragma unroll
    for (int a = 0; a < KD; ++a)
#pragma unroll
        for (int v = 0; v < VK; ++v) kacc[a][v] = 0.0f;
    const int a_items = TH * NQ;
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
    auto fetch_z = [&](Raw4<T> (&reg)[MAXZ], int plane) {
        const T* src = zg + (long long)plane * HW;
#pragma unroll
        for (int i = 0; i < MAXZ; ++i)
            if (zg_off[i] >= 0) reg[i] = load4_raw<T, VEC>(src + zg_off[i], (zs_off[i] >> 26) & 7);
    };
    auto stage_z = [&](const Raw4<T> (&reg)[MAXZ], int plane) {
        float* dst = sbuf + (plane & (NSB - 1)) * lay.plane_s;
#pragma unroll
        for (int i = 0; i < MAXZ; ++i)
            if (zg_off[i] >= 0)
                *reinterpret_cast<float4*>(dst + (zs_off[i] & 0x3ffffff)) =
                    rectify(to_float4(reg[i]), zb[i], (zs_off[i] >> 26) & 7);
    };
    auto fetch_x = [&](Raw4<T> (&reg)[MAXX], int plane) {
        const T* src = xg + (long long)plane * HW;
#pragma unroll
        for (int i = 0; i < MAXX; ++i) {
            const int id = tid + i * NT;
            if (id < nx) {
                const ChunkDesc dsc = xdesc[id];
                if (dsc.goff >= 0) reg[i] = load4_raw<T, VEC>(src + dsc.goff, desc_n(dsc.soff));
            }
        }
    };
    auto stage_x = [&](const Raw4<T> (&reg)[MAXX], int slot) {
        float* dst = xring + slot * lay.plane_t;
#pragma unroll
        for (int i = 0; i < MAXX; ++i) {
            const int id = tid + i * NT;
            if (id < nx) {
                const ChunkDesc dsc = xdesc[id];
                if (dsc.goff >= 0) stage_chunk<PW, false>(dst, dsc.soff, to_float4(reg[i]));
            }
        }
    };
    // plane loads without prefetch (prologue; the only loads of a 2-D problem): chunks are
    // decoded on the fly
    auto load_z_now = [&](int plane) {
        const T* src = zg + (long long)plane * HW;
        float* dst = sbuf + (plane & (NSB - 1)) * lay.plane_s;
        for (int id = tid; id < nz; id += NT) {
            const int c4 = id % NQ, t = id / NQ, r = t % RS, ch = t / RS;
            const int h = h0 - 2 * PH + r, w = 4 * c4, n = min(4, W - w);
            if (h < 0 || h >= H) continue;
            const int soff = z_soff(ch, r, c4, n);
            const float4 v = load4<T, VEC>(src + ch * SP + h * RWZ + w, n);
            const float b = ch == 0 ? bj[0] : ch == 1 ? bj[1] : ch == 2 ? bj[2] : bj[3];
            *reinterpret_cast<float4*>(dst + (soff & 0x3ffffff)) = rectify(v, b, n);
        }
    };
    auto load_x_now = [&](int plane, int slot) {
        const T* src = xg + (long long)plane * HW;
        float* dst = xring + slot * lay.plane_t;
        for (int id = tid; id < nx; id += NT) {
            const int c4 = id % NQ, r = id / NQ;
            const int h = h0 - PH + r, w = 4 * c4, n = min(4, W - w);
            if (h < 0 || h >= H) continue;
            const int soff = (r * pitch) | (w << 16) | (n << 26);
            stage_chunk<PW, false>(dst, soff, load4<T, VEC>(src + h * RWX + w, n));
        }
    };
    const int qbase = d0 - 3 * PD - 1;  // ring slot of plane q is (q - qbase) % RING
    auto slot_of = [&](int q) { return (q - qbase) % RING; };

    // ---- prologue: first source plane
    const int p_first = d0 - 2 * PD, p_last = d1 - 1 + 2 * PD;
    if (p_first >= 0 && p_first < D) load_z_now(p_first);
    if (KD == 1) load_x_now(p_first, 0);
    __syncthreads();

    for (int p = p_first; p <= p_last; ++p) {
        // -------- prefetch (global loads stay in flight during the K phase)
        Raw4<T> zr[MAXZ], xr[MAXX];
        const bool have_z = KD > 1 && p + 1 <= p_last && p + 1 >= 0 && p + 1 < D;
        const int xq = p - PD;
        const bool have_x = KD > 1 && xq >= 0 && xq < D && xq >= d0 - PD && xq <= d1 - 1 + PD;
        if (have_z) fetch_z(zr, p + 1);
        if (have_x) fetch_x(xr, xq);

        // -------- K phase: source plane p feeds t1 planes p+PD-kd
        const bool s_ok = p >= 0 && p < D;
        const int qdone = p - PD;  // t1 plane completed by this step
        const bool q_need = qdone >= d0 - PD && qdone <= d1 - 1 + PD && qdone >= 0 && qdone < D;
        auto k_accumulate = [&](int row, int strip, float (&acc)[KD][VK]) {
            const float* sp = sbuf + (p & (NSB - 1)) * lay.plane_s + row * pitch;
            int qo[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) qo[q] = phys_quad<true>(2 * strip + q) << 2;
            // rolled on purpose: the body is the unit the instruction cache holds
#pragma unroll 1
            for (int kh = 0; kh < KH; ++kh) {
#pragma unroll
                for (int jj = 0; jj < 2; ++jj) {
                    const int j = 2 * cpair + jj;
                    const float* rp = sp + (j * RS + kh) * pitch;
                    float sv[16];
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 t = *reinterpret_cast<const float4*>(rp + qo[q]);
                        sv[4 * q] = t.x; sv[4 * q + 1] = t.y; sv[4 * q + 2] = t.z; sv[4 * q + 3] = t.w;
                    }
                    float w[WKP];
#pragma unroll
                    for (int q4 = 0; q4 < WKP / 4; ++q4) {
                        const float4 t = *reinterpret_cast<const float4*>(
                            wK + (kh * SCH + j) * WKP + 4 * q4);
                        w[4 * q4] = t.x; w[4 * q4 + 1] = t.y; w[4 * q4 + 2] = t.z; w[4 * q4 + 3] = t.w;
                    }
#pragma unroll
                    for (int kd = 0; kd < KD; ++kd)
#pragma unroll
                        for (int kw = 0; kw < KW; ++kw)
#pragma unroll
                            for (int v = 0; v < VK; ++v)
                                acc[kd][v] = fmaf(sv[4 - PW + v + kw], w[kd * KW + kw], acc[kd][v]);
                }
            }
        };
        // add the two channel halves; each lane then owns one quad of the strip.  `row < 0`
        // marks a lane that only takes part in the exchange.
        auto k_finish = [&](int row, int strip, const float (&part)[VK]) {
            float tv[VA];
#pragma unroll
            for (int i = 0; i < VA; ++i) {
                const float send = cpair ? part[i] : part[VA + i];
                const float keep = cpair ? part[VA + i] : part[i];
                tv[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
            }
            if (row < 0) return;
            const int w0 = VK * strip + VA * cpair;
            // the ring holds t1 as it is stored (rounded to the storage type), so the
            // denominator here is the one backward recomputes from the saved t1
#pragma unroll
            for (int v = 0; v < VA; ++v) tv[v] = (w0 + v >= W) ? 0.0f : to_f32(from_f32<T>(tv[v]));
            store_strip<VA, PW, false>(t1ring + slot_of(qdone) * lay.plane_t + row * pitch, w0, tv);
            const int h = h0 - PH + row;
            if (qdone >= d0 && qdone < d1 && row >= PH && row < PH + TH)
                store_strip_global<T, VEC, VA>(tg + (long long)qdone * HW + h * RWX, w0, W, tv);
        };
        if (KD > 1) {
            if (k_ok && s_ok) k_accumulate(k_row, k_strip, kacc);
            if (q_need) k_finish(k_ok ? k_row : -1, k_strip, kacc[KD - 1]);
            // rotate the running sums: slot kd now stands for plane (p+1)+PD-kd
#pragma unroll
            for (int kd = KD - 1; kd > 0; --kd)
#pragma unroll
                for (int v = 0; v < VK; ++v) kacc[kd][v] = kacc[kd - 1][v];
#pragma unroll
            for (int v = 0; v < VK; ++v) kacc[0][v] = 0.0f;
        } else if (s_ok && q_need) {
            // no depth taps: nothing persists between planes, so strips are simply looped over
            // (all lanes run every round: the channel halves exchange partial sums)
            const int rounds = (n_kitems + NG - 1) / NG;
#pragma unroll 1
            for (int r = 0; r < rounds; ++r) {
                const int item = k_slot + r * NG;
                const int row = item < n_kitems ? item / NS8 : 0, strip = item < n_kitems ? item % NS8 : 0;
                const int h = h0 - PH + row;
                const bool ok = item < n_kitems && h >= 0 && h < H;
                float acc[KD][VK];
#pragma unroll
                for (int v = 0; v < VK; ++v) acc[0][v] = 0.0f;
                if (ok) k_accumulate(row, strip, acc);
                k_finish(ok ? row : -1, strip, acc[KD - 1]);
            }
        }

        // -------- stage the prefetched planes
        if (have_z) stage_z(zr, p + 1);
        if (have_x) stage_x(xr, slot_of(xq));
        __syncthreads();

        // -------- A phase: output plane d
        const int d = p - 2 * PD;
        if (d < d0 || d >= d1) continue;
#pragma unroll 1
        for (int item = tid; item < a_items; item += NT) {
            const int a_row = item / NQ, a_q = item % NQ;
            const int hrow = h0 + a_row, w0 = VA * a_q;
            Raw4<T> zraw[SCH];   // converted in the epilogue, after the tap sweep
#pragma unroll
            for (int j = 0; j < SCH; ++j)
                zraw[j] = load_strip_raw<T, VEC>(zg + j * SP + (long long)d * HW + hrow * RWZ, w0, W);
            // accumulators hold channel pairs (2jp, 2jp+1) of one voxel
            f32x2 an[SCH / 2][VA], ad[SCH / 2][VA];
            {
                const f32x2 e2 = pack2(P.eps, P.eps);
#pragma unroll
                for (int jp = 0; jp < SCH / 2; ++jp)
#pragma unroll
                    for (int v = 0; v < VA; ++v) { an[jp][v] = e2; ad[jp][v] = e2; }
            }
#pragma unroll 1
            for (int kd = 0; kd < KD; ++kd) {
                const int q = d + PD - kd;
                if (q < 0 || q >= D) continue;
                const int slot = slot_of(q);
#pragma unroll
                for (int kh = 0; kh < KH; ++kh) {
                    const int rr = a_row + PH + PH - kh;  // ring row of h + PH - kh
                    adjoint_row2<KW, NQA>(xring + slot * lay.plane_t + rr * pitch,
                                          t1ring + slot * lay.plane_t + rr * pitch, a_q + 1,
                                          wA + (kd * KH + kh) * KW * SCH, an, ad);
                }
            }
#pragma unroll
            for (int j = 0; j < SCH; ++j) {
                float ov[VA], zj[VA];
                raw_to_array(zraw[j], zj);
#pragma unroll
                for (int v = 0; v < VA; ++v) {
                    float s = zj[v] + bj[j];
                    if (P.relu) s = fmaxf(s, 0.0f);
                    ov[v] = fast_div(s * lane_of(an[j / 2][v], j & 1), lane_of(ad[j / 2][v], j & 1));
                }
                store_strip_global<T, VEC, VA>(og + j * SP + (long long)d * HW + hrow * RWZ,
                                               w0, W, ov);
            }
        }
    }
}

}  // namespace dw4
}  // namespace ndc
