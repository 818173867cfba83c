// Fused forward update for the depthwise ratio-4 geometry (m = 1, sc = 4):
//
//     s = relu(z + b);  t1 = K(s);  out = (s * (A(x) + eps)) / (A(t1) + eps)
//
// in ONE kernel.  t1 never makes a round trip through HBM: each CTA marches through its depth
// chunk and keeps the planes it needs in shared-memory rings.  Per step p (a source plane):
//
//   prefetch   z plane p+1 and x plane p-PD into registers (global loads in flight)
//   K phase    every K-thread owns a strip of the t1 band (TH + 2*PH rows) and keeps KD
//              running sums, one per t1 plane that source plane p contributes to; plane
//              p-PD is complete after this step and goes to the t1 ring (and to HBM)
//   stage      the prefetched planes are rectified/biased and written to shared memory
//   barrier
//   A phase    output plane d = p-2*PD: A(x) and A(t1) from the rings, epilogue, store
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
    static constexpr int WKP = (KD * KW + 3) / 4 * 4;  // padded weights per (kh, j) in the K layout
    static constexpr int RING = KD > 1 ? KD + 1 : 1;  // planes per ring
    static constexpr int NSB = KD > 1 ? 2 : 1;        // source buffers
    // float offsets
    int wA, wK, sbuf, t1ring, xring, zdesc, xdesc, total_floats;
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
        zdesc = o; o += 2 * (SCH * RS * 2 * t.NS);
        xdesc = o; o += 2 * (RT * 2 * t.NS);
        total_floats = o;
    }
};

template <typename T, int KD, int KH, int KW, int NT, int RK, int RA, int MAXZ, int MAXX, int MINB,
          bool VEC>
__global__ void __launch_bounds__(NT, MINB) fwd_kernel(const FwdParams P) {
    constexpr int PD = KD / 2, PH = KH / 2, PW = KW / 2;
    using L = FwdSmem<KD, KH, KW>;
    constexpr int WKP = L::WKP, RING = L::RING, NSB = L::NSB;
    extern __shared__ __align__(16) float smem[];
    const L lay(P.t);
    const int tid = threadIdx.x;
    const int NS = P.t.NS, pitch = P.t.pitch, H = P.H, W = P.W, D = P.D;
    const long long HW = (long long)H * W, SP = HW * D;

    // ---- which work item
    int blk = blockIdx.x;
    const int th = blk % P.t.nth; blk /= P.t.nth;
    const int dch = blk % P.t.ndc; blk /= P.t.ndc;
    const int bc = blk;                 // b * C + c
    const int c = bc % P.C;
    const int h0 = th * P.t.TH;
    const int TH = min(P.t.TH, H - h0);
    const int d0 = dch * P.t.DC, d1 = min(D, d0 + P.t.DC);
    const int RS = lay.RS, RT = lay.RT;

    const T* xg = reinterpret_cast<const T*>(P.x) + (long long)bc * SP;
    const T* zg = reinterpret_cast<const T*>(P.z) + (long long)bc * SCH * SP;
    T* og = reinterpret_cast<T*>(P.out) + (long long)bc * SCH * SP;
    T* tg = reinterpret_cast<T*>(P.t1) + (long long)bc * SP;

    float* wA = smem + lay.wA;
    float* wK = smem + lay.wK;
    float* sbuf = smem + lay.sbuf;
    float* t1ring = smem + lay.t1ring;
    float* xring = smem + lay.xring;
    ChunkDesc* zdesc = reinterpret_cast<ChunkDesc*>(smem + lay.zdesc);
    ChunkDesc* xdesc = reinterpret_cast<ChunkDesc*>(smem + lay.xdesc);

    // ---- one-time set-up: zero the planes, stage the filter, build the loader tables
    for (int i = tid; i < lay.zdesc - lay.sbuf; i += NT) sbuf[i] = 0.0f;
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
    const int nz = SCH * RS * 2 * NS, nx = RT * 2 * NS;
    build_descs(zdesc, SCH, RS, NS, pitch, h0 - 2 * PH, H, W, SP, NT);
    build_descs(xdesc, 1, RT, NS, pitch, h0 - PH, H, W, SP, NT);
    float bj[SCH];
#pragma unroll
    for (int j = 0; j < SCH; ++j) bj[j] = P.bias ? P.bias[c * SCH + j] : 0.0f;

    // ---- this thread's strips
    int k_row[RK], k_strip[RK]; bool k_ok[RK];
    float kacc[RK][KD][V];
#pragma unroll
    for (int r = 0; r < RK; ++r) {
        const int item = tid + r * NT;
        k_row[r] = item / NS; k_strip[r] = item % NS;
        const int h = h0 - PH + k_row[r];
        k_ok[r] = item < (TH + 2 * PH) * NS && h >= 0 && h < H;
#pragma unroll
        for (int a = 0; a < KD; ++a)
#pragma unroll
            for (int v = 0; v < V; ++v) kacc[r][a][v] = 0.0f;
    }
    int a_row[RA], a_strip[RA]; bool a_ok[RA];
#pragma unroll
    for (int r = 0; r < RA; ++r) {
        const int item = tid + r * NT;
        a_row[r] = item / NS; a_strip[r] = item % NS;
        a_ok[r] = item < TH * NS;
    }
    __syncthreads();

    // stage helpers ----------------------------------------------------------------------
    auto stage_z = [&](const float4 (&reg)[MAXZ], int plane) {
        float* dst = sbuf + (plane & (NSB - 1)) * lay.plane_s;
#pragma unroll
        for (int i = 0; i < MAXZ; ++i) {
            const int id = tid + i * NT;
            if (id < nz) {
                const ChunkDesc dsc = zdesc[id];
                if (dsc.goff >= 0) {
                    const int so = dsc.soff & 0xffffff, n = dsc.soff >> 24;
                    const int j = id / (RS * 2 * NS);
                    const float b = j == 0 ? bj[0] : j == 1 ? bj[1] : j == 2 ? bj[2] : bj[3];
                    float4 v = reg[i];
                    v.x += b; v.y += b; v.z += b; v.w += b;
                    if (P.relu) {
                        v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f);
                        v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
                    }
                    if (n < 4) {  // elements past the end of the row stay zero
                        if (n < 2) v.y = 0.f;
                        if (n < 3) v.z = 0.f;
                        v.w = 0.f;
                    }
                    *reinterpret_cast<float4*>(dst + so) = v;
                }
            }
        }
    };
    auto fetch_z = [&](float4 (&reg)[MAXZ], int plane) {
        const T* src = zg + (long long)plane * HW;
#pragma unroll
        for (int i = 0; i < MAXZ; ++i) {
            const int id = tid + i * NT;
            if (id < nz) {
                const ChunkDesc dsc = zdesc[id];
                if (dsc.goff >= 0) reg[i] = load4<T, VEC>(src + dsc.goff, dsc.soff >> 24);
            }
        }
    };
    auto fetch_x = [&](float4 (&reg)[MAXX], int plane) {
        const T* src = xg + (long long)plane * HW;
#pragma unroll
        for (int i = 0; i < MAXX; ++i) {
            const int id = tid + i * NT;
            if (id < nx) {
                const ChunkDesc dsc = xdesc[id];
                if (dsc.goff >= 0) reg[i] = load4<T, VEC>(src + dsc.goff, dsc.soff >> 24);
            }
        }
    };
    auto stage_x = [&](const float4 (&reg)[MAXX], int slot) {
        float* dst = xring + slot * lay.plane_t;
#pragma unroll
        for (int i = 0; i < MAXX; ++i) {
            const int id = tid + i * NT;
            if (id < nx) {
                const ChunkDesc dsc = xdesc[id];
                if (dsc.goff >= 0)
                    *reinterpret_cast<float4*>(dst + (dsc.soff & 0xffffff)) = reg[i];
            }
        }
    };
    const int qbase = d0 - 3 * PD - 1;  // ring slot of plane q is (q - qbase) % RING
    auto slot_of = [&](int q) { return (q - qbase) % RING; };

    // plane loads without prefetch (prologue; the only loads of a 2-D problem)
    auto load_z_now = [&](int plane) {
        const T* src = zg + (long long)plane * HW;
        float* dst = sbuf + (plane & (NSB - 1)) * lay.plane_s;
        for (int id = tid; id < nz; id += NT) {
            const ChunkDesc dsc = zdesc[id];
            if (dsc.goff < 0) continue;
            const int so = dsc.soff & 0xffffff, n = dsc.soff >> 24;
            const int j = id / (RS * 2 * NS);
            const float b = j == 0 ? bj[0] : j == 1 ? bj[1] : j == 2 ? bj[2] : bj[3];
            float4 v = load4<T, VEC>(src + dsc.goff, n);
            v.x += b; v.y += b; v.z += b; v.w += b;
            if (P.relu) {
                v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f);
                v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
            }
            if (n < 4) {
                if (n < 2) v.y = 0.f;
                if (n < 3) v.z = 0.f;
                v.w = 0.f;
            }
            *reinterpret_cast<float4*>(dst + so) = v;
        }
    };
    auto load_x_now = [&](int plane, int slot) {
        const T* src = xg + (long long)plane * HW;
        float* dst = xring + slot * lay.plane_t;
        for (int id = tid; id < nx; id += NT) {
            const ChunkDesc dsc = xdesc[id];
            if (dsc.goff < 0) continue;
            *reinterpret_cast<float4*>(dst + (dsc.soff & 0xffffff)) =
                load4<T, VEC>(src + dsc.goff, dsc.soff >> 24);
        }
    };

    // ---- prologue: first source plane
    const int p_first = d0 - 2 * PD, p_last = d1 - 1 + 2 * PD;
    if (p_first >= 0 && p_first < D) load_z_now(p_first);
    if (KD == 1) load_x_now(p_first, 0);
    __syncthreads();

    for (int p = p_first; p <= p_last; ++p) {
        // -------- prefetch (global loads stay in flight during the K phase)
        float4 zr[MAXZ], xr[MAXX];
        const bool have_z = KD > 1 && p + 1 <= p_last && p + 1 >= 0 && p + 1 < D;
        const int xq = p - PD;
        const bool have_x = KD > 1 && xq >= 0 && xq < D && xq >= d0 - PD && xq <= d1 - 1 + PD;
        if (have_z) fetch_z(zr, p + 1);
        if (have_x) fetch_x(xr, xq);

        // -------- K phase: source plane p feeds t1 planes p+PD-kd
        const bool s_ok = p >= 0 && p < D;
        const int qdone = p - PD;  // t1 plane completed by this step
        const bool q_need = qdone >= d0 - PD && qdone <= d1 - 1 + PD && qdone >= 0 && qdone < D;
#pragma unroll
        for (int r = 0; r < RK; ++r) {
            if (k_ok[r]) {
                if (s_ok) {
                    const float* sp = sbuf + (p & (NSB - 1)) * lay.plane_s + k_row[r] * pitch;
#pragma unroll
                    for (int kh = 0; kh < KH; ++kh) {
#pragma unroll
                        for (int j = 0; j < SCH; ++j) {
                            float sv[16];
                            load_window(sp + (j * RS + kh) * pitch, k_strip[r], sv);
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
                                    for (int v = 0; v < V; ++v)
                                        kacc[r][kd][v] = fmaf(sv[ORG + v + kw - PW], w[kd * KW + kw],
                                                              kacc[r][kd][v]);
                        }
                    }
                }
                if (q_need) {
                    const int w0 = V * k_strip[r];
                    float tv[V];
#pragma unroll
                    for (int v = 0; v < V; ++v) tv[v] = (w0 + v < W) ? kacc[r][KD - 1][v] : 0.0f;
                    store_strip(t1ring + slot_of(qdone) * lay.plane_t + k_row[r] * pitch, k_strip[r], tv);
                    const int h = h0 - PH + k_row[r];
                    if (qdone >= d0 && qdone < d1 && k_row[r] >= PH && k_row[r] < PH + TH)
                        store_strip_global<T, VEC>(tg + (long long)qdone * HW + (long long)h * W, w0, W, tv);
                }
            }
            // rotate the running sums: slot kd now stands for plane (p+1)+PD-kd
#pragma unroll
            for (int kd = KD - 1; kd > 0; --kd)
#pragma unroll
                for (int v = 0; v < V; ++v) kacc[r][kd][v] = kacc[r][kd - 1][v];
#pragma unroll
            for (int v = 0; v < V; ++v) kacc[r][0][v] = 0.0f;
        }

        // -------- stage the prefetched planes
        if (have_z) stage_z(zr, p + 1);
        if (have_x) stage_x(xr, slot_of(xq));
        __syncthreads();

        // -------- A phase: output plane d
        const int d = p - 2 * PD;
        if (d < d0 || d >= d1) continue;
#pragma unroll
        for (int r = 0; r < RA; ++r) {
            if (!a_ok[r]) continue;
            const int hrow = h0 + a_row[r], w0 = V * a_strip[r];
            float zv[SCH][V];
#pragma unroll
            for (int j = 0; j < SCH; ++j)
                load_strip_global<T, VEC>(zg + j * SP + (long long)d * HW + (long long)hrow * W, w0, W, zv[j]);
            float an[SCH][V], ad[SCH][V];
#pragma unroll
            for (int j = 0; j < SCH; ++j)
#pragma unroll
                for (int v = 0; v < V; ++v) { an[j][v] = P.eps; ad[j][v] = P.eps; }
#pragma unroll
            for (int kd = 0; kd < KD; ++kd) {
                const int q = d + PD - kd;
                if (q < 0 || q >= D) continue;
                const int slot = slot_of(q);
#pragma unroll
                for (int kh = 0; kh < KH; ++kh) {
                    const int rr = a_row[r] + PH + PH - kh;  // ring row of h + PH - kh
                    float xv[16], tv[16];
                    load_window(xring + slot * lay.plane_t + rr * pitch, a_strip[r], xv);
                    load_window(t1ring + slot * lay.plane_t + rr * pitch, a_strip[r], tv);
#pragma unroll
                    for (int kw = 0; kw < KW; ++kw) {
                        const float4 w4 = *reinterpret_cast<const float4*>(
                            wA + ((kd * KH + kh) * KW + kw) * SCH);
                        const float wj[SCH] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
                        for (int j = 0; j < SCH; ++j)
#pragma unroll
                            for (int v = 0; v < V; ++v) {
                                an[j][v] = fmaf(xv[ORG + v + PW - kw], wj[j], an[j][v]);
                                ad[j][v] = fmaf(tv[ORG + v + PW - kw], wj[j], ad[j][v]);
                            }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < SCH; ++j) {
                float ov[V];
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    float s = zv[j][v] + bj[j];
                    if (P.relu) s = fmaxf(s, 0.0f);
                    ov[v] = __fdividef(s * an[j][v], ad[j][v]);
                }
                store_strip_global<T, VEC>(og + j * SP + (long long)d * HW + (long long)hrow * W, w0, W, ov);
            }
        }
    }
}

}  // namespace dw4
}  // namespace ndc
