// Shared pieces of the tiled depthwise kernels (m = 1, sc = 4).
//
// Work decomposition.  One CTA owns one (sample, group) pair, a band of TH rows spanning the
// full width W, and a chunk of DC planes, and marches through the chunk plane by plane.
// Planes live in shared memory as float32 rows of `pitch` floats, in one of two layouts:
//
//   ring rows (single-channel planes read by A-type sweeps: adjoint taps, many accumulators,
//   strips of 4 voxels): shared column c holds w = c - (4 + PW), PW = kW/2.  With that shift
//   the window of a strip that starts at a multiple of 4 begins on a 16-byte quad and is two
//   quads long.  Consecutive lanes read consecutive quads, so these rows stay linear.
//
//   source rows (4-channel planes read by K-type sweeps: running sums along depth, strips of
//   8 voxels): shared column c holds w = c - 4, so 16-byte chunks from HBM land on whole quads
//   (vector stores, cp.async); a strip's window is the four quads 2k .. 2k+3.  The eight lanes
//   of a quarter-warp are two quads apart, so quads are XOR-swizzled (`phys_quad<true>`) to hit
//   eight distinct bank groups.
#pragma once

#include "ndc_common.cuh"

namespace ndc {
namespace dw4 {

constexpr int SCH = 4;   // source channels per group
constexpr int VA = 4;    // voxels per strip, A-type sweeps
constexpr int VK = 8;    // voxels per strip, K-type sweeps

// Host-side tiling decision for one geometry.
struct Tiling {
    int NQ;     // quads (4 voxels) per row = ceil(W/4)
    int pitch;  // floats per shared-memory row
    int TH;     // rows per band
    int nth;    // bands along H
    int DC;     // planes per chunk
    int ndc;    // chunks along D
};

// floats per shared row: the data quads, one quad of left margin, and enough on the right for
// the last strip's window (3 quads past an 8-strip start, rounded to an even quad count)
__host__ __device__ constexpr int row_pitch(int W) {
    return 4 * (2 * (((W + 3) / 4 + 1) / 2) + 4);
}

template <bool SWZ> __device__ __forceinline__ int phys_quad(int quad) {
    return SWZ ? (quad ^ ((quad >> 3) & 1)) : quad;
}

// NQW consecutive quads of a shared row starting at quad `first`.
template <int NQW, bool SWZ>
__device__ __forceinline__ void load_window(const float* row, int first, float (&v)[4 * NQW]) {
#pragma unroll
    for (int q = 0; q < NQW; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(row + (phys_quad<SWZ>(first + q) << 2));
        v[4 * q + 0] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
}

// Shared float offset (within a row) of column `col`.
template <bool SWZ> __device__ __forceinline__ int col_off(int col) {
    return (phys_quad<SWZ>(col >> 2) << 2) | (col & 3);
}

// Store N voxels starting at volume column w0 into a shared row (scalar: the column shift
// makes these stores unaligned).
template <int N, int PW, bool SWZ>
__device__ __forceinline__ void store_strip(float* row, int w0, const float (&v)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) row[col_off<SWZ>(w0 + 4 + PW + i)] = v[i];
}

// Four consecutive elements of a global row, converted to float32.  `n` of them are inside
// the row (1..4); with VEC the address is 16-byte (8-byte for bfloat16) aligned and n == 4.
template <typename T, bool VEC>
__device__ __forceinline__ float4 load4(const T* p, int n);

template <>
__device__ __forceinline__ float4 load4<float, true>(const float* p, int) {
    return __ldg(reinterpret_cast<const float4*>(p));
}
template <>
__device__ __forceinline__ float4 load4<float, false>(const float* p, int n) {
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    r.x = __ldg(p);
    if (n > 1) r.y = __ldg(p + 1);
    if (n > 2) r.z = __ldg(p + 2);
    if (n > 3) r.w = __ldg(p + 3);
    return r;
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16, true>(const __nv_bfloat16* p, int) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    const float2 fa = __bfloat1622float2(a), fb = __bfloat1622float2(b);
    return make_float4(fa.x, fa.y, fb.x, fb.y);
}
template <>
__device__ __forceinline__ float4 load4<__nv_bfloat16, false>(const __nv_bfloat16* p, int n) {
    float4 r = make_float4(0.f, 0.f, 0.f, 0.f);
    r.x = __bfloat162float(p[0]);
    if (n > 1) r.y = __bfloat162float(p[1]);
    if (n > 2) r.z = __bfloat162float(p[2]);
    if (n > 3) r.w = __bfloat162float(p[3]);
    return r;
}

// The same four elements as they sit in memory.  Loads that are issued early (prefetch, top of
// an item) keep the raw form and convert where the values are used: a conversion right after
// the load would make the warp wait for the memory there.
template <typename T> struct Raw4;
template <> struct Raw4<float> { float4 v; };
template <> struct Raw4<__nv_bfloat16> { uint2 v; };

__device__ __forceinline__ float4 to_float4(const Raw4<float>& r) { return r.v; }
__device__ __forceinline__ float4 to_float4(const Raw4<__nv_bfloat16>& r) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.v.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// An opaque use of a raw strip: what is computed from it afterwards cannot be scheduled before
// this point.
__device__ __forceinline__ void hold_raw(Raw4<float>& r) {
    asm volatile("" : "+f"(r.v.x), "+f"(r.v.y), "+f"(r.v.z), "+f"(r.v.w));
}
__device__ __forceinline__ void hold_raw(Raw4<__nv_bfloat16>& r) {
    asm volatile("" : "+r"(r.v.x), "+r"(r.v.y));
}

template <typename T, bool VEC>
__device__ __forceinline__ Raw4<T> load4_raw(const T* p, int n);
template <>
__device__ __forceinline__ Raw4<float> load4_raw<float, true>(const float* p, int) {
    Raw4<float> r; r.v = __ldg(reinterpret_cast<const float4*>(p)); return r;
}
template <>
__device__ __forceinline__ Raw4<float> load4_raw<float, false>(const float* p, int n) {
    Raw4<float> r; r.v = load4<float, false>(p, n); return r;
}
template <>
__device__ __forceinline__ Raw4<__nv_bfloat16> load4_raw<__nv_bfloat16, true>(const __nv_bfloat16* p, int) {
    Raw4<__nv_bfloat16> r; r.v = __ldg(reinterpret_cast<const uint2*>(p)); return r;
}
template <>
__device__ __forceinline__ Raw4<__nv_bfloat16> load4_raw<__nv_bfloat16, false>(const __nv_bfloat16* p, int n) {
    const unsigned short* q = reinterpret_cast<const unsigned short*>(p);
    unsigned e0 = q[0], e1 = n > 1 ? q[1] : 0u, e2 = n > 2 ? q[2] : 0u, e3 = n > 3 ? q[3] : 0u;
    Raw4<__nv_bfloat16> r; r.v = make_uint2(e0 | (e1 << 16), e2 | (e3 << 16)); return r;
}
// four voxels of a global row from column w0 (zero past the end of the row), raw
template <typename T, bool VEC>
__device__ __forceinline__ Raw4<T> load_strip_raw(const T* row, int w0, int W) {
    const int n = W - w0;
    if (n > 0) return load4_raw<T, VEC>(row + w0, n < 4 ? n : 4);
    Raw4<T> r; r.v = {}; return r;
}
template <typename T>
__device__ __forceinline__ void raw_to_array(const Raw4<T>& r, float (&v)[4]) {
    const float4 t = to_float4(r);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}

template <typename T, bool VEC>
__device__ __forceinline__ void store4(T* p, int n, float4 v);

template <>
__device__ __forceinline__ void store4<float, true>(float* p, int, float4 v) {
    *reinterpret_cast<float4*>(p) = v;
}
template <>
__device__ __forceinline__ void store4<float, false>(float* p, int n, float4 v) {
    p[0] = v.x;
    if (n > 1) p[1] = v.y;
    if (n > 2) p[2] = v.z;
    if (n > 3) p[3] = v.w;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16, true>(__nv_bfloat16* p, int, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const unsigned*>(&a);
    raw.y = *reinterpret_cast<const unsigned*>(&b);
    *reinterpret_cast<uint2*>(p) = raw;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16, false>(__nv_bfloat16* p, int n, float4 v) {
    p[0] = __float2bfloat16_rn(v.x);
    if (n > 1) p[1] = __float2bfloat16_rn(v.y);
    if (n > 2) p[2] = __float2bfloat16_rn(v.z);
    if (n > 3) p[3] = __float2bfloat16_rn(v.w);
}

// Load / store N (a multiple of 4) voxels of a global row from column w0; elements at
// w >= W read as 0 / are skipped.
template <typename T, bool VEC, int N>
__device__ __forceinline__ void load_strip_global(const T* row, int w0, int W, float (&v)[N]) {
#pragma unroll
    for (int q = 0; q < N / 4; ++q) {
        const int w = w0 + 4 * q, n = W - w;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n > 0) t = load4<T, VEC>(row + w, n < 4 ? n : 4);
        v[4 * q + 0] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
}
template <typename T, bool VEC, int N>
__device__ __forceinline__ void store_strip_global(T* row, int w0, int W, const float (&v)[N]) {
#pragma unroll
    for (int q = 0; q < N / 4; ++q) {
        const int w = w0 + 4 * q, n = W - w;
        if (n > 0)
            store4<T, VEC>(row + w, n < 4 ? n : 4,
                           make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
    }
}

// Global-memory strides (in elements) of the slab a CTA works on.
//   Volumes (and images handled band by band): channel-major planes of H x W, one (sample,
//   group) pair per slab: plane stride H*W, channel stride D*H*W, row stride W.
//   Rows mode (kernel K x 1 x K, see the host side): a 2-D batch is addressed as ONE volume per
//   group whose planes are the image rows and whose plane rows are the images of the batch
//   (kernel height 1: they never mix).  Plane stride W, channel stride D*W (one image), row
//   stride = one sample (C channels of x-like tensors, 4*C of z-like ones).  The CTA's band of
//   images is folded into its base pointers, so rows are counted from the band's first image.
template <bool ROWS>
struct SlabAddr {
    long long plane, chan, row_x, row_z;
    __device__ __forceinline__ SlabAddr(int C, int D, int H, int W) {
        if (ROWS) {
            plane = W; chan = (long long)D * W;
            row_x = chan * C; row_z = row_x * SCH;
        } else {
            plane = (long long)H * W; chan = plane * D;
            row_x = W; row_z = W;
        }
    }
};

// Plane loader.  A plane region of `rows` rows is cut into chunks of 4 consecutive elements;
// chunk -> (channel, row, quad) decoding is done once per CTA into a descriptor table in
// shared memory: .goff = element offset inside the plane (or -1 for a row outside the
// volume, which stays zero); .soff = float offset of the shared ROW | (volume column << 16)
// | (valid elements << 26) | (channel << 29).
struct ChunkDesc { int goff, soff; };
__device__ __forceinline__ int desc_row(int soff) { return soff & 0xffff; }
__device__ __forceinline__ int desc_w(int soff) { return (soff >> 16) & 0x3ff; }
__device__ __forceinline__ int desc_n(int soff) { return (soff >> 26) & 7; }
__device__ __forceinline__ int desc_ch(int soff) { return (soff >> 29) & 3; }

__device__ __forceinline__ void build_descs(ChunkDesc* tab, int channels, int rows, int NQ,
                                            int pitch, int h_first, int H, int W, long long SP,
                                            long long row_stride, int nthreads) {
    const int total = channels * rows * NQ;
    for (int id = threadIdx.x; id < total; id += nthreads) {
        const int c4 = id % NQ;
        const int t = id / NQ;
        const int r = t % rows, ch = t / rows;
        const int h = h_first + r, w = 4 * c4;
        ChunkDesc d;
        const int n = W - w;
        if (h < 0 || h >= H) {
            d.goff = -1; d.soff = 0;
        } else {
            d.goff = (int)(ch * SP + h * row_stride) + w;
            d.soff = ((ch * rows + r) * pitch) | (w << 16) | ((n < 4 ? n : 4) << 26) | (ch << 29);
        }
        tab[id] = d;
    }
}

// Write a chunk's 4 values into its shared row at columns w+4+PW .. (unaligned by PW).
template <int PW, bool SWZ>
__device__ __forceinline__ void stage_chunk(float* plane, int soff, float4 v) {
    float* row = plane + desc_row(soff);
    const int c = desc_w(soff) + 4 + PW;
    row[col_off<SWZ>(c)] = v.x;
    row[col_off<SWZ>(c + 1)] = v.y;
    row[col_off<SWZ>(c + 2)] = v.z;
    row[col_off<SWZ>(c + 3)] = v.w;
}

// ---- per-thread strip staging with cp.async ---------------------------------------------
// A thread that walks over items (4-voxel strips) needs, for each item, a few strips of
// per-voxel operands straight from HBM (z, upstream gradient, ...).  Loading them when the
// item starts exposes the full memory latency at low occupancy, so the strips of the NEXT
// item are requested with cp.async while the current item is computed.  Each thread owns two
// slots (double buffer) of NSTR strips; slot layout [buffer][strip][thread] in 16-byte (8-byte
// for bfloat16) units, so the read-back is conflict free.  Without VEC (rows not 16-byte
// aligned) the strips are loaded directly instead.
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

template <typename T, bool VEC, int NSTR, int NT>
struct StripFetcher {
    static constexpr int kUnit = sizeof(T) == 4 ? 16 : 8;                    // bytes per strip
    static constexpr int kFloats = VEC ? 2 * NSTR * NT * kUnit / 4 : 0;      // shared floats needed
    char* base;
    int buf;
    __device__ __forceinline__ StripFetcher(float* smem_area) : base(reinterpret_cast<char*>(smem_area)), buf(0) {}
    __device__ __forceinline__ char* slot(int b, int s) const {
        return base + ((size_t)(b * NSTR + s) * NT + threadIdx.x) * kUnit;
    }
    // request the strips at src[0..NSTR) for the item after the current one
    __device__ __forceinline__ void request(const T* const (&src)[NSTR]) {
        if (!VEC) return;
        buf ^= 1;
#pragma unroll
        for (int s = 0; s < NSTR; ++s) {
            const unsigned dst = (unsigned)__cvta_generic_to_shared(slot(buf, s));
            if (kUnit == 16)
                asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src[s]) : "memory");
            else
                asm volatile("cp.async.ca.shared.global [%0], [%1], 8;\n" ::"r"(dst), "l"(src[s]) : "memory");
        }
        cp_async_commit();
    }
    // strips of the current item: the ones requested last (VEC) or loaded now (otherwise)
    __device__ __forceinline__ void receive(const T* const (&src)[NSTR], int w0, int W, float (&v)[NSTR][VA]) {
        if (VEC) {
            cp_async_wait_all();
#pragma unroll
            for (int s = 0; s < NSTR; ++s) {
                if (kUnit == 16) {
                    const float4 t = *reinterpret_cast<const float4*>(slot(buf, s));
                    v[s][0] = t.x; v[s][1] = t.y; v[s][2] = t.z; v[s][3] = t.w;
                } else {
                    const uint2 raw = *reinterpret_cast<const uint2*>(slot(buf, s));
                    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
                    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
                    v[s][0] = a.x; v[s][1] = a.y; v[s][2] = b.x; v[s][3] = b.y;
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < NSTR; ++s) load_strip_global<T, false, VA>(src[s] - w0, w0, W, v[s]);
        }
    }
};

// Two float32 lanes in one 64-bit register, for `fma.rn.f32x2`: one issue slot for two
// fused multiply-adds, each rounded exactly like `fmaf`.  The sweeps pack two source channels
// of the same voxel into a pair, so filter weights (stored channel-minor) load as ready pairs
// and only the window value has to be duplicated.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(f32x2 p, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(p));
}
__device__ __forceinline__ void fma2(f32x2& acc, f32x2 a, f32x2 b) {
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(acc) : "l"(a), "l"(b));
}
// lane `hi` (0 or 1, a compile-time value after unrolling) of a pair
__device__ __forceinline__ float lane_of(f32x2 p, int hi) {
    float lo, up;
    unpack2(p, lo, up);
    return hi ? up : lo;
}

// One filter row (KW taps) of an adjoint sweep over two single-channel planes at once:
// an[jp][v] += x[w0 + v + PW - kw] * hA[kw][2jp .. 2jp+1], ad likewise from t.  `xrow`/`trow`
// are ring rows in the shifted layout, `quad` the strip's first window quad, `w_row` the KW x SCH
// weights of this (kd, kh), channel-minor.
template <int KW, int NQA>
__device__ __forceinline__ void adjoint_row2(const float* xrow, const float* trow, int quad,
                                             const float* w_row, f32x2 (&an)[SCH / 2][VA],
                                             f32x2 (&ad)[SCH / 2][VA]) {
    constexpr int PW = KW / 2;
    float xv[4 * NQA], tv[4 * NQA];
    load_window<NQA, false>(xrow, quad, xv);
    load_window<NQA, false>(trow, quad, tv);
    f32x2 x2[VA + KW - 1], t2[VA + KW - 1];
#pragma unroll
    for (int i = 0; i < VA + KW - 1; ++i) {
        x2[i] = pack2(xv[i], xv[i]);
        t2[i] = pack2(tv[i], tv[i]);
    }
#pragma unroll
    for (int kw = 0; kw < KW; ++kw) {
        const float4 w4 = *reinterpret_cast<const float4*>(w_row + kw * SCH);
        const f32x2 wp[SCH / 2] = {pack2(w4.x, w4.y), pack2(w4.z, w4.w)};
#pragma unroll
        for (int jp = 0; jp < SCH / 2; ++jp)
#pragma unroll
            for (int v = 0; v < VA; ++v) {
                fma2(an[jp][v], x2[v + 2 * PW - kw], wp[jp]);
                fma2(ad[jp][v], t2[v + 2 * PW - kw], wp[jp]);
            }
    }
}

// x / (y) with one reciprocal approximation: |relative error| <= 2 ulp, y > 0 and normal.
__device__ __forceinline__ float fast_div(float x, float y) { return __fdividef(x, y); }

}  // namespace dw4
}  // namespace ndc
