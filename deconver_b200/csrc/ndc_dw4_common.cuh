// Shared pieces of the tiled depthwise kernels (m = 1, sc = 4).
//
// Work decomposition.  One CTA owns one (sample, group) pair, a band of TH rows spanning the
// full width W, and a chunk of DC planes, and marches through the chunk plane by plane.
// Planes live in shared memory as float32 rows of `pitch = 8*NS + 8` floats, NS = ceil(W/8)
// strips of 8 voxels; shared column c holds w = c - 4, so rows are 16-byte aligned and the
// four columns on either side are the zero padding of the volume.  Within a row the 16-byte
// quads are XOR-swizzled (`swz`) so that a quarter-warp of consecutive strips reads eight
// distinct bank groups.
//
// A thread's unit of work is a strip: 8 consecutive voxels of one row.  The 8 + 2*pad
// inputs a strip needs are read as four aligned quads (16 floats) covering w0-4 .. w0+11.
#pragma once

#include "ndc_common.cuh"

namespace ndc {
namespace dw4 {

constexpr int V = 8;     // voxels per strip
constexpr int SCH = 4;   // source channels per group
constexpr int ORG = 4;   // shared column of w = 0

// Host-side tiling decision for one geometry.
struct Tiling {
    int NS;     // strips per row
    int pitch;  // floats per shared-memory row
    int TH;     // rows per band
    int nth;    // bands along H
    int DC;     // planes per chunk
    int ndc;    // chunks along D
    int vec;    // rows of the global tensors are 16-byte aligned: vector loads and stores
};

__device__ __forceinline__ int swz(int quad) { return quad ^ ((quad >> 3) & 1); }

// Float offset, within a row, of the quad that holds shared column `col` (col % 4 == 0).
__device__ __forceinline__ int quad_off(int col) { return swz(col >> 2) << 2; }

// The 16 floats w0-4 .. w0+11 of a row (w0 = 8*strip), as four swizzled quads.
__device__ __forceinline__ void load_window(const float* row, int strip, float (&v)[16]) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 t = *reinterpret_cast<const float4*>(row + (swz(2 * strip + q) << 2));
        v[4 * q + 0] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
}

// Store the 8 voxels of a strip into a shared row.
__device__ __forceinline__ void store_strip(float* row, int strip, const float (&v)[V]) {
    *reinterpret_cast<float4*>(row + (swz(2 * strip + 1) << 2)) = make_float4(v[0], v[1], v[2], v[3]);
    *reinterpret_cast<float4*>(row + (swz(2 * strip + 2) << 2)) = make_float4(v[4], v[5], v[6], v[7]);
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

// Load / store the 8 voxels of a strip of a global row; elements at w >= W are 0 / skipped.
template <typename T, bool VEC>
__device__ __forceinline__ void load_strip_global(const T* row, int w0, int W, float (&v)[V]) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int w = w0 + 4 * q, n = W - w;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (n > 0) t = load4<T, VEC>(row + w, n < 4 ? n : 4);
        v[4 * q + 0] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
}
template <typename T, bool VEC>
__device__ __forceinline__ void store_strip_global(T* row, int w0, int W, const float (&v)[V]) {
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int w = w0 + 4 * q, n = W - w;
        if (n > 0)
            store4<T, VEC>(row + w, n < 4 ? n : 4,
                           make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
    }
}

// Plane loader.  A plane region of `rows` rows is cut into chunks of 4 consecutive elements;
// chunk -> (row, quad) decoding is done once per CTA into a descriptor table in shared
// memory: .x = element offset inside the plane (or -1 for a row outside the volume, which
// stays zero), .y = float offset inside the shared plane | (valid elements << 24).
struct ChunkDesc { int goff, soff; };

__device__ __forceinline__ void build_descs(ChunkDesc* tab, int channels, int rows, int NS,
                                            int pitch, int h_first, int H, int W, long long SP,
                                            int nthreads) {
    const int per_row = 2 * NS;
    const int total = channels * rows * per_row;
    for (int id = threadIdx.x; id < total; id += nthreads) {
        const int c4 = id % per_row;
        const int t = id / per_row;
        const int r = t % rows, ch = t / rows;
        const int h = h_first + r, w = 4 * c4;
        ChunkDesc d;
        const int n = W - w;
        if (h < 0 || h >= H || n <= 0) {
            d.goff = -1; d.soff = 0;
        } else {
            d.goff = (int)(ch * SP) + h * W + w;
            d.soff = ((ch * rows + r) * pitch + quad_off(w + ORG)) | ((n < 4 ? n : 4) << 24);
        }
        tab[id] = d;
    }
}

}  // namespace dw4
}  // namespace ndc
