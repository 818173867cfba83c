// Helpers shared by the per-slab kernels (instance norm, bias add / bias gradient): a
// (sample, channel) slab of a channels-first tensor is cut into `nsplit` parts, one CTA each, so
// that the grid fills the GPU even when batch x channels is small.
#pragma once

#include "ndc_common.cuh"

namespace ndc {
namespace slab {

constexpr int kNT = 256;          // threads per CTA
constexpr int kMaxSplit = 64;     // parts per slab, at most

template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    typedef float4 raw;
    __device__ static void unpack(const raw& r, float (&v)[4]) { v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
    __device__ static raw pack(const float (&v)[4]) { return make_float4(v[0], v[1], v[2], v[3]); }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    typedef uint4 raw;
    __device__ static void unpack(const raw& r, float (&v)[8]) {
        const unsigned w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static raw pack(const float (&v)[8]) {
        unsigned w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            w[i] = *reinterpret_cast<const unsigned*>(&p);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

// element range [begin, end) of part `part` of a slab of `sp` elements cut into `nsplit` parts
// whose boundaries are multiples of `align` elements
__device__ __forceinline__ void part_range(long long sp, int nsplit, int part, int align,
                                           long long& begin, long long& end) {
    const long long units = (sp + align - 1) / align;
    const long long per = (units + nsplit - 1) / nsplit;
    begin = min(sp, (long long)part * per * align);
    end = min(sp, (long long)(part + 1) * per * align);
}

// Fixed-order sum of two values over the CTA; valid in every thread afterwards.
__device__ __forceinline__ void cta_sum2(float& a, float& b, float* scratch) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, off);
        b += __shfl_xor_sync(0xffffffffu, b, off);
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    __syncthreads();
    if (lane == 0) { scratch[2 * warp] = a; scratch[2 * warp + 1] = b; }
    __syncthreads();
    a = 0.0f; b = 0.0f;
#pragma unroll
    for (int w = 0; w < kNT / 32; ++w) { a += scratch[2 * w]; b += scratch[2 * w + 1]; }
}


// parts per slab: enough CTAs for about four per multiprocessor, parts of at least 4096 elements
inline int choose_split(long long slabs, long long sp) {
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) {
        (void)cudaGetLastError();
        sms = 148;
    }
    long long want = (4LL * sms + slabs - 1) / slabs;
    const long long most = sp / 4096 > 0 ? sp / 4096 : 1;
    if (want > most) want = most;
    if (want > kMaxSplit) want = kMaxSplit;
    return (int)(want < 1 ? 1 : want);
}

}  // namespace slab
}  // namespace ndc
