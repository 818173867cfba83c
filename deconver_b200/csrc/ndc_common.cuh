// Shared device/host helpers of the NDC kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ndc_b200.h"

#include <atomic>

namespace ndc {

// Process-wide count of kernel launches, for ndc_launch_count().
inline std::atomic<unsigned long long>& launch_counter() {
    static std::atomic<unsigned long long> n{0};
    return n;
}
// Call once after every kernel launch.
inline void launched(int n = 1) { launch_counter().fetch_add(n, std::memory_order_relaxed); }

// Geometry handed to every kernel by value.
struct Geo {
    int B, G, m, sc;
    int D, H, W;
    int kD, kH, kW;
    int pD, pH, pW;
    int KT;        // taps
    long long SP;  // D*H*W
    float eps;
    int relu;      // rectify the source on load
    int has_bias;
};

inline Geo make_geo(const NdcDesc& d, bool has_bias) {
    Geo g;
    g.B = d.batch; g.G = d.groups; g.m = d.m; g.sc = d.sc;
    g.D = d.D; g.H = d.H; g.W = d.W;
    g.kD = d.kD; g.kH = d.kH; g.kW = d.kW;
    g.pD = d.kD / 2; g.pH = d.kH / 2; g.pW = d.kW / 2;
    g.KT = d.kD * d.kH * d.kW;
    g.SP = (long long)d.D * d.H * d.W;
    g.eps = d.eps;
    g.relu = d.relu_input ? 1 : 0;
    g.has_bias = has_bias ? 1 : 0;
    return g;
}

// Storage <-> float32.  All arithmetic is float32 whatever the storage type.
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// Deterministic block-wide sum: shuffle tree inside each warp, then a fixed-order tree over
// the warp partials in shared memory.  Every thread of the block must call it; the result is
// valid in thread 0.  `scratch` holds at least blockDim.x / 32 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarp = (blockDim.x + 31) >> 5;
    __syncthreads();  // scratch may still be read by a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        v = lane < nwarp ? scratch[lane] : 0.0f;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) v += __shfl_down_sync(0xffffffffu, v, off);
    }
    return v;
}

}  // namespace ndc
