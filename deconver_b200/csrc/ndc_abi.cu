// C-ABI entry points of libndc_b200.so: validation, dispatch, status codes.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "ndc_b200.h"
#include "ndc_common.cuh"
#include "ndc_generic.cuh"
#define NDC_DW4_EXTERN   // the tiled kernels are compiled in ndc_dw4_inst.cu
#include "ndc_dw4_host.cuh"

namespace {

thread_local char g_err[512] = "";

int fail(int status, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

int cuda_fail(cudaError_t e, const char* what) {
    return fail(NDC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

constexpr int kMaxChannels = 16;  // per-group channel counts the kernels are sized for
constexpr int kMaxTaps = 343;

int validate(const NdcDesc* d) {
    if (!d) return fail(NDC_ERR_INVALID, "descriptor is NULL");
    if (d->flags & ~NDC_FLAG_FORCE_GENERIC)
        return fail(NDC_ERR_INVALID, "descriptor.flags has unknown bits set (0x%x)", d->flags);
    if (d->batch <= 0 || d->groups <= 0 || d->m <= 0 || d->sc <= 0)
        return fail(NDC_ERR_INVALID, "batch, groups, m and sc must be positive (got %d, %d, %d, %d)",
                    d->batch, d->groups, d->m, d->sc);
    if (d->D <= 0 || d->H <= 0 || d->W <= 0)
        return fail(NDC_ERR_INVALID, "spatial extents must be positive (got %d x %d x %d)", d->D,
                    d->H, d->W);
    if (d->kD <= 0 || d->kH <= 0 || d->kW <= 0 || !(d->kD & 1) || !(d->kH & 1) || !(d->kW & 1))
        return fail(NDC_ERR_INVALID, "kernel extents must be positive and odd (got %d x %d x %d)",
                    d->kD, d->kH, d->kW);
    if (d->dtype != NDC_F32 && d->dtype != NDC_BF16)
        return fail(NDC_ERR_INVALID, "dtype must be NDC_F32 or NDC_BF16 (got %d)", d->dtype);
    if (!(d->eps >= 0.0f)) return fail(NDC_ERR_INVALID, "eps must be non-negative");
    if (d->m > kMaxChannels || d->sc > kMaxChannels)
        return fail(NDC_ERR_UNSUPPORTED, "m and sc are limited to %d per group (got %d, %d)",
                    kMaxChannels, d->m, d->sc);
    if ((long long)d->kD * d->kH * d->kW > kMaxTaps)
        return fail(NDC_ERR_UNSUPPORTED, "kernels are limited to %d taps", kMaxTaps);
    return NDC_OK;
}

int check_ptr(const void* p, const char* name, int dtype) {
    if (!p) return fail(NDC_ERR_INVALID, "%s is NULL", name);
    const uintptr_t a = (uintptr_t)p;
    const uintptr_t need = dtype == NDC_BF16 ? 2 : 4;
    if (a % need) return fail(NDC_ERR_ALIGNMENT, "%s is not aligned to %d bytes", name, (int)need);
    return NDC_OK;
}

#define NDC_TRY(expr)                  \
    do {                               \
        int _st = (expr);              \
        if (_st != NDC_OK) return _st; \
    } while (0)

int path_of(const NdcDesc* d) {
    if (d->flags & NDC_FLAG_FORCE_GENERIC) return NDC_PATH_GENERIC;
    const ndc::Geo g = ndc::make_geo(*d, false);
    if (!ndc::dw4::covers(g)) return NDC_PATH_GENERIC;
    return ndc::dw4::rows_class(g) ? NDC_PATH_DEPTHWISE4_ROWS : NDC_PATH_DEPTHWISE4;
}

}  // namespace

// ---- measurement aid: register-only chains of fused multiply-adds ------------------------
namespace {

template <bool PACKED>
__global__ void __launch_bounds__(256) fma_chain_kernel(float* out, int iters, float a, float b) {
    constexpr int ILP = 8;   // independent chains per thread
    if (PACKED) {
        unsigned long long acc[ILP], av, bv;
        asm("mov.b64 %0, {%1, %1};" : "=l"(av) : "f"(a));
        asm("mov.b64 %0, {%1, %1};" : "=l"(bv) : "f"(b));
#pragma unroll
        for (int i = 0; i < ILP; ++i) {
            const float v = threadIdx.x * 0.001f + i;
            asm("mov.b64 %0, {%1, %1};" : "=l"(acc[i]) : "f"(v));
        }
        for (int it = 0; it < iters; ++it)
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int i = 0; i < ILP; ++i)
                    asm volatile("fma.rn.f32x2 %0, %0, %1, %2;" : "+l"(acc[i]) : "l"(av), "l"(bv));
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < ILP; ++i) {
            float lo, hi;
            asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(acc[i]));
            s += lo + hi;
        }
        out[blockIdx.x * blockDim.x + threadIdx.x] = s;
    } else {
        float acc[ILP];
#pragma unroll
        for (int i = 0; i < ILP; ++i) acc[i] = threadIdx.x * 0.001f + i;
        for (int it = 0; it < iters; ++it)
#pragma unroll
            for (int r = 0; r < 8; ++r)
#pragma unroll
                for (int i = 0; i < ILP; ++i) acc[i] = fmaf(acc[i], a, b);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < ILP; ++i) s += acc[i];
        out[blockIdx.x * blockDim.x + threadIdx.x] = s;
    }
}

}  // namespace

extern "C" {

int ndc_version(void) { return NDC_B200_VERSION; }

const char* ndc_last_error(void) { return g_err; }

const char* ndc_status_string(int status) {
    switch (status) {
        case NDC_OK: return "ok";
        case NDC_ERR_INVALID: return "invalid argument";
        case NDC_ERR_UNSUPPORTED: return "unsupported geometry";
        case NDC_ERR_WORKSPACE: return "workspace missing, too small or misaligned";
        case NDC_ERR_CUDA: return "CUDA error";
        case NDC_ERR_ALIGNMENT: return "misaligned pointer";
        default: return "unknown status";
    }
}

uint64_t ndc_launch_count(void) {
    return (uint64_t)ndc::launch_counter().load(std::memory_order_relaxed);
}

int ndc_query(const NdcDesc* desc, int32_t* path) {
    NDC_TRY(validate(desc));
    if (path) *path = path_of(desc);
    return NDC_OK;
}

int ndc_fwd(const NdcDesc* desc, const void* x, const void* z, const float* h, const float* bias,
            void* out, void* t1, void* stream) {
    NDC_TRY(validate(desc));
    NDC_TRY(check_ptr(x, "x", desc->dtype));
    NDC_TRY(check_ptr(z, "z", desc->dtype));
    NDC_TRY(check_ptr(h, "h", NDC_F32));
    NDC_TRY(check_ptr(out, "out", desc->dtype));
    NDC_TRY(check_ptr(t1, "t1", desc->dtype));
    if (bias) NDC_TRY(check_ptr(bias, "bias", NDC_F32));
    const ndc::Geo g = ndc::make_geo(*desc, bias != nullptr);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    typedef __nv_bfloat16 bf16;
    if (path_of(desc) != NDC_PATH_GENERIC) {
        bool handled = false;
        if (desc->dtype == NDC_F32)
            e = ndc::dw4::forward<float>(g, (const float*)x, (const float*)z, h, bias, (float*)out,
                                         (float*)t1, desc->dtype, st, handled);
        else
            e = ndc::dw4::forward<bf16>(g, (const bf16*)x, (const bf16*)z, h, bias, (bf16*)out,
                                        (bf16*)t1, desc->dtype, st, handled);
        if (e != cudaSuccess) return cuda_fail(e, "ndc_fwd (depthwise) launch");
        if (handled) return NDC_OK;
    }
    if (desc->dtype == NDC_F32)
        e = ndc::generic::forward<float>(g, (const float*)x, (const float*)z, h, bias, (float*)out,
                                         (float*)t1, st);
    else
        e = ndc::generic::forward<bf16>(g, (const bf16*)x, (const bf16*)z, h, bias, (bf16*)out,
                                        (bf16*)t1, st);
    if (e != cudaSuccess) return cuda_fail(e, "ndc_fwd launch");
    return NDC_OK;
}

size_t ndc_bwd_workspace_bytes(const NdcDesc* desc) {
    if (validate(desc) != NDC_OK) return 0;
    const ndc::Geo g = ndc::make_geo(*desc, false);
    if (path_of(desc) != NDC_PATH_GENERIC) {
        ndc::dw4::BwdPlan p;
        if (ndc::dw4::plan_bwd_any(g, p)) return p.bytes;
    }
    return ndc::generic::bwd_scratch(g).bytes;
}

int ndc_bwd(const NdcDesc* desc, const void* x, const void* z, const void* t1, const float* h,
            const float* bias, const void* gout, void* gx, void* gz, float* gh, float* gb,
            void* workspace, size_t workspace_bytes, void* stream) {
    NDC_TRY(validate(desc));
    NDC_TRY(check_ptr(x, "x", desc->dtype));
    NDC_TRY(check_ptr(z, "z", desc->dtype));
    NDC_TRY(check_ptr(t1, "t1", desc->dtype));
    NDC_TRY(check_ptr(h, "h", NDC_F32));
    NDC_TRY(check_ptr(gout, "gout", desc->dtype));
    if (bias) NDC_TRY(check_ptr(bias, "bias", NDC_F32));
    if (gx) NDC_TRY(check_ptr(gx, "gx", desc->dtype));
    if (gz) NDC_TRY(check_ptr(gz, "gz", desc->dtype));
    if (gh) NDC_TRY(check_ptr(gh, "gh", NDC_F32));
    if (gb) NDC_TRY(check_ptr(gb, "gb", NDC_F32));
    if (gb && !gz) return fail(NDC_ERR_INVALID, "gb needs gz: pass a gz buffer when gb is wanted");
    if (!gx && !gz && !gh) return NDC_OK;  // nothing wanted
    const size_t need = ndc_bwd_workspace_bytes(desc);
    if (!workspace || workspace_bytes < need)
        return fail(NDC_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need,
                    workspace ? workspace_bytes : (size_t)0);
    if ((uintptr_t)workspace % 256)
        return fail(NDC_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    const ndc::Geo g = ndc::make_geo(*desc, bias != nullptr);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (path_of(desc) != NDC_PATH_GENERIC) {
        ndc::dw4::BwdPlan p;
        if (ndc::dw4::plan_bwd_any(g, p)) {
            typedef __nv_bfloat16 bf16;
            if (desc->dtype == NDC_F32)
                e = ndc::dw4::backward<float>(g, p, (const float*)x, (const float*)z,
                                              (const float*)t1, h, bias, (const float*)gout,
                                              (float*)gx, (float*)gz, gh, gb, workspace,
                                              desc->dtype, st);
            else
                e = ndc::dw4::backward<bf16>(g, p, (const bf16*)x, (const bf16*)z, (const bf16*)t1,
                                             h, bias, (const bf16*)gout, (bf16*)gx, (bf16*)gz, gh,
                                             gb, workspace, desc->dtype, st);
            if (e != cudaSuccess) return cuda_fail(e, "ndc_bwd (depthwise) launch");
            return NDC_OK;
        }
    }
    if (desc->dtype == NDC_F32)
        e = ndc::generic::backward<float>(g, (const float*)x, (const float*)z, (const float*)t1, h,
                                          bias, (const float*)gout, (float*)gx, (float*)gz, gh, gb,
                                          workspace, st);
    else
        e = ndc::generic::backward<__nv_bfloat16>(
            g, (const __nv_bfloat16*)x, (const __nv_bfloat16*)z, (const __nv_bfloat16*)t1, h, bias,
            (const __nv_bfloat16*)gout, (__nv_bfloat16*)gx, (__nv_bfloat16*)gz, gh, gb, workspace,
            st);
    if (e != cudaSuccess) return cuda_fail(e, "ndc_bwd launch");
    return NDC_OK;
}

// Scratch of ndc_bwd_static.  In host code this name is only a stand-in for the symbol; the
// device address is looked up per device below and that pointer is what the kernels get.
static __device__ __align__(256) unsigned char g_static_workspace[NDC_STATIC_WORKSPACE_BYTES];

int ndc_bwd_static(const NdcDesc* desc, const void* x, const void* z, const void* t1,
                   const float* h, const float* bias, const void* gout, void* gx, void* gz,
                   float* gh, float* gb, void* stream) {
    NDC_TRY(validate(desc));
    const size_t need = ndc_bwd_workspace_bytes(desc);
    if (need > (size_t)NDC_STATIC_WORKSPACE_BYTES)
        return fail(NDC_ERR_WORKSPACE,
                    "ndc_bwd_static: this geometry needs %zu bytes of scratch, the built-in array "
                    "holds %zu; use ndc_bwd with a caller-provided workspace",
                    need, (size_t)NDC_STATIC_WORKSPACE_BYTES);
    // one address per device, found on first use with that device current
    constexpr int kMaxDevices = 64;
    static void* addr[kMaxDevices] = {};
    static std::mutex mu;
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return cuda_fail(e, "ndc_bwd_static: cudaGetDevice");
    if (dev < 0 || dev >= kMaxDevices)
        return fail(NDC_ERR_UNSUPPORTED, "ndc_bwd_static: device ordinal %d is not supported", dev);
    void* ws = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!addr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_workspace);
            if (e != cudaSuccess) return cuda_fail(e, "ndc_bwd_static: cudaGetSymbolAddress");
            addr[dev] = p;
        }
        ws = addr[dev];
    }
    return ndc_bwd(desc, x, z, t1, h, bias, gout, gx, gz, gh, gb, ws,
                   (size_t)NDC_STATIC_WORKSPACE_BYTES, stream);
}

int ndc_probe_fp32_fma(int32_t packed, int32_t iters, float* out, size_t out_elems,
                       uint64_t* fma_count, void* stream) {
    if (iters <= 0) return fail(NDC_ERR_INVALID, "ndc_probe_fp32_fma: iters must be positive");
    NDC_TRY(check_ptr(out, "out", NDC_F32));
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return cuda_fail(e, "ndc_probe_fp32_fma: device query");
    const int threads = 256, blocks = sms * 4;
    if (out_elems < (size_t)threads * blocks)
        return fail(NDC_ERR_WORKSPACE, "ndc_probe_fp32_fma: out must hold %d floats, %zu given",
                    threads * blocks, out_elems);
    cudaStream_t st = (cudaStream_t)stream;
    if (packed) fma_chain_kernel<true><<<blocks, threads, 0, st>>>(out, iters, 0.999f, 0.001f);
    else fma_chain_kernel<false><<<blocks, threads, 0, st>>>(out, iters, 0.999f, 0.001f);
    ndc::launched();
    e = cudaGetLastError();
    if (e != cudaSuccess) return cuda_fail(e, "ndc_probe_fp32_fma launch");
    // per thread: iters x 8 rounds x 8 chains, two lanes per packed instruction
    if (fma_count)
        *fma_count = (uint64_t)threads * blocks * (uint64_t)iters * 64u * (packed ? 2u : 1u);
    return NDC_OK;
}

int ndc_gconv(const NdcDesc* desc, const void* in, const float* h, const float* bias,
              int32_t adjoint, void* out, void* stream) {
    NDC_TRY(validate(desc));
    NDC_TRY(check_ptr(in, "in", desc->dtype));
    NDC_TRY(check_ptr(h, "h", NDC_F32));
    NDC_TRY(check_ptr(out, "out", desc->dtype));
    if (bias) NDC_TRY(check_ptr(bias, "bias", NDC_F32));
    const ndc::Geo g = ndc::make_geo(*desc, bias != nullptr);
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e;
    if (desc->dtype == NDC_F32)
        e = ndc::generic::gconv<float>(g, (const float*)in, h, bias, adjoint != 0, (float*)out, st);
    else
        e = ndc::generic::gconv<__nv_bfloat16>(g, (const __nv_bfloat16*)in, h, bias, adjoint != 0,
                                               (__nv_bfloat16*)out, st);
    if (e != cudaSuccess) return cuda_fail(e, "ndc_gconv launch");
    return NDC_OK;
}

}  // extern "C"
