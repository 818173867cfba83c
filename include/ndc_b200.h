/*
 * ndc_b200 - nonnegative-deconvolution (NDC) source update for NVIDIA B200 (sm_100a).
 *
 * C ABI of the shared library `libndc_b200.so`.  Every entry point takes raw DEVICE pointers,
 * caller-allocated outputs and workspace, and an explicit CUDA stream; it returns a status
 * code, never throws and never aborts the process.  Nothing here depends on PyTorch.
 *
 * The update (per group g, with m = C/groups filter channels, sc source channels,
 * pad = k/2, all convolutions stride 1, zero padded, odd kernels):
 *
 *     K(u)[o,p] = sum_{i,tau} u[i, p + tau - pad] * h[o,i,tau]
 *     A(v)[i,p] = sum_{o,tau} v[o, p + pad - tau] * h[o,i,tau]          (A = K^T)
 *     s   = relu(z + bias)            (ReLU and bias optional, see NdcDesc)
 *     t1  = K(s)
 *     out = (s * (A(x) + eps)) / (A(t1) + eps)
 *
 * Tensor layout: contiguous, channels first.
 *     x, t1, gx            (batch, groups*m,  D, H, W)
 *     z, out, gout, gz     (batch, groups*sc, D, H, W)
 *     h, gh                (groups*m, sc, kD, kH, kW)      always float32
 *     bias, gb             (groups*sc)                     always float32
 * 1-D and 2-D problems set the leading extents (and kernel extents) to 1.
 * The large tensors are stored as float32 or bfloat16 (NdcDesc.dtype); all arithmetic and
 * every reduction is float32.
 *
 * Each declaration cites the interface of the reference project (pashtari/deconver, paths
 * within that project) that it replaces.
 */
#ifndef NDC_B200_H
#define NDC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NDC_B200_VERSION 1

enum NdcDType { NDC_F32 = 0, NDC_BF16 = 1 };

enum NdcStatus {
    NDC_OK = 0,
    NDC_ERR_INVALID = 1,     /* null pointer, non-positive extent, even kernel, bad dtype   */
    NDC_ERR_UNSUPPORTED = 2, /* geometry outside what the kernels cover                     */
    NDC_ERR_WORKSPACE = 3,   /* workspace missing, too small or misaligned                  */
    NDC_ERR_CUDA = 4,        /* a CUDA runtime call or a launch failed                      */
    NDC_ERR_ALIGNMENT = 5    /* a tensor pointer is not aligned to its element size         */
};

enum NdcFlags {
    NDC_FLAG_FORCE_GENERIC = 1 /* run the generic kernels even where the tiled ones apply    */
};

/* Which family of kernels a geometry runs on (informational; results are the same). */
enum NdcPath {
    NDC_PATH_GENERIC = 0, /* any m, sc <= 16, any odd kernel with <= 343 taps                */
    NDC_PATH_DEPTHWISE4 = 1, /* m = 1, sc = 4, kernel 3x3x3, 1x5x5 or 1x3x3: tiled, fused    */
    NDC_PATH_DEPTHWISE4_ROWS = 2 /* the same kernels marching down the rows of 2-D images:
                                    5x5 or 3x3, up to 512 columns, at least 8 rows, enough
                                    images in the batch to fill a 32-thread CTA             */
};

/*
 * Geometry of one update.  Mirrors the arguments of the reference's
 * `DeconvUpdate.forward(ctx, x, z, h, bias, groups, m, sc, eps, relu_input)`
 * (deconver/deconvolution/functional.py:105-106) plus the launch geometry its wrappers
 * derive from the tensors (deconver/deconvolution/kernels.py:687-725).
 */
typedef struct NdcDesc {
    int32_t batch;
    int32_t groups;
    int32_t m;          /* filter (input) channels per group                               */
    int32_t sc;         /* source channels per group                                       */
    int32_t D, H, W;    /* spatial extent; missing leading dimensions are 1                */
    int32_t kD, kH, kW; /* kernel extent, all odd; missing leading dimensions are 1        */
    float eps;          /* added to numerator and denominator                              */
    int32_t relu_input; /* 1: s = relu(z + bias) (first iteration); 0: s = z + bias        */
    int32_t dtype;      /* NdcDType of x, z, t1, out, gout, gx, gz                         */
    int32_t flags;      /* bitwise OR of NdcFlags; 0 for normal use                        */
} NdcDesc;

/* Library version (NDC_B200_VERSION of the build). */
int ndc_version(void);

/* Message of the last failure on the calling thread ("" if none).  Replaces the Python
 * exceptions of the reference's wrappers (deconver/deconvolution/kernels.py:715-716). */
const char *ndc_last_error(void);

/* Short name of a status code. */
const char *ndc_status_string(int status);

/* Number of kernel launches this library has issued in this process (all threads).  Lets a
 * caller verify that the CUDA path, and not some other path, did the work. */
uint64_t ndc_launch_count(void);

/*
 * Whether a geometry is covered, and by which kernel family.  Returns NDC_OK and writes an
 * NdcPath to *path, or NDC_ERR_INVALID / NDC_ERR_UNSUPPORTED.  Host-only; no CUDA call.
 * Replaces `kernels_supported` / `wgrad_supported` / `triton_available`
 * (deconver/deconvolution/kernels.py:114-163).
 */
int ndc_query(const NdcDesc *desc, int32_t *path);

/*
 * Forward of one update: writes `out` and `t1` (t1 is what backward needs, besides x and z).
 * `bias` may be NULL.  Replaces `kernels.gconv` + `kernels.deconv_fwd` as called by
 * `DeconvUpdate.forward` (deconver/deconvolution/functional.py:105-116;
 * deconver/deconvolution/kernels.py:728-788).
 */
int ndc_fwd(const NdcDesc *desc, const void *x, const void *z, const float *h,
            const float *bias, void *out, void *t1, void *stream);

/*
 * Bytes of scratch `ndc_bwd` needs for this geometry (0 on an invalid descriptor).  The
 * workspace must be 256-byte aligned device memory; its contents need not be initialised
 * and are undefined afterwards.
 */
size_t ndc_bwd_workspace_bytes(const NdcDesc *desc);

/*
 * Backward of one update.  Inputs: x, z, t1 (as written by ndc_fwd), h, bias (or NULL),
 * upstream gradient gout.  Outputs, each optional (NULL = not wanted):
 *     gx  gradient w.r.t. x
 *     gz  gradient w.r.t. z           (required if gb is wanted)
 *     gh  gradient w.r.t. h, float32, overwritten (not accumulated into)
 *     gb  gradient w.r.t. bias, float32, overwritten
 * The reductions behind gh and gb use a fixed partition and a fixed summation order:
 * results are bitwise reproducible from run to run.
 * Replaces the seven kernel launches and four torch reductions of `DeconvUpdate.backward`
 * (deconver/deconvolution/functional.py:118-182; kernels `deconv_bwd`, `gconv`, `wgrad`,
 * `deconv_gz`, deconver/deconvolution/kernels.py:791-894).
 */
int ndc_bwd(const NdcDesc *desc, const void *x, const void *z, const void *t1, const float *h,
            const float *bias, const void *gout, void *gx, void *gz, float *gh, float *gb,
            void *workspace, size_t workspace_bytes, void *stream);

/*
 * Size of the library-owned scratch array used by ndc_bwd_static.  Every GPU that uses this
 * library holds these bytes until the process exits.  When they are reserved depends on the
 * CUDA module-loading mode: with lazy loading (the default) it can be as late as the first
 * ndc_bwd_static call on that device, so make that call at start-up, while memory is there.
 */
#define NDC_STATIC_WORKSPACE_BYTES (16u * 1024u * 1024u)

/*
 * ndc_bwd for callers that cannot allocate device memory.  It has no counterpart in the
 * reference project.  Some hosts of this library own no allocator they are allowed to call
 * at the point where a backward pass runs: a plugin running inside another framework's
 * memory plan, a real-time or embedded inference/training loop that forbids cudaMalloc
 * after start-up, or code running while the process has handed all free device memory to a
 * pool it does not control.  For them the scratch that ndc_bwd takes from the caller lives
 * in a fixed array inside the library instead; inputs and outputs are still the caller's.
 *
 *  - Same arguments and results as ndc_bwd, minus the workspace.  No cudaMalloc, cudaFree or
 *    any other allocating call is made.
 *  - Limit: the geometry must need at most NDC_STATIC_WORKSPACE_BYTES of scratch; ask
 *    ndc_bwd_workspace_bytes for the exact figure of a geometry (it depends on the kernel
 *    family and its tiling, not only on the tensor sizes).  Larger ones are refused with
 *    NDC_ERR_WORKSPACE and a message naming both numbers.
 *  - The first call on each device looks up the array's device address (once per device,
 *    with that device current) and may be the moment the driver reserves the array.  Make
 *    that first call at start-up: before any stream capture, and before device memory is
 *    handed out to pools that could leave too little for it.
 *  - All calls on a device share the one array and it keeps whatever the last call left in
 *    it.  Nothing in it needs to start at zero: every value is written before it is read.
 *    Two calls whose kernels can overlap on the GPU (different streams, or different host
 *    threads) race on it; issue them on one stream or order them yourself.
 */
int ndc_bwd_static(const NdcDesc *desc, const void *x, const void *z, const void *t1,
                   const float *h, const float *bias, const void *gout, void *gx, void *gz,
                   float *gh, float *gb, void *stream);

/*
 * Instance normalisation of a (batch, channels, spatial...) tensor, forward and backward:
 *     y = (x - mean) * rstd [* weight[c] + bias[c]],   rstd = 1 / sqrt(var + eps),
 * mean and biased variance taken over the `spatial` positions of each (sample, channel) slab.
 * Replaces the `norm1` / `norm2` modules of the reference's `DeconverBlock`
 * (deconver/deconver.py:52-65), for which its configurations pass torch's InstanceNorm{2,3}d;
 * that library kernel runs one block per slab, which leaves most of the GPU idle at the small
 * per-GPU batches of the batch-sharded training step.  Here every slab is split over as many
 * CTAs as fill the device.  `weight`, `bias` (float32, per channel) may be NULL.  `mean_rstd`
 * receives (mean, rstd) per slab (2 * batch * channels floats) for the backward call, or may be
 * NULL in forward.  `workspace`: ndc_inorm_workspace_bytes(batch, channels) bytes of device
 * memory, 16-byte aligned, contents undefined before and after.  `gweight`, `gbias` (float32,
 * overwritten) may be NULL.  Sums use a fixed order: results are bitwise reproducible.
 * Errors: status code, message from ndc_inorm_last_error().
 */
size_t ndc_inorm_workspace_bytes(int32_t batch, int32_t channels);
const char *ndc_inorm_last_error(void);
int ndc_inorm_fwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void *x,
                  const float *weight, const float *bias, float eps, void *y, float *mean_rstd,
                  void *workspace, size_t workspace_bytes, void *stream);
int ndc_inorm_bwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void *x,
                  const void *gy, const float *weight, const float *mean_rstd, void *gx,
                  float *gweight, float *gbias, void *workspace, size_t workspace_bytes,
                  void *stream);

/*
 * Bias of the channels-first linear layer (`Linear`, deconver/layers/linear.py:34-58: a 1x1
 * `nn.Conv1d` over the flattened spatial axes).  The product itself stays a library GEMM; these
 * two calls replace what the library wraps around it:
 *     ndc_bias_add    y[b, c, :] += bias[c]            in place, y of dtype `dtype`
 *     ndc_bias_grad   gbias[c] = sum_{b, p} gy[b, c, p]  float32, overwritten, fixed order
 * `spatial` = positions per (sample, channel).  ndc_bias_grad needs
 * ndc_bias_grad_workspace_bytes(batch, channels) bytes of device scratch.  Errors: status code,
 * message from ndc_bias_last_error().
 */
size_t ndc_bias_grad_workspace_bytes(int32_t batch, int32_t channels);
const char *ndc_bias_last_error(void);
int ndc_bias_add(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, void *y,
                 const float *bias, void *stream);
int ndc_bias_grad(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype, const void *gy,
                  float *gbias, void *workspace, size_t workspace_bytes, void *stream);

/*
 * The same bias fused with the erf-form GELU (`nn.GELU()`, approximate='none'; erf evaluated to
 * an absolute error below 1e-6) between the two projections of the network's
 * MLP (`MLP`, deconver/layers/mlp.py:53-59: Linear, nn.GELU(), Dropout, Linear, Dropout), for
 * the bias-less product h of the first projection:
 *     ndc_bias_gelu_fwd   out = gelu(h + bias[c])                      one pass over h
 *     ndc_bias_gelu_bwd   gh = ga * gelu'(h + bias[c]);  gbias[c] = sum_{b, p} gh[b, c, p]
 * bias may be NULL (plain GELU); gbias may be NULL (then no workspace is needed), else it is
 * float32, overwritten, summed in a fixed order and the call needs
 * ndc_bias_grad_workspace_bytes(batch, channels) bytes of device scratch.  out / gh may not
 * alias h.  Errors as above.
 */
int ndc_bias_gelu_fwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype,
                      const void *h, const float *bias, void *out, void *stream);
int ndc_bias_gelu_bwd(int32_t batch, int32_t channels, int64_t spatial, int32_t dtype,
                      const void *ga, const void *h, const float *bias, void *gh, float *gbias,
                      void *workspace, size_t workspace_bytes, void *stream);

/*
 * Measurement aid; no counterpart in the reference project.  Launches one kernel of
 * register-only fused multiply-add chains (4 blocks of 256 threads per multiprocessor, 8
 * independent chains per thread, iters x 64 instructions per thread) on `stream`: plain
 * `fmaf` (packed = 0) or the two-lane `fma.rn.f32x2` (packed = 1).  `out` receives one float
 * per thread (out_elems >= 1024 x the device's multiprocessor count).  *fma_count is set to
 * the number of scalar multiply-adds the launch performs; timing it (CUDA events on the
 * same stream) gives the float32 multiply-add peak the NDC kernels are measured against.
 */
int ndc_probe_fp32_fma(int32_t packed, int32_t iters, float *out, size_t out_elems,
                       uint64_t *fma_count, void *stream);

/*
 * Grouped convolution K (adjoint = 0: groups*sc -> groups*m channels) or its adjoint A
 * (adjoint = 1: groups*m -> groups*sc channels) of a tensor of dtype desc->dtype.
 * With adjoint = 0, `bias` (or NULL) and desc->relu_input are applied to the input as it is
 * read, and out-of-volume taps contribute 0.  Replaces `kernels.gconv`
 * (deconver/deconvolution/kernels.py:728-759).
 */
int ndc_gconv(const NdcDesc *desc, const void *in, const float *h, const float *bias,
              int32_t adjoint, void *out, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* NDC_B200_H */
