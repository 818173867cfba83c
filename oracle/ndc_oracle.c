/*
 * CPU oracle for the nonnegative-deconvolution (NDC) source update, in plain C.
 * TEST INFRASTRUCTURE: only the test-suite, the smoke check and the benchmark's
 * CPU-baseline leg may load this library.  The product never links or calls it.
 *
 * It restates, with direct loops, the operator conventions and the backward formulas of
 * the reference's fused update (paths are within the reference project):
 *
 *   K(u)[o,p] = sum_{i,tau} u[i, p + tau - pad] * h[o,i,tau]
 *   A(v)[i,p] = sum_{o,tau} v[o, p + pad - tau] * h[o,i,tau]
 *                                   deconver/deconvolution/kernels.py:32-39
 *   s   = relu(z + b)   (bias and ReLU optional; out-of-volume taps contribute 0)
 *                                   deconver/deconvolution/kernels.py:227-233
 *   t1  = K(s);  out = (s * (A(x) + eps)) / (A(t1) + eps)
 *                                   deconver/deconvolution/functional.py:105-116,
 *                                   deconver/deconvolution/kernels.py:401-414
 *   gnum = g*s/d;  gden = -(gnum*n)/d;  gt1 = K(gden);  gx = K(gnum)
 *   gz   = [z+b>0] * ((g*n)/d + A(gt1));  gb = sum gz
 *   gh[o,i,tau] = sum_{b,p} gden[i,p] t1[o,p+pad-tau] + gnum[i,p] x[o,p+pad-tau]
 *                           + s[i,p] gt1[o,p+pad-tau]
 *                                   deconver/deconvolution/functional.py:118-182,
 *                                   deconver/deconvolution/kernels.py:488-493, :566-575, :868
 *
 * Parity pin: tests/test_oracle_golden.py checks both precisions of this file against
 * fixtures produced by the reference's own ReferenceDeconv (tests/golden/).
 *
 * Layout: contiguous channels-first.  x (B, G*m, D,H,W); z, out, gout, gz (B, G*sc, D,H,W);
 * t1, gx (B, G*m, D,H,W); h, gh (G*m, sc, kD,kH,kW); bias, gb (G*sc).
 * The body is instantiated twice, for double and for float.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int B, G, m, sc;
    int D, H, W;
    int kD, kH, kW;
} ndc_oracle_dims;

#define REAL double
#define SUFFIX(name) name##_f64
#include "ndc_oracle_body.inc"
#undef REAL
#undef SUFFIX

#define REAL float
#define SUFFIX(name) name##_f32
#include "ndc_oracle_body.inc"
#undef REAL
#undef SUFFIX
