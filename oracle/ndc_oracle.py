"""CPU oracle for the nonnegative-deconvolution (NDC) source update.  TEST INFRASTRUCTURE.

This file restates, in plain PyTorch on the CPU, the algorithm of the reference's eager
("general") path.  It exists so that the CUDA path can be checked and so that a CPU
baseline can be timed beside it.  Only the test-suite, the smoke check and the benchmark's
CPU-baseline leg may import it; the product package never does.

Parity pin: every function here is checked against outputs of the reference itself
(`ReferenceDeconv`, imported from the reference tree when the fixtures were generated) by
`tests/test_oracle_golden.py`, using the fixtures under `tests/golden/`.

What is restated, and from where (paths are within the reference project):

* `batched_conv`   - `deconver/deconvolution/operations.py:12-31` (batch folded into groups)
* `t`, `flip`      - `deconver/deconvolution/operations.py:52-57`
* `update_s`       - `deconver/deconvolution/deconv.py:191-195`
* `ndc_layer`      - `deconver/deconvolution/reference.py:254-273` (forward), `:190-207`
                     (iteration loop and the no-grad window), `:113-118` (initializer)
* `deconv_update`  - the same update expressed at the boundary of the fused autograd node,
                     `deconver/deconvolution/functional.py:105-116`; gradients come from
                     autograd, which is what the reference's eager path does
* `K`, `A`         - operator conventions of `deconver/deconvolution/kernels.py:32-39`,
                     written as ordinary grouped cross-correlations (used as an
                     independent second statement of the same update)
* `max_norm_error` - `tests/test_deconv_equivalence.py:51-59`
"""

from contextlib import nullcontext
from typing import Optional, Sequence

import torch
import torch.nn.functional as F
from torch import Tensor

_CONV = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}


# ----------------------------------------------------------------- eager-path restatement


def batched_conv(inp: Tensor, weight: Tensor, padding: Sequence[int]) -> Tensor:
    """Per-sample convolution: sample ``n`` of ``inp`` is correlated with ``weight[n]``.

    ``inp`` is ``(N, Cin, *S)`` and ``weight`` is ``(N, Cout, Cin, *k)``.  The N samples are
    folded into the group axis of one grouped convolution.
    """
    n = inp.shape[0]
    nd = inp.dim() - 2
    folded = inp.reshape(1, n * inp.shape[1], *inp.shape[2:])
    w = weight.reshape(n * weight.shape[1], weight.shape[2], *weight.shape[3:])
    out = _CONV[nd](folded, w, groups=n, padding=tuple(padding))
    return out.reshape(n, -1, *out.shape[2:])


def t(h: Tensor) -> Tensor:
    return h.transpose(1, 2)


def flip(h: Tensor) -> Tensor:
    return torch.flip(h, dims=tuple(range(3 - h.dim(), 0)))


def update_s(x: Tensor, s: Tensor, h: Tensor, eps: float, padding: Sequence[int]) -> Tensor:
    """One multiplicative update ``s <- s * (A x + eps) / (A K s + eps)``.

    Tensors are in the channel-split layout: ``x`` ``(B*G, m, *S)``, ``s`` ``(B*G, sc, *S)``,
    ``h`` ``(B*G, m, sc, *k)``.
    """
    ht = t(flip(h))
    num = batched_conv(x, ht, padding) + eps
    den = batched_conv(batched_conv(s, h, padding), ht, padding) + eps
    return s * num / den


def _split(v: Tensor, groups: int) -> Tensor:
    # "b (g c) ... -> (b g) c ..."
    b, gc = v.shape[:2]
    return v.reshape(b * groups, gc // groups, *v.shape[2:])


def _merge(v: Tensor, groups: int) -> Tensor:
    bg, c = v.shape[:2]
    return v.reshape(bg // groups, groups * c, *v.shape[2:])


def ndc_layer(
    x: Tensor,
    weight: Tensor,
    bias: Optional[Tensor],
    h0: Tensor,
    *,
    groups: int,
    eps: float = 1e-16,
    num_iters: int = 1,
    num_grad_iters: Optional[int] = None,
) -> Tensor:
    """Forward of the whole layer: projection, rectification, iterated updates.

    ``weight`` is the 1x1 projection ``(G*sc, C, 1)``, ``bias`` ``(G*sc,)``, ``h0`` the
    filter parameter ``(C, sc, *k)``.  Differentiable through autograd.
    """
    num_grad_iters = num_iters if num_grad_iters is None else num_grad_iters
    b = x.shape[0]
    ks = h0.shape[2:]
    pad = [k // 2 for k in ks]
    z = F.conv1d(x.flatten(2), weight, bias).view(b, -1, *x.shape[2:])
    s = F.relu(z)
    h = F.relu(h0.expand(b, *h0.shape))
    if groups != 1:
        xs, s, h = _split(x, groups), _split(s, groups), _split(h, groups)
    else:
        xs = x
    for it in range(1, num_iters + 1):
        ctx = torch.no_grad() if it < num_iters - num_grad_iters + 1 else nullcontext()
        with ctx:
            s = update_s(xs, s, h, eps, pad)
    return _merge(s, groups) if groups != 1 else s


def deconv_update(
    x: Tensor,
    z: Tensor,
    h: Tensor,
    bias: Optional[Tensor],
    *,
    groups: int,
    m: int,
    sc: int,
    eps: float,
    relu_input: bool,
) -> Tensor:
    """The update at the fused node's boundary, built from the eager-path pieces.

    ``x`` ``(B, G*m, *S)``, ``z`` ``(B, G*sc, *S)`` pre-bias and (if ``relu_input``)
    pre-ReLU, ``h`` the rectified filter ``(G*m, sc, *k)``, ``bias`` ``(G*sc,)`` or None.
    """
    b = x.shape[0]
    nd = x.dim() - 2
    pad = [k // 2 for k in h.shape[2:]]
    s = z if bias is None else z + bias.view(1, -1, *([1] * nd))
    if relu_input:
        s = F.relu(s)
    hb = h.expand(b, *h.shape)
    if groups != 1:
        xs, ss, hs = _split(x, groups), _split(s, groups), _split(hb, groups)
    else:
        xs, ss, hs = x, s, hb
    out = update_s(xs, ss, hs, eps, pad)
    return _merge(out, groups) if groups != 1 else out


def deconv_update_grads(x, z, h, bias, gout, **cfg):
    """``(out, gx, gz, gh, gb)`` of :func:`deconv_update` by autograd, in the input dtype."""
    x = x.detach().clone().requires_grad_(True)
    z = z.detach().clone().requires_grad_(True)
    h = h.detach().clone().requires_grad_(True)
    bias_l = None if bias is None else bias.detach().clone().requires_grad_(True)
    out = deconv_update(x, z, h, bias_l, **cfg)
    out.backward(gout)
    return (
        out.detach(),
        x.grad,
        z.grad,
        h.grad,
        None if bias_l is None else bias_l.grad,
    )


# ------------------------------------------------------- second, operator-form statement


def K(u: Tensor, h: Tensor, groups: int) -> Tensor:
    """``K(u)[o, p] = sum_{i, tau} u[i, p + tau - pad] h[o, i, tau]`` per group."""
    nd = u.dim() - 2
    pad = tuple(k // 2 for k in h.shape[2:])
    return _CONV[nd](u, h, groups=groups, padding=pad)


def A(v: Tensor, h: Tensor, groups: int) -> Tensor:
    """Adjoint of :func:`K`: ``A(v)[i, p] = sum_{o, tau} v[o, p + pad - tau] h[o, i, tau]``."""
    nd = v.dim() - 2
    ks = h.shape[2:]
    pad = tuple(k // 2 for k in ks)
    m = h.shape[0] // groups
    sc = h.shape[1]
    w = h.reshape(groups, m, sc, *ks).transpose(1, 2).reshape(groups * sc, m, *ks)
    w = torch.flip(w, dims=tuple(range(-nd, 0)))
    return _CONV[nd](v, w, groups=groups, padding=pad)


def deconv_update_operator_form(x, z, h, bias, *, groups, m, sc, eps, relu_input):
    nd = x.dim() - 2
    s = z if bias is None else z + bias.view(1, -1, *([1] * nd))
    if relu_input:
        s = F.relu(s)
    t1 = K(s, h, groups)
    return s * (A(x, h, groups) + eps) / (A(t1, h, groups) + eps), t1


# ------------------------------------------------------------------------------- metric


def max_norm_error(a: Tensor, b: Tensor) -> float:
    """``max|a - b| / max|b|`` evaluated in float64."""
    diff = (a.double() - b.double()).abs()
    scale = b.double().abs().max().clamp_min(1e-30)
    return (diff.max() / scale).item()
