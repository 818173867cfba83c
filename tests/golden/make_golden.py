"""Generate the golden fixtures in this directory from the reference implementation itself.

Run once, on a machine that has the reference checkout, as

    python tests/golden/make_golden.py --reference /path/to/deconver

It imports the reference's `ReferenceDeconv` (the frozen ground-truth layer,
`deconver/deconvolution/reference.py:121-273`), runs it on seeded inputs on the CPU in
float64 and float32, and stores inputs and results as compressed `.npz` files.  The tests
then pin the CPU oracle (and through it the CUDA path) to these files; nothing at test time
needs the reference checkout.

Two kinds of fixture:

* `update_*.npz`  - one multiplicative update at the boundary of the fused node
  (`deconver/deconvolution/functional.py:105-182`): inputs `x, z, h, bias, gout`, results
  `out, gx, gz, gh, gb`.  The results come from the reference's own `update_s`
  (`reference.py:169-173`) applied to `relu(z + bias)` in the channel-split layout, with
  autograd for the gradients.
* `layer_*.npz`   - the whole layer: parameters `h0, weight, bias`, input `x`, upstream
  `gout`; results `y`, `gx`, `gh0`, `gweight`, `gbias` from `ReferenceDeconv.forward`.
* `cfg1_digest.npz` - the 2-D benchmark geometry (1,32,256,256), k=5x5, ratio 4: parameters
  plus a strided subsample and norms of the forward result (the full tensors are too large
  to commit; `x` is regenerated from its seed at test time).
* `cfg3_digest.npz` - the 3-D benchmark geometry, forward and backward: X (2,64,64,64,64),
  k=3x3x3, ratio 4, upstream gradient N(0,1); parameters, strided subsamples of the output
  and of the input gradient, and the full parameter gradients, from a float64 run (`x` and
  the upstream gradient are regenerated from their seeds at test time).  The projection bias
  is shifted by +1 as the reference's own comparisons do
  (`tests/test_deconv_equivalence.py:69-76`), so the layer is well conditioned.

`update_zero_*` fixtures hold whole blocks where the source is exactly zero, so the
denominator is `eps` alone there and the ratios are of the order of 1e16: the regime the
reference's comparisons avoid at the layer level, pinned here at the update boundary where
float32 and float64 still agree.
"""

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# name, layer kwargs, batch, spatial, relu_input/bias form
UPDATE_CASES = [
    ("dw3d", dict(channels=8, ratio=4, groups=-1, kernel_size=(3, 3, 3)), 2, (6, 5, 7), True),
    ("dw3d_wide", dict(channels=4, ratio=4, groups=-1, kernel_size=(3, 3, 3)), 1, (5, 9, 37), True),
    ("dw2d_k5", dict(channels=6, ratio=4, groups=-1, kernel_size=(5, 5)), 2, (11, 9), True),
    ("dw2d_k3", dict(channels=16, ratio=4, groups=-1, kernel_size=(3, 3)), 2, (17, 15), True),
    ("grouped", dict(channels=12, ratio=2, groups=3, kernel_size=(3, 3, 3)), 2, (7, 6, 5), True),
    ("dense", dict(channels=8, ratio=1, groups=1, kernel_size=(3, 3, 3)), 2, (6, 6, 6), True),
    ("aniso", dict(channels=6, ratio=2, groups=2, kernel_size=(3, 5, 3)), 2, (6, 7, 5), True),
    ("dw1d_k5", dict(channels=8, ratio=2, groups=-1, kernel_size=(5,)), 2, (11,), True),
    ("g5_2d", dict(channels=10, ratio=3, groups=5, kernel_size=(3, 3)), 2, (9, 8), True),
    ("brats512", dict(channels=512, ratio=4, groups=-1, kernel_size=(3, 3, 3)), 1, (3, 4, 3), True),
    ("later_iter", dict(channels=8, ratio=4, groups=-1, kernel_size=(3, 3, 3)), 2, (6, 5, 7), False),
    ("b3", dict(channels=6, ratio=4, groups=-1, kernel_size=(3, 3, 3)), 3, (9, 8, 7), True),
    # whole zero neighbourhoods of the source (denominator = eps): see `zero_blocks`
    ("zero_dw3d", dict(channels=6, ratio=4, groups=-1, kernel_size=(3, 3, 3)), 2, (10, 9, 12), True),
    ("zero_dw2d_k5", dict(channels=4, ratio=4, groups=-1, kernel_size=(5, 5)), 2, (21, 24), True),
    ("zero_later_iter", dict(channels=4, ratio=4, groups=-1, kernel_size=(3, 3, 3)), 1, (9, 8, 8), False),
    ("zero_grouped", dict(channels=8, ratio=2, groups=2, kernel_size=(3, 3, 3)), 2, (8, 7, 6), True),
]

LAYER_CASES = [
    ("layer_dw3d", dict(channels=16, ratio=4, groups=-1, kernel_size=(3, 3, 3), num_iters=1), 2, (7, 6, 8), 1.0),
    ("layer_dw3d_nobias_shift", dict(channels=16, ratio=4, groups=-1, kernel_size=(3, 3, 3), num_iters=1), 2, (7, 6, 8), 0.0),
    ("layer_dw2d_k5", dict(channels=8, ratio=4, groups=-1, kernel_size=(5, 5), num_iters=1), 2, (13, 12), 1.0),
    ("layer_iters_3_1", dict(channels=8, ratio=2, groups=-1, kernel_size=(3, 3, 3), num_iters=3, num_grad_iters=1), 2, (6, 6, 6), 1.0),
    ("layer_iters_2_2", dict(channels=8, ratio=2, groups=-1, kernel_size=(3, 3, 3), num_iters=2, num_grad_iters=2), 2, (6, 6, 6), 1.0),
    ("layer_iters_3_3", dict(channels=8, ratio=2, groups=-1, kernel_size=(3, 3, 3), num_iters=3, num_grad_iters=3), 2, (6, 6, 6), 1.0),
    ("layer_grouped", dict(channels=12, ratio=2, groups=3, kernel_size=(3, 3, 3), num_iters=1), 2, (7, 6, 5), 1.0),
]


def _np(t):
    return None if t is None else t.detach().cpu().numpy()


def zero_blocks(z, G, sc, first_iter):
    """Make the source exactly zero on whole blocks: the first half of the leading spatial axis
    for every channel, and the whole volume for the channels of group 0 in sample 0.  Before the
    first iteration the source is `relu(z + bias)` with |bias| well below 2, so -2 does it."""
    z = z.clone()
    off = -2.0 if first_iter else 0.0
    half = z.shape[2] // 2
    z[:, :, :half] = off
    z[0, :sc] = off
    return z


def update_case(ReferenceDeconv, name, kwargs, batch, spatial, first_iter, seed=0):
    torch.manual_seed(seed)
    ref = ReferenceDeconv(**kwargs)
    G, sc, C = ref.groups, ref.source_channels, ref.channels
    m = C // G
    torch.manual_seed(seed + 1)
    x = torch.rand(batch, C, *spatial)
    if first_iter:
        # pre-bias, pre-ReLU projection output, as the fused node receives it
        z = torch.randn(batch, G * sc, *spatial) * 0.5 + 0.25
        bias = torch.randn(G * sc) * 0.2
    else:
        # later iterations get an already rectified, biased source and no bias
        z = torch.relu(torch.randn(batch, G * sc, *spatial) * 0.5 + 0.4)
        bias = None
    if name.startswith("zero_"):
        z = zero_blocks(z, G, sc, first_iter)
    h = torch.relu(ref.init.h0.detach() + 0.05)
    torch.manual_seed(seed + 2)
    gout = torch.randn(batch, G * sc, *spatial)

    results = {}
    for tag, dt in (("f64", torch.float64), ("f32", torch.float32)):
        mod = ReferenceDeconv(**kwargs).to(dt)
        xl = x.to(dt).requires_grad_(True)
        zl = z.to(dt).requires_grad_(True)
        hl = h.to(dt).requires_grad_(True)
        bl = None if bias is None else bias.to(dt).requires_grad_(True)
        nd = len(spatial)
        s = zl if bl is None else zl + bl.view(1, -1, *([1] * nd))
        if first_iter:
            s = torch.relu(s)
        hb = hl.expand(batch, *hl.shape)
        if G != 1:
            xs, ss, hs = mod.split_channels(xl), mod.split_channels(s), mod.split_channels(hb)
        else:
            xs, ss, hs = xl, s, hb
        out = mod.update_s(xs, ss, hs)  # the reference's own update
        if G != 1:
            out = mod.merge_channels(out)
        out.backward(gout.to(dt))
        results.update({
            f"out_{tag}": _np(out), f"gx_{tag}": _np(xl.grad), f"gz_{tag}": _np(zl.grad),
            f"gh_{tag}": _np(hl.grad),
        })
        if bl is not None:
            results[f"gb_{tag}"] = _np(bl.grad)
    meta = dict(groups=G, m=m, sc=sc, eps=ref.eps, relu_input=int(first_iter),
                kernel_size=np.array(kwargs["kernel_size"]))
    arrays = dict(x=_np(x), z=_np(z), h=_np(h), gout=_np(gout), **meta, **results)
    if bias is not None:
        arrays["bias"] = _np(bias)
    np.savez_compressed(os.path.join(HERE, f"update_{name}.npz"), **arrays)
    print(f"update_{name}: out {results['out_f64'].shape}")


def layer_case(ReferenceDeconv, name, kwargs, batch, spatial, bias_shift, seed=0):
    torch.manual_seed(seed)
    ref = ReferenceDeconv(**kwargs)
    with torch.no_grad():
        ref.init.linear.linear.bias.add_(bias_shift)
    state = {k: v.clone() for k, v in ref.state_dict().items()}
    torch.manual_seed(seed + 1)
    x = torch.rand(batch, kwargs["channels"], *spatial)
    torch.manual_seed(seed + 2)
    gout = torch.randn(batch, ref.groups * ref.source_channels, *spatial)
    results = {}
    for tag, dt in (("f64", torch.float64), ("f32", torch.float32)):
        mod = ReferenceDeconv(**kwargs)
        mod.load_state_dict(state)
        mod = mod.to(dt)
        xl = x.to(dt).requires_grad_(True)
        y = mod(xl)
        y.backward(gout.to(dt))
        results[f"y_{tag}"] = _np(y)
        results[f"gx_{tag}"] = _np(xl.grad)
        for pname, p in mod.named_parameters():
            key = {"init.h0": "gh0", "init.linear.linear.weight": "gweight",
                   "init.linear.linear.bias": "gbias"}[pname]
            if p.grad is not None:
                results[f"{key}_{tag}"] = _np(p.grad)
    arrays = dict(
        x=_np(x), gout=_np(gout), h0=_np(state["init.h0"]),
        weight=_np(state["init.linear.linear.weight"]),
        bias=_np(state["init.linear.linear.bias"]),
        groups=ref.groups, sc=ref.source_channels, eps=ref.eps,
        num_iters=ref.num_iters, num_grad_iters=ref.num_grad_iters,
        kernel_size=np.array(kwargs["kernel_size"]), **results,
    )
    np.savez_compressed(os.path.join(HERE, f"{name}.npz"), **arrays)
    print(f"{name}: y {results['y_f64'].shape}")


def cfg1_digest(ReferenceDeconv):
    """2-D benchmark geometry: X (1,32,256,256) uniform, K = |N(0,1)|/25, defaults, seed 0."""
    kwargs = dict(channels=32, ratio=4, groups=-1, kernel_size=(5, 5))
    torch.manual_seed(0)
    ref = ReferenceDeconv(**kwargs)
    with torch.no_grad():
        ref.init.h0.copy_(torch.randn(32, 4, 5, 5).abs() / 25)
    torch.manual_seed(1)
    x = torch.rand(1, 32, 256, 256)
    with torch.no_grad():
        y32 = ref(x)
        y64 = ref.double()(x.double())
    flat = y64.flatten()
    idx = torch.arange(0, flat.numel(), 997)
    state = ref.state_dict()
    np.savez_compressed(
        os.path.join(HERE, "cfg1_digest.npz"),
        h0=_np(state["init.h0"].float()), weight=_np(state["init.linear.linear.weight"].float()),
        bias=_np(state["init.linear.linear.bias"].float()),
        x_seed=1, x_shape=np.array(x.shape), stride=997,
        y_sub_f64=_np(flat[idx]), y_sub_f32=_np(y32.flatten()[idx]),
        y_sum_f64=float(flat.sum()), y_abs_max_f64=float(flat.abs().max()),
        y_l2_f64=float(flat.square().sum().sqrt()),
        x_sum=float(x.double().sum()),
    )
    print("cfg1_digest:", tuple(y64.shape))


def cfg3_digest(ReferenceDeconv):
    """3-D benchmark geometry, forward + backward: X (2,64,64,64,64) uniform, K = |N(0,1)|/27,
    upstream gradient N(0,1), projection bias shifted by +1; float64 on the CPU."""
    kwargs = dict(channels=64, ratio=4, groups=-1, kernel_size=(3, 3, 3))
    torch.manual_seed(0)
    ref = ReferenceDeconv(**kwargs)
    with torch.no_grad():
        ref.init.h0.copy_(torch.randn(64, 4, 3, 3, 3).abs() / 27)
        ref.init.linear.linear.bias.add_(1.0)
    state = {k: v.clone() for k, v in ref.state_dict().items()}
    x = torch.rand(2, 64, 64, 64, 64, generator=torch.Generator().manual_seed(1))
    gout = torch.randn(2, 256, 64, 64, 64, generator=torch.Generator().manual_seed(2))
    mod = ref.double()
    xl = x.double().requires_grad_(True)
    y = mod(xl)
    y.backward(gout.double())
    yf, gxf = y.detach().flatten(), xl.grad.flatten()
    ys, gs = 4093, 1021          # primes: the samples walk through every channel and row
    np.savez_compressed(
        os.path.join(HERE, "cfg3_digest.npz"),
        h0=_np(state["init.h0"]), weight=_np(state["init.linear.linear.weight"]),
        bias=_np(state["init.linear.linear.bias"]),
        x_seed=1, gout_seed=2, x_shape=np.array(x.shape), gout_shape=np.array(gout.shape),
        x_sum=float(x.double().sum()), gout_sum=float(gout.double().sum()),
        y_stride=ys, gx_stride=gs,
        y_sub_f64=_np(yf[::ys]), gx_sub_f64=_np(gxf[::gs]),
        y_abs_max_f64=float(yf.abs().max()), gx_abs_max_f64=float(gxf.abs().max()),
        y_sum_f64=float(yf.sum()), gx_sum_f64=float(gxf.sum()),
        gh0_f64=_np(mod.init.h0.grad), gweight_f64=_np(mod.init.linear.linear.weight.grad),
        gbias_f64=_np(mod.init.linear.linear.bias.grad),
    )
    print("cfg3_digest:", tuple(y.shape))


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--only", default="", help="comma-separated fixture names to (re)generate")
    args = ap.parse_args()
    only = set(filter(None, args.only.split(",")))
    sys.path.insert(0, args.reference)
    from deconver.deconvolution.reference import ReferenceDeconv

    torch.set_num_threads(max(1, os.cpu_count() or 1))
    for case in UPDATE_CASES:
        if not only or "update_" + case[0] in only:
            update_case(ReferenceDeconv, *case)
    for case in LAYER_CASES:
        if not only or case[0] in only:
            layer_case(ReferenceDeconv, *case)
    if not only or "cfg1_digest" in only:
        cfg1_digest(ReferenceDeconv)
    if not only or "cfg3_digest" in only:
        cfg3_digest(ReferenceDeconv)


if __name__ == "__main__":
    main()
