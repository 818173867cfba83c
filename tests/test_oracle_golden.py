"""Pin the CPU oracle (both the PyTorch restatement and the plain-C one) to the fixtures
that were produced by the reference's own `ReferenceDeconv` (tests/golden/make_golden.py)."""

import numpy as np
import pytest
import torch

from conftest import golden_names, load_golden, max_norm_error, update_cfg
from oracle import ndc_oracle as O

UPDATE = golden_names("update_")
LAYER = golden_names("layer_")


def _t(a, dt):
    return None if a is None else torch.from_numpy(np.asarray(a)).to(dt)


@pytest.mark.parametrize("name", UPDATE)
@pytest.mark.parametrize("tag,dt,tol", [("f64", torch.float64, 1e-12), ("f32", torch.float32, 2e-5)])
def test_torch_oracle_update(name, tag, dt, tol):
    g = load_golden(name)
    cfg = update_cfg(g)
    out, gx, gz, gh, gb = O.deconv_update_grads(
        _t(g["x"], dt), _t(g["z"], dt), _t(g["h"], dt), _t(g.get("bias"), dt), _t(g["gout"], dt), **cfg
    )
    got = dict(out=out, gx=gx, gz=gz, gh=gh, gb=gb)
    for k, v in got.items():
        if v is None:
            assert f"{k}_f64" not in g
            continue
        assert max_norm_error(v.numpy(), g[f"{k}_f64"]) < tol, (name, k)
    # the operator-form statement (K and A as grouped correlations) gives the same update
    out2, _ = O.deconv_update_operator_form(
        _t(g["x"], dt), _t(g["z"], dt), _t(g["h"], dt), _t(g.get("bias"), dt), **cfg)
    assert max_norm_error(out2.numpy(), g["out_f64"]) < tol


@pytest.mark.parametrize("name", UPDATE)
@pytest.mark.parametrize("npdt,tol", [(np.float64, 1e-12), (np.float32, 2e-5)])
def test_c_oracle_update(c_oracle, name, npdt, tol):
    g = load_golden(name)
    cfg = update_cfg(g)
    a = {k: (None if g.get(k) is None else g[k].astype(npdt)) for k in ("x", "z", "h", "bias", "gout")}
    out, t1 = c_oracle.forward(a["x"], a["z"], a["h"], a["bias"], **cfg)
    gx, gz, gh, gb = c_oracle.backward(a["x"], a["z"], a["h"], a["bias"], a["gout"], **cfg)
    assert max_norm_error(out, g["out_f64"]) < tol
    assert max_norm_error(gx, g["gx_f64"]) < tol
    assert max_norm_error(gz, g["gz_f64"]) < tol
    assert max_norm_error(gh, g["gh_f64"]) < tol
    if "gb_f64" in g:
        assert max_norm_error(gb, g["gb_f64"]) < tol
    # t1 = K(s) agrees with the grouped-correlation statement
    dt = torch.float64 if npdt == np.float64 else torch.float32
    _, t1_ref = O.deconv_update_operator_form(
        _t(a["x"], dt), _t(a["z"], dt), _t(a["h"], dt), _t(a["bias"], dt), **cfg)
    assert max_norm_error(t1, t1_ref.numpy()) < tol


@pytest.mark.parametrize("name", LAYER)
@pytest.mark.parametrize("tag,dt,tol,gtol", [("f64", torch.float64, 1e-12, 1e-11),
                                               ("f32", torch.float32, 1e-5, 1e-3)])
def test_torch_oracle_layer(name, tag, dt, tol, gtol):
    g = load_golden(name)
    x = _t(g["x"], dt).requires_grad_(True)
    w = _t(g["weight"], dt).requires_grad_(True)
    b = _t(g["bias"], dt).requires_grad_(True)
    h0 = _t(g["h0"], dt).requires_grad_(True)
    y = O.ndc_layer(x, w, b, h0, groups=int(g["groups"]), eps=float(g["eps"]),
                    num_iters=int(g["num_iters"]), num_grad_iters=int(g["num_grad_iters"]))
    assert max_norm_error(y.detach().numpy(), g["y_f64"]) < tol
    y.backward(_t(g["gout"], dt))
    for key, p in (("gx", x), ("gweight", w), ("gbias", b), ("gh0", h0)):
        ref = g.get(f"{key}_f64")
        if ref is None:
            assert p.grad is None or float(p.grad.abs().max()) == 0.0
            continue
        assert max_norm_error(p.grad.numpy(), ref) < gtol, (name, key)


def test_cfg1_digest():
    """The 2-D benchmark geometry (CPU-runnable case): X (1,32,256,256), k=5x5, ratio 4."""
    g = load_golden("cfg1_digest")
    torch.manual_seed(int(g["x_seed"]))
    x = torch.rand(*[int(v) for v in g["x_shape"]])
    assert abs(float(x.double().sum()) - float(g["x_sum"])) < 1e-6 * float(g["x_sum"])
    with torch.no_grad():
        y = O.ndc_layer(x, _t(g["weight"], torch.float32), _t(g["bias"], torch.float32),
                        _t(g["h0"], torch.float32), groups=32)
    sub = y.flatten()[:: int(g["stride"])].numpy()
    assert max_norm_error(sub, g["y_sub_f64"]) < 1e-5
    assert abs(float(y.double().sum()) - float(g["y_sum_f64"])) < 1e-4 * abs(float(g["y_sum_f64"]))


def test_cfg3_digest():
    """The 3-D benchmark geometry, forward and backward, float32 on the CPU (about half a
    minute): the oracle's port of the layer against the digest of the reference's float64 run."""
    g = load_golden("cfg3_digest")
    x = torch.rand(*[int(v) for v in g["x_shape"]],
                   generator=torch.Generator().manual_seed(int(g["x_seed"])))
    gout = torch.randn(*[int(v) for v in g["gout_shape"]],
                       generator=torch.Generator().manual_seed(int(g["gout_seed"])))
    assert abs(float(x.double().sum()) - float(g["x_sum"])) < 1e-6 * float(g["x_sum"])
    assert abs(float(gout.double().sum()) - float(g["gout_sum"])) < 1e-3
    x.requires_grad_(True)
    w = _t(g["weight"], torch.float32).requires_grad_(True)
    b = _t(g["bias"], torch.float32).requires_grad_(True)
    h0 = _t(g["h0"], torch.float32).requires_grad_(True)
    y = O.ndc_layer(x, w, b, h0, groups=64)
    y.backward(gout)
    ysub = y.detach().flatten()[:: int(g["y_stride"])].double().numpy()
    assert np.abs(ysub - g["y_sub_f64"]).max() / float(g["y_abs_max_f64"]) < 1e-5
    gsub = x.grad.flatten()[:: int(g["gx_stride"])].double().numpy()
    assert np.abs(gsub - g["gx_sub_f64"]).max() / float(g["gx_abs_max_f64"]) < 1e-3
    for key, p in (("gh0", h0), ("gweight", w), ("gbias", b)):
        assert max_norm_error(p.grad.numpy(), g[f"{key}_f64"]) < 1e-3, key
