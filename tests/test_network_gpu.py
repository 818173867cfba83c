"""Whole-network check: a small 3-stage 3-D `Deconver` picks this library's layer up unchanged.

Counterpart of the reference's `tests/test_deconv_equivalence.py:311-379`.  The U-Net around
the NDC layer is the reference's own code, taken unmodified from an installation of the
reference under `baseline/_ref` (`pip install --no-deps --target baseline/_ref <checkout>`);
without that directory the test is skipped.  `deconver_b200.Deconv` is swapped in with the
monkey-patch the reference's tests use (`:321-330` there), the original network's checkpoint
is loaded into it, and both are compared with a float64 CPU run of the original network: the
network on this library must be no further from it than the original network is (x1.5), for
the output, the input gradient and every parameter gradient.  TF32 is switched off for the
library convolutions of both networks, so the bound is the float32 one (about 1e-5) rather than
the 1e-3 .. 1e-2 that TF32 leaves in the untouched parts of the network.
"""

import os
import sys

import pytest
import torch

import deconver_b200 as dcb

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

NETWORK = dict(
    in_channels=4, out_channels=3, spatial_dims=3, encoder_depth=(1, 1, 1),
    encoder_width=(8, 16, 32), strides=(1, 2, 2), decoder_depth=(1, 1),
    norm=torch.nn.InstanceNorm3d, act=torch.nn.ReLU, groups=-1, ratio=4,
    kernel_size=(3, 3, 3), num_iters=1, mlp_ratio=4,
)


@pytest.fixture(scope="module")
def reference():
    if not os.path.isdir(os.path.join(REF, "deconver")):
        pytest.skip("no reference installation under baseline/_ref")
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import deconver
    import deconver.deconver as deconver_module
    from deconver.deconvolution.reference import ReferenceDeconv
    return deconver, deconver_module, ReferenceDeconv


def _network(reference, layer_cls, dev, norm=None):
    """`norm` given: the network also gets this library's InstanceNorm3d, Linear and MLP."""
    dc, module, _ = reference
    import deconver.layers.mlp as mlp_module
    original, linear, mlp = module.Deconv, module.Linear, module.MLP
    module.Deconv = layer_cls
    if norm is not None:
        module.Linear = mlp_module.Linear = dcb.Linear
        module.MLP = dcb.MLP
    try:
        torch.manual_seed(0)
        kwargs = dict(NETWORK, norm=norm) if norm is not None else NETWORK
        return dc.Deconver(**kwargs).to(dev).eval()
    finally:
        module.Deconv = original
        module.Linear = mlp_module.Linear = linear
        module.MLP = mlp


def _errors(a, b):
    diff = (a.double() - b.double()).abs()
    return (diff.max() / b.double().abs().max().clamp_min(1e-30)).item()


@pytest.mark.parametrize("own_norm", [False, True], ids=["layer", "layer_and_norm"])
def test_network_on_this_layer_is_as_close_to_float64_as_the_original(reference, own_norm):
    """`own_norm`: the network is also given this library's InstanceNorm3d as its `norm` class
    and this library's Linear for its 1x1 projections."""
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    dcb.load_library()
    dev = torch.device("cuda:0")
    _, _, ReferenceDeconv = reference
    old = _network(reference, ReferenceDeconv, dev)
    new = _network(reference, dcb.Deconv, dev, norm=dcb.InstanceNorm3d if own_norm else None)
    assert any(isinstance(m, dcb.InstanceNorm3d) for m in new.modules()) == own_norm
    mixers = [m for m in new.modules() if type(m).__name__ == "DeconvMixer"]
    assert mixers and all((type(m.out_proj) is dcb.Linear) == own_norm for m in mixers)
    assert any(isinstance(m, dcb.MLP) for m in new.modules()) == own_norm
    assert any(isinstance(m, dcb.Deconv) for m in new.modules())
    assert not any(isinstance(m, ReferenceDeconv) for m in new.modules())
    assert list(old.state_dict()) == list(new.state_dict())
    new.load_state_dict(old.state_dict(), strict=True)

    torch.manual_seed(1)
    x0 = torch.rand(2, 4, 16, 16, 16)
    g0 = torch.randn(2, 3, 16, 16, 16)

    def run(module, dtype, device):
        module = module.to(device=device, dtype=dtype)
        x = x0.to(device=device, dtype=dtype).clone().requires_grad_(True)
        module.zero_grad(set_to_none=True)
        out = module(x)
        out.backward(g0.to(device=device, dtype=dtype))
        tensors = [out.detach().double().cpu().clone(), x.grad.double().cpu().clone()]
        tensors += [p.grad.double().cpu().clone() for p in module.parameters()
                    if p.grad is not None]
        module.to(device=dev, dtype=torch.float32)
        return tensors

    launches = dcb.load_library().ndc_launch_count()
    old_flags = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        new32 = run(new, torch.float32, dev)
        assert dcb.load_library().ndc_launch_count() > launches, "the CUDA library did not run"
        ref32 = run(old, torch.float32, dev)
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old_flags
    exact = run(old, torch.float64, "cpu")
    assert len(exact) == len(new32) == len(ref32)
    for i, (e, r, n) in enumerate(zip(exact, ref32, new32)):
        e_ref, e_new = _errors(r, e), _errors(n, e)
        assert e_new <= max(e_ref, 1e-5) * 1.5, (
            f"tensor {i}: error {e_new:.3e} on this library exceeds the original's {e_ref:.3e}")
