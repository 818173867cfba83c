"""Instance normalisation kernels against PyTorch's `instance_norm` evaluated in float64.

The modules stand in for the `norm` class of the reference's blocks (`DeconverBlock.norm1/2`,
`deconver/deconver.py:52-65`; its configurations pass `torch.nn.InstanceNorm{2,3}d`).
Tolerances (max-norm relative): float32 1e-5 forward and 1e-4 backward; bfloat16 storage 2e-2.
"""

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import deconver_b200 as dcb
from conftest import max_norm_error

pytestmark = pytest.mark.gpu

CASES = [
    # batch, channels, spatial, affine
    (2, 64, (64, 64, 64), False),      # stage-1 geometry of the 3-D network at a per-GPU batch of 2
    (2, 512, (8, 8, 8), False),
    (3, 5, (7, 9, 11), True),          # odd sizes: scalar path
    (1, 3, (37,), True),
    (4, 32, (256, 256), False),
    (1, 1, (130000,), False),          # one slab, many parts
    (2, 6, (1, 2, 3), True),           # six positions per slab
]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    dcb.load_library()
    return torch.device("cuda:0")


def _reference(x, w, b, g, eps):
    x64 = x.double().requires_grad_(True)
    w64 = None if w is None else w.double().requires_grad_(True)
    b64 = None if b is None else b.double().requires_grad_(True)
    y = F.instance_norm(x64, weight=w64, bias=b64, eps=eps)
    y.backward(g.double())
    return y.detach(), x64.grad, None if w64 is None else w64.grad, None if b64 is None else b64.grad


@pytest.mark.parametrize("case", CASES, ids=lambda c: "b%d_c%d_%s%s" % (
    c[0], c[1], "x".join(map(str, c[2])), "_affine" if c[3] else ""))
@pytest.mark.parametrize("dtype,tol,gtol", [(torch.float32, 1e-5, 1e-4), (torch.bfloat16, 2e-2, 2e-2)],
                         ids=["f32", "bf16"])
def test_instance_norm_matches_float64(dev, case, dtype, tol, gtol):
    B, C, S, affine = case
    gen = torch.Generator().manual_seed(B * 100 + C)
    # a mean well away from zero: the variance must not lose digits to cancellation
    x = (torch.randn(B, C, *S, generator=gen) * 0.7 + 5.0).to(dtype)
    g = torch.randn(B, C, *S, generator=gen).to(dtype)
    w = (torch.rand(C, generator=gen) + 0.5) if affine else None
    b = torch.randn(C, generator=gen) if affine else None
    ref = _reference(x.float(), w, b, g.float(), 1e-5)
    xd = x.to(dev).requires_grad_(True)
    wd = None if w is None else w.to(dev).requires_grad_(True)
    bd = None if b is None else b.to(dev).requires_grad_(True)
    y = dcb.instance_norm(xd, wd, bd, 1e-5)
    y.backward(g.to(dev))
    torch.cuda.synchronize()
    assert y.dtype == dtype and y.shape == x.shape
    assert max_norm_error(y.detach().float().cpu().numpy(), ref[0].numpy()) < tol
    assert max_norm_error(xd.grad.float().cpu().numpy(), ref[1].numpy()) < gtol
    if affine:
        assert max_norm_error(wd.grad.cpu().numpy(), ref[2].numpy()) < max(gtol, 1e-4)
        assert max_norm_error(bd.grad.cpu().numpy(), ref[3].numpy()) < max(gtol, 1e-4)


def test_module_matches_torch_module_and_is_reproducible(dev):
    torch.manual_seed(0)
    x = torch.randn(2, 16, 12, 10, 20, device=dev)
    mine, theirs = dcb.InstanceNorm3d(16), torch.nn.InstanceNorm3d(16)
    assert list(mine.state_dict()) == list(theirs.state_dict())
    a, b = mine(x), mine(x)
    assert torch.equal(a, b)
    assert max_norm_error(a.cpu().numpy(), theirs(x).double().cpu().numpy()) < 1e-5
    affine = dcb.InstanceNorm2d(8, affine=True).to(dev)
    assert sorted(affine.state_dict()) == sorted(torch.nn.InstanceNorm2d(8, affine=True).state_dict())
    with pytest.raises(ValueError):
        affine(x)
    with pytest.raises(RuntimeError, match="CUDA"):
        dcb.instance_norm(torch.randn(1, 2, 4))
    with pytest.raises(NotImplementedError):
        dcb.InstanceNorm1d(4, track_running_stats=True)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 64, 256, (32, 32, 32)), (3, 5, 7, (9, 11)), (1, 16, 8, (4100,))],
                         ids=["volume", "odd", "row"])
def test_linear_matches_conv1d(dev, dtype, tol, shape):
    """`deconver_b200.Linear` (library product + this library's bias add and bias gradient)
    against the plain `nn.Conv1d` form of the reference's `Linear` (`layers/linear.py:34-58`),
    evaluated in float64."""
    B, Ci, Co, S = shape
    torch.manual_seed(Ci + Co)
    mine = dcb.Linear(Ci, Co).to(device=dev, dtype=dtype)
    ref = torch.nn.Conv1d(Ci, Co, 1).double()
    ref.load_state_dict({k.replace("linear.", ""): v.double().cpu() for k, v in mine.state_dict().items()})
    assert sorted(mine.state_dict()) == ["linear.bias", "linear.weight"]
    x = torch.randn(B, Ci, *S).to(dtype)
    g = torch.randn(B, Co, *S).to(dtype)
    xd = x.to(dev).requires_grad_(True)
    old_flags = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = False        # the product is a library call: float32, not TF32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        y = mine(xd)
        y.backward(g.to(dev))
        torch.cuda.synchronize()
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old_flags
    x64 = x.double().flatten(2).requires_grad_(True)
    y64 = ref(x64)
    y64.backward(g.double().flatten(2))
    assert y.shape == (B, Co, *S) and y.dtype == dtype
    assert max_norm_error(y.detach().float().cpu().flatten(2).numpy(), y64.detach().numpy()) < tol
    assert max_norm_error(mine.linear.bias.grad.float().cpu().numpy(), ref.bias.grad.numpy()) < max(tol, 1e-4)
    assert max_norm_error(mine.linear.weight.grad.float().cpu().numpy(), ref.weight.grad.numpy()) < max(tol, 1e-4)
    assert max_norm_error(xd.grad.float().cpu().flatten(2).numpy(), x64.grad.numpy()) < max(tol, 1e-4)
