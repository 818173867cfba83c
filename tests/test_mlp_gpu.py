"""The fused bias + GELU kernels and the MLP built on them, against float64 PyTorch.

The module stands in for the `MLP` of the reference's blocks (`deconver/layers/mlp.py:9-62`:
Linear, nn.GELU(), Dropout, Linear, Dropout; `DeconverBlock.mlp`, `deconver/deconver.py:58`).
Tolerances (max-norm relative): float32 1e-5 forward and 1e-4 backward; bfloat16 storage 2e-2.
"""

import pytest
import torch
import torch.nn.functional as F

import deconver_b200 as dcb
from conftest import max_norm_error

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    dcb.load_library()
    return torch.device("cuda", 0)


CASES = [
    # batch, channels, spatial, with bias
    (2, 256, (32, 32, 32), True),      # hidden tensor of a stage of the 3-D network
    (3, 5, (7, 9, 11), True),          # odd sizes: scalar path
    (1, 3, (37,), False),
    (1, 1, (130000,), True),           # one slab, many parts
    (2, 6, (1, 2, 3), True),
]


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)], ids=["f32", "bf16"])
@pytest.mark.parametrize("case", CASES, ids=[str(c[:3]) for c in CASES])
def test_bias_gelu_matches_float64(dev, dtype, tol, case):
    B, C, S, with_bias = case
    torch.manual_seed(C)
    h = (torch.randn(B, C, *S) * 2.0).to(dtype)
    bias = torch.randn(C) if with_bias else None
    ga = torch.randn(B, C, *S).to(dtype)
    hd = h.to(dev).requires_grad_(True)
    bd = bias.to(dev).requires_grad_(True) if with_bias else None
    out = dcb.bias_gelu(hd, bd)
    out.backward(ga.to(dev))
    torch.cuda.synchronize()
    h64 = h.double().requires_grad_(True)
    b64 = bias.double().requires_grad_(True) if with_bias else None
    u = h64 + b64.view(1, C, *([1] * len(S))) if with_bias else h64
    ref = F.gelu(u)
    ref.backward(ga.double())
    assert out.dtype == dtype and out.shape == h.shape
    assert max_norm_error(out.detach().float().cpu().numpy(), ref.detach().numpy()) < tol
    assert max_norm_error(hd.grad.float().cpu().numpy(), h64.grad.numpy()) < max(tol, 1e-4)
    if with_bias:
        assert max_norm_error(bd.grad.float().cpu().numpy(), b64.grad.numpy()) < max(tol, 1e-4)


def test_bias_gelu_is_reproducible(dev):
    torch.manual_seed(0)
    h = torch.randn(2, 64, 24, 24, 24, device=dev, requires_grad=True)
    b = torch.randn(64, device=dev, requires_grad=True)
    g = torch.randn_like(h)
    grads = []
    for _ in range(2):
        h.grad = b.grad = None
        dcb.bias_gelu(h, b).backward(g)
        grads.append((h.grad.clone(), b.grad.clone()))
    assert torch.equal(grads[0][0], grads[1][0]) and torch.equal(grads[0][1], grads[1][1])


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)], ids=["f32", "bf16"])
def test_mlp_matches_plain_sequence(dev, dtype, tol):
    """`deconver_b200.MLP` against Linear -> GELU -> Linear written with plain convolutions in
    float64, same parameters; parameter names are those of the reference's MLP."""
    B, C, S = 2, 16, (12, 10, 8)
    torch.manual_seed(3)
    mine = dcb.MLP(C, ratio=4).to(device=dev, dtype=dtype)
    assert sorted(mine.state_dict()) == ["block.0.linear.bias", "block.0.linear.weight",
                                         "block.3.linear.bias", "block.3.linear.weight"]
    w1, b1 = mine.block[0].linear.weight, mine.block[0].linear.bias
    w2, b2 = mine.block[3].linear.weight, mine.block[3].linear.bias
    x = torch.randn(B, C, *S).to(dtype)
    g = torch.randn(B, C, *S).to(dtype)
    xd = x.to(dev).requires_grad_(True)
    old_flags = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
    torch.backends.cudnn.allow_tf32 = False        # the products are library calls: float32, not TF32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        y = mine(xd)
        y.backward(g.to(dev))
        torch.cuda.synchronize()
    finally:
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old_flags
    p64 = [t.detach().double().cpu().requires_grad_(True) for t in (w1, b1, w2, b2)]
    x64 = x.double().flatten(2).requires_grad_(True)
    y64 = F.conv1d(F.gelu(F.conv1d(x64, p64[0], p64[1])), p64[2], p64[3])
    y64.backward(g.double().flatten(2))
    assert y.shape == x.shape and y.dtype == dtype
    assert max_norm_error(y.detach().float().cpu().flatten(2).numpy(), y64.detach().numpy()) < tol
    assert max_norm_error(xd.grad.float().cpu().flatten(2).numpy(), x64.grad.numpy()) < max(tol, 1e-4)
    for mine_p, ref_p in zip((w1, b1, w2, b2), p64):
        assert max_norm_error(mine_p.grad.float().cpu().numpy(), ref_p.grad.numpy()) < max(tol, 1e-4)
