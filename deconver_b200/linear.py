"""Channels-first linear layer.

Mirrors `deconver/layers/linear.py:7-58` of the reference: a 1x1 `nn.Conv1d` over the flattened
spatial axes, so the parameters are named `linear.weight` / `linear.bias` and checkpoints move
both ways.  The product is a library GEMM; on CUDA the bias is added (and its gradient
reduced) by this library's own kernels (`csrc/ndc_bias.cu`): the library's broadcast add is not
vectorised and its reduction uses one block per output channel, which shows at the small per-GPU
batches of a batch-sharded training step.  For bfloat16 the weight gradient is a split batched
GEMM (`_weight_grad`).  CPU tensors and other dtypes take the plain `nn.Conv1d` with its bias.
"""

from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn
from torch.autograd.function import once_differentiable

from . import _lib

_DTYPES = {torch.float32: _lib.NDC_F32, torch.bfloat16: _lib.NDC_BF16}


def _check(status: int) -> None:
    if status != _lib.NDC_OK:
        raise _lib.NdcError(status, _lib.load().ndc_bias_last_error().decode("utf-8", "replace"))


class _BiasAdd(torch.autograd.Function):
    """``y[b, c, :] += bias[c]`` in place on a fresh `(B, C, L)` product."""

    @staticmethod
    def forward(ctx, y, bias):
        B, C, L = y.shape
        bf = bias.detach().to(torch.float32).contiguous()
        if y.numel():
            with torch.cuda.device(y.device):
                _check(_lib.load().ndc_bias_add(B, C, L, _DTYPES[y.dtype], y.data_ptr(), bf.data_ptr(),
                                                torch.cuda.current_stream().cuda_stream))
        ctx.mark_dirty(y)
        ctx.bias_dtype = bias.dtype
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, gy):
        gbias = None
        if ctx.needs_input_grad[1]:
            g = gy.contiguous()
            B, C, L = g.shape
            gbias = torch.zeros(C, device=g.device, dtype=torch.float32)
            if g.numel():
                lib = _lib.load()
                with torch.cuda.device(g.device):
                    nbytes = lib.ndc_bias_grad_workspace_bytes(B, C)
                    ws = torch.empty(nbytes, device=g.device, dtype=torch.uint8)
                    _check(lib.ndc_bias_grad(B, C, L, _DTYPES[g.dtype], g.data_ptr(), gbias.data_ptr(),
                                             ws.data_ptr(), nbytes,
                                             torch.cuda.current_stream().cuda_stream))
            gbias = gbias.to(ctx.bias_dtype)
        return gy, gbias


def _weight_grad(gy: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``dW[o, c] = sum_{b, p} gy[b, o, p] * x[b, c, p]`` of a 1x1 convolution, ``(Co, Ci)``.

    This is a GEMM with a tiny output and a huge inner dimension (every position of every
    sample).  At the small per-GPU batches of a batch-sharded training step the library's
    convolution backward takes 3-4x the time the two reads need (0.31 ms against 0.09 ms for
    bfloat16 tensors of 2 x 256 x 64^3 and 2 x 64 x 64^3).  Here the positions of each sample
    are cut into S slices (up to 32, of at least 2048 positions: enough tiles per launch to
    fill the GPU) and ONE strided batched GEMM (library) multiplies all slices, with
    float32 partial products (the samples accumulate into the same S partial products, which are
    then added in a fixed order); no operand is copied: the slices are views of the tensors as
    they lie.  Batches above 4, float32 and CPU tensors keep
    the library's own weight gradient, which is the faster one there (measured on the 3-D
    network's training step: 28.1 against 29.6 ms at batch 4, level at 52.7 ms at batch 8).
    """
    B, Co, N = gy.shape
    Ci = x.shape[1]
    S = 1
    while S * 2 <= 32 and N % (S * 2 * 8) == 0 and N // (S * 2) >= 2048:
        S *= 2
    if gy.dtype != torch.bfloat16 or not gy.is_cuda or B > 4 or S == 1:
        return torch.nn.grad.conv1d_weight(x, (Co, Ci, 1), gy)[:, :, 0]
    L = N // S
    acc = None
    for b in range(B):
        a = gy[b].view(Co, S, L).transpose(0, 1)          # (S, Co, L), strides (L, N, 1)
        c = x[b].view(Ci, S, L).permute(1, 2, 0)          # (S, L, Ci), strides (L, 1, N)
        acc = (torch.bmm(a, c, out_dtype=torch.float32) if acc is None
               else torch.baddbmm(acc, a, c, out_dtype=torch.float32))
    return acc.sum(0)


def _channel_gemm(w2: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """``y[b] = w2 @ x[b]`` for a ``(Co, Ci)`` matrix (any strides) and a contiguous
    ``(B, Ci, N)`` tensor: one strided batched GEMM (library) with the matrix repeated by a zero
    batch stride.  The same product as a 1x1 `conv1d`, bit for bit where both were compared, but
    the convolution route converts the tensor to channels-last and back for some shapes (256 -> 64
    channels over 4 x 128^3 positions: 4.49 ms against 0.98 ms here; never slower where measured).
    """
    return torch.bmm(w2.unsqueeze(0).expand(x.shape[0], *w2.shape), x)


class Conv1x1(torch.autograd.Function):
    """``y = W x`` over the channel axis of a contiguous ``(B, Ci, N)`` tensor, no bias: library
    GEMMs for the product and the input gradient, `_weight_grad` for the weight."""

    @staticmethod
    def forward(ctx, x, weight):
        ctx.save_for_backward(x, weight)
        return _channel_gemm(weight[:, :, 0], x)

    @staticmethod
    @once_differentiable
    def backward(ctx, gy):
        x, weight = ctx.saved_tensors
        gy = gy.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = _channel_gemm(weight[:, :, 0].t(), gy)                      # W^T gy
        if ctx.needs_input_grad[1]:
            gw = _weight_grad(gy, x).unsqueeze(-1).to(weight.dtype)
        return gx, gw


def conv1x1(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """1x1 convolution of a ``(B, Ci, N)`` tensor with ``weight`` ``(Co, Ci, 1)``, no bias."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 3:
        return Conv1x1.apply(x.contiguous(), weight)
    return F.conv1d(x, weight, None)


class Linear(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.flatten = nn.Flatten(start_dim=2)
        self.linear = nn.Conv1d(in_channels, out_channels, kernel_size=1, bias=bias,
                                device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        flat = self.flatten(x)
        bias = self.linear.bias
        if not flat.is_cuda or flat.dtype not in _DTYPES or flat.dim() != 3:
            y = self.linear(flat)
        elif bias is None:
            y = conv1x1(flat, self.linear.weight)
        else:
            y = _BiasAdd.apply(conv1x1(flat, self.linear.weight), bias)
        return y.view(shape[0], -1, *shape[2:])
