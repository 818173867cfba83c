"""Channels-first MLP with the first projection's bias fused into the GELU.

Mirrors `deconver/layers/mlp.py:9-62` of the reference: `block = Sequential(Linear, GELU,
Dropout, Linear, Dropout)`, the same constructor and the same parameter names
(`block.0.linear.weight`, ...), so checkpoints move both ways.  On CUDA (float32 / bfloat16) the
first projection runs without its bias and one kernel of this library (`csrc/ndc_bias.cu`)
computes ``gelu(h + bias)`` in a single pass over the hidden tensor, the largest of the block;
the backward computes ``ga * gelu'(h + bias)`` and the bias gradient in one pass.  The library
sequence is a broadcast add, a GELU pass, and on the way back a GELU-gradient pass plus a
reduction: two extra trips over the hidden tensor.  CPU tensors and other dtypes run the plain
sequence.
"""

from typing import Optional

import torch
from torch import nn
from torch.autograd.function import once_differentiable
from torch.nn.modules.utils import _pair

from . import _lib
from .linear import _DTYPES, Linear, _check, conv1x1


class _BiasGelu(torch.autograd.Function):
    """``gelu(h + bias[c])`` (erf form, erf to an absolute error below 1e-6) of a contiguous
    ``(B, C, L)`` tensor."""

    @staticmethod
    def forward(ctx, h, bias):
        h = h.contiguous()
        B, C, L = h.shape
        bf = None if bias is None else bias.detach().to(torch.float32).contiguous()
        out = torch.empty_like(h)
        if h.numel():
            with torch.cuda.device(h.device):
                _check(_lib.load().ndc_bias_gelu_fwd(
                    B, C, L, _DTYPES[h.dtype], h.data_ptr(), 0 if bf is None else bf.data_ptr(),
                    out.data_ptr(), torch.cuda.current_stream().cuda_stream))
        ctx.save_for_backward(h, bf)
        ctx.bias_dtype = None if bias is None else bias.dtype
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, ga):
        h, bf = ctx.saved_tensors
        ga = ga.contiguous()
        B, C, L = h.shape
        want_bias = bf is not None and ctx.needs_input_grad[1]
        gh = torch.empty_like(h)
        gbias = torch.zeros(C, device=h.device, dtype=torch.float32) if want_bias else None
        if h.numel():
            lib = _lib.load()
            with torch.cuda.device(h.device):
                nbytes = lib.ndc_bias_grad_workspace_bytes(B, C) if want_bias else 0
                ws = torch.empty(nbytes, device=h.device, dtype=torch.uint8) if want_bias else None
                _check(lib.ndc_bias_gelu_bwd(
                    B, C, L, _DTYPES[h.dtype], ga.data_ptr(), h.data_ptr(),
                    0 if bf is None else bf.data_ptr(), gh.data_ptr(),
                    gbias.data_ptr() if want_bias else 0, ws.data_ptr() if want_bias else 0, nbytes,
                    torch.cuda.current_stream().cuda_stream))
        return gh, (gbias.to(ctx.bias_dtype) if want_bias else None)


def bias_gelu(h: torch.Tensor, bias: Optional[torch.Tensor]) -> torch.Tensor:
    """``gelu(h + bias)`` over the channel axis (dim 1) of a CUDA float32 / bfloat16 tensor."""
    if not h.is_cuda or h.dtype not in _DTYPES:
        raise RuntimeError("bias_gelu runs on CUDA float32 / bfloat16 tensors only")
    shape = h.shape
    return _BiasGelu.apply(h.reshape(shape[0], shape[1], -1), bias).view(shape)


class MLP(nn.Module):
    def __init__(self, in_channels: int, out_channels: Optional[int] = None,
                 hidden_channels: Optional[int] = None, ratio: float = 4.0,
                 dropout=0.0, **kwargs):
        super().__init__()
        out_channels = out_channels or in_channels
        hidden_channels = hidden_channels or int(ratio * in_channels)
        dropout = _pair(dropout)
        self.block = nn.Sequential(
            Linear(in_channels, hidden_channels, **kwargs),
            nn.GELU(),
            nn.Dropout(dropout[0]),
            Linear(hidden_channels, out_channels, **kwargs),
            nn.Dropout(dropout[1]),
        )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        first, act, drop1, second, drop2 = self.block
        fused = (x.is_cuda and x.dtype in _DTYPES and x.dim() >= 3 and isinstance(act, nn.GELU)
                 and act.approximate == "none" and type(first) is Linear)
        if not fused:
            return self.block(x)
        shape = x.shape
        h = conv1x1(x.flatten(2), first.linear.weight)
        a = _BiasGelu.apply(h, first.linear.bias)
        a = drop1(a)
        return drop2(second(a.view(shape[0], -1, *shape[2:])))
