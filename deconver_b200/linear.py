"""Channels-first linear layer.

Mirrors `deconver/layers/linear.py:7-58` of the reference: a 1x1 `nn.Conv1d` over the flattened
spatial axes, so the parameters are named `linear.weight` / `linear.bias` and checkpoints move
both ways.  The product is the library's convolution; on CUDA the bias is added (and its gradient
reduced) by this library's own kernels (`csrc/ndc_bias.cu`): the library's broadcast add is not
vectorised and its reduction uses one block per output channel, which shows at the small per-GPU
batches of a batch-sharded training step.  CPU tensors and other dtypes take the plain
`nn.Conv1d` with its bias.
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
        if bias is None or not flat.is_cuda or flat.dtype not in _DTYPES or flat.dim() != 3:
            y = self.linear(flat)
        else:
            y = _BiasAdd.apply(F.conv1d(flat, self.linear.weight, None), bias)
        return y.view(shape[0], -1, *shape[2:])
