"""Channels-first linear layer, kept for state-dict compatibility.

Mirrors `deconver/layers/linear.py:7-58` of the reference: a 1x1 `nn.Conv1d` over the
flattened spatial axes, so the parameters are named `linear.weight` / `linear.bias`.
"""

from typing import Optional

import torch
from torch import nn


class Linear(nn.Module):
    def __init__(self, in_channels: int, out_channels: int, bias: bool = True,
                 device: Optional[torch.device] = None, dtype: Optional[torch.dtype] = None):
        super().__init__()
        self.flatten = nn.Flatten(start_dim=2)
        self.linear = nn.Conv1d(in_channels, out_channels, kernel_size=1, bias=bias,
                                device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        y = self.linear(self.flatten(x))
        return y.view(shape[0], -1, *shape[2:])
