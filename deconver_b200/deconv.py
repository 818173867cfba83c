"""The NDC (nonnegative deconvolution) layer on the sm_100a kernels.

`Deconv` keeps the constructor, the methods and the state-dict keys of the reference's
`deconver/deconvolution/deconv.py:48-295` (`init.h0`, `init.linear.linear.weight`,
`init.linear.linear.bias`), so it can stand in for it inside `DeconvMixer` unchanged.  What
differs is the dispatch: there is exactly one compute path, the CUDA kernels behind
`deconv_update`.  Configurations they do not cover raise `NotImplementedError`; there is no
Triton path, no eager path and no CPU path to fall back to.
"""

import math
from contextlib import nullcontext
from typing import Any, Optional, Sequence

import torch
import torch.nn.functional as F
from torch import Tensor, nn

from .functional import deconv_update, kernels_apply
from .linear import Linear, conv1x1

__all__ = ["Initializer", "Deconv", "NDC"]

_CONV = {1: F.conv1d, 2: F.conv2d, 3: F.conv3d}


class Initializer(nn.Module):
    """Learned starting point: filter `h0` and the 1x1 projection that makes the source.

    Same parameters and initialisation as `deconv.py:20-45` of the reference.
    """

    def __init__(self, channels: int, source_channels: int, kernel_size: Sequence[int],
                 groups: int) -> None:
        super().__init__()
        groups = channels if groups is None else groups
        assert channels % groups == 0, "`channels` must be divisible by groups"
        h0 = torch.empty(channels, source_channels, *kernel_size)
        nn.init.kaiming_uniform_(h0, a=math.sqrt(5))
        self.h0 = nn.Parameter(h0)
        self.linear = Linear(channels, groups * source_channels)

    def forward(self, x: Tensor) -> tuple[Tensor, Tensor]:
        h = self.h0.expand(x.shape[0], *self.h0.shape)
        return F.relu(self.linear(x)), F.relu(h)


def _batched_conv(inp: Tensor, weight: Tensor, padding) -> Tensor:
    """Sample ``n`` of `inp` correlated with `weight[n]` (used by `reconstruct`/`loss` only)."""
    n = inp.shape[0]
    folded = inp.reshape(1, n * inp.shape[1], *inp.shape[2:])
    w = weight.reshape(n * weight.shape[1], weight.shape[2], *weight.shape[3:])
    out = _CONV[inp.dim() - 2](folded, w, groups=n, padding=padding)
    return out.reshape(n, -1, *out.shape[2:])


class Deconv(nn.Module):
    """Deconvolution layer: fits a non-negative source ``s`` with ``x ~ conv(s, h)`` by
    multiplicative updates from a learned initialisation, and returns ``s``."""

    def __init__(
        self,
        channels: int,
        kernel_size=Sequence[int],
        source_channels: Optional[int] = None,
        ratio: float = 1,
        groups: int = -1,
        update_source=True,
        update_filter=False,
        eps: float = 1e-16,
        num_iters: int = 1,
        num_grad_iters: Optional[int] = None,
        verbose: bool = False,
        **kwargs,
    ) -> None:
        super().__init__()
        self.channels = channels
        self.groups = channels if groups == -1 else groups
        assert self.channels % self.groups == 0, "`channels` must be divisible by groups"
        self.source_channels = round(
            channels * ratio / self.groups if source_channels is None else source_channels
        )
        self.kernel_size = tuple(kernel_size)
        self.init = Initializer(self.channels, self.source_channels, self.kernel_size, self.groups)
        self.update_source = update_source
        self.update_filter = update_filter
        self.num_iters = num_iters
        self.num_grad_iters = num_iters if num_grad_iters is None else num_grad_iters
        self.eps = eps
        self.verbose = verbose
        self.filter_channels = self.channels // self.groups
        self._conv_kwargs = dict(kwargs)
        self._padding = tuple(k // 2 for k in self.kernel_size)

    # ------------------------------------------------------------------ dispatch

    def unsupported_reason(self, x: Optional[Tensor] = None) -> Optional[str]:
        """Why this configuration (and input) cannot run, or None if it can."""
        if any(k % 2 == 0 for k in self.kernel_size):
            return "even kernel sizes are not supported"
        if not self.update_source:
            return "update_source=False is not supported"
        if self.update_filter:
            return "update_filter=True is not supported"
        if self.verbose:
            return "verbose=True is not supported"
        if self._conv_kwargs:
            return f"extra convolution arguments {sorted(self._conv_kwargs)} are not supported"
        if self.num_iters < 1:
            return "num_iters must be at least 1"
        if x is None:
            return None
        if not x.is_cuda:
            return f"input is on {x.device}; this layer runs on CUDA only"
        if x.dim() - 2 != len(self.kernel_size):
            return f"input rank {x.dim() - 2} does not match kernel_size {self.kernel_size}"
        if torch.is_autocast_enabled(x.device.type):
            return "autocast is not supported; cast the module and its input instead"
        if not kernels_apply(x, self.filter_channels, self.source_channels, self.kernel_size):
            return (f"dtype {x.dtype} / geometry m={self.filter_channels}, "
                    f"sc={self.source_channels}, k={self.kernel_size} is outside the kernels")
        return None

    def fast_path_applicable(self, x: Optional[Tensor] = None) -> bool:
        """Kept under the reference's name (`deconv.py:113-151`): whether the kernels apply."""
        return self.unsupported_reason(x) is None

    def context(self, it: int) -> Any:
        if it < self.num_iters - self.num_grad_iters + 1:
            return torch.no_grad()
        return nullcontext()

    def _fit(self, x: Tensor) -> tuple[Tensor, Tensor]:
        reason = self.unsupported_reason(x)
        if reason is not None:
            raise NotImplementedError(f"deconver_b200.Deconv: {reason}")
        x = x.contiguous()
        h = F.relu(self.init.h0)  # batch-invariant
        # the source enters the update pre-ReLU and pre-bias: the kernels apply both on load
        projection = self.init.linear.linear
        s = conv1x1(x.flatten(2), projection.weight)
        s = s.view(x.shape[0], -1, *x.shape[2:])
        bias = projection.bias
        rectify = True
        for it in range(1, self.num_iters + 1):
            with self.context(it):
                s = deconv_update(
                    x, s, h, bias,
                    groups=self.groups, m=self.filter_channels, sc=self.source_channels,
                    eps=self.eps, relu_input=rectify,
                )
            rectify = False
            bias = None  # later iterations start from an already biased, rectified source
        return s, h

    # ----------------------------------------------------------------- interface

    def fit(self, x: Tensor) -> tuple[Tensor, Tensor]:
        s, h = self._fit(x)
        # the filter is reported in its batched form, as the reference does
        return s, h.expand(x.shape[0], *h.shape).contiguous()

    def split_channels(self, v: Tensor) -> Tensor:
        # "b (g c) ... -> (b g) c ..."
        return v.reshape(v.shape[0] * self.groups, v.shape[1] // self.groups, *v.shape[2:])

    def merge_channels(self, v: Tensor) -> Tensor:
        return v.reshape(v.shape[0] // self.groups, self.groups * v.shape[1], *v.shape[2:])

    def reconstruct(self, s: Tensor, h: Tensor) -> Tensor:
        """``x_hat = conv(s, h)`` for a batched filter `h` of shape ``(B, C, sc, *k)``."""
        if self.groups != 1:
            s, h = self.split_channels(s), self.split_channels(h)
        x_hat = _batched_conv(s, h, self._padding)
        return self.merge_channels(x_hat) if self.groups != 1 else x_hat

    def loss(self, x: Tensor, s: Tensor, h: Tensor) -> Tensor:
        """Relative reconstruction error on channel-split tensors (`deconv.py:278-284`)."""
        y = _batched_conv(s, h, self._padding)
        num = (x - y).flatten(1).square().sum(1).sqrt() + 1e-16
        den = x.flatten(1).square().sum(1).sqrt() + 1e-16
        return num / den

    def forward(self, x: Tensor) -> Tensor:
        return self._fit(x)[0]


NDC = Deconv
