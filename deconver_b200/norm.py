"""Instance normalisation on the library's own CUDA kernels.

`InstanceNorm1d/2d/3d` take the constructor arguments of `torch.nn.InstanceNorm{1,2,3}d` and can
be handed to the reference's network wherever it takes a `norm` class (`DeconverBlock`,
`deconver/deconver.py:52-65`; the published configurations pass `torch.nn.InstanceNorm3d`).
torch's kernel works with one block per (sample, channel) slab; at the small per-GPU batches of a
batch-sharded training step that is fewer blocks than the GPU has multiprocessors.  The kernels
behind this module split every slab over enough blocks to fill the device
(`csrc/ndc_inorm.cu`).

CUDA tensors, float32 or bfloat16 (statistics always in float32); no running statistics.
"""

from typing import Optional

import torch
from torch import Tensor, nn
from torch.autograd.function import once_differentiable

from . import _lib

__all__ = ["InstanceNorm1d", "InstanceNorm2d", "InstanceNorm3d", "instance_norm"]

_DTYPES = {torch.float32: _lib.NDC_F32, torch.bfloat16: _lib.NDC_BF16}


def _check(status: int) -> None:
    if status != _lib.NDC_OK:
        msg = _lib.load().ndc_inorm_last_error().decode("utf-8", "replace")
        raise _lib.NdcError(status, msg)


def _f32(t: Optional[Tensor]) -> Optional[Tensor]:
    return None if t is None else t.detach().to(torch.float32).contiguous()


def _ptr(t: Optional[Tensor]):
    return None if t is None else t.data_ptr()


class _InstanceNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        if not x.is_cuda:
            raise RuntimeError(f"deconver_b200: instance norm input is on {x.device}; CUDA only")
        if x.dtype not in _DTYPES:
            raise NotImplementedError(f"deconver_b200: instance norm of {x.dtype} is not supported")
        if x.dim() < 3:
            raise ValueError("instance norm expects (batch, channels, spatial...)")
        x = x.contiguous()
        B, C = x.shape[:2]
        sp = x[0, 0].numel()
        y = torch.empty_like(x)
        stats = torch.empty(B * C * 2, device=x.device, dtype=torch.float32)
        wf, bf = _f32(weight), _f32(bias)
        if x.numel():
            lib = _lib.load()
            with torch.cuda.device(x.device):
                nbytes = lib.ndc_inorm_workspace_bytes(B, C)
                ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
                stream = torch.cuda.current_stream().cuda_stream
                _check(lib.ndc_inorm_fwd(B, C, sp, _DTYPES[x.dtype], _ptr(x), _ptr(wf), _ptr(bf),
                                         float(eps), _ptr(y), _ptr(stats), _ptr(ws), nbytes, stream))
        ctx.save_for_backward(x, weight, stats)
        ctx.has_bias = bias is not None
        return y

    @staticmethod
    @once_differentiable
    def backward(ctx, gy):
        x, weight, stats = ctx.saved_tensors
        need_x, need_w, need_b = ctx.needs_input_grad[:3]
        need_w = need_w and weight is not None
        need_b = need_b and ctx.has_bias
        B, C = x.shape[:2]
        sp = x[0, 0].numel()
        gy = gy.contiguous()
        if gy.dtype != x.dtype:
            gy = gy.to(x.dtype)
        gx = torch.empty_like(x)
        gw = torch.empty(C, device=x.device, dtype=torch.float32) if need_w else None
        gb = torch.empty(C, device=x.device, dtype=torch.float32) if need_b else None
        if x.numel():
            lib = _lib.load()
            with torch.cuda.device(x.device):
                nbytes = lib.ndc_inorm_workspace_bytes(B, C)
                ws = torch.empty(nbytes, device=x.device, dtype=torch.uint8)
                stream = torch.cuda.current_stream().cuda_stream
                _check(lib.ndc_inorm_bwd(B, C, sp, _DTYPES[x.dtype], _ptr(x), _ptr(gy),
                                         _ptr(_f32(weight)), _ptr(stats), _ptr(gx), _ptr(gw), _ptr(gb),
                                         _ptr(ws), nbytes, stream))
        else:
            for t in (gw, gb):
                if t is not None:
                    t.zero_()
        if gw is not None and gw.dtype != weight.dtype:
            gw = gw.to(weight.dtype)
        if gb is not None and weight is not None and gb.dtype != weight.dtype:
            gb = gb.to(weight.dtype)
        return gx if need_x else None, gw, gb, None


def instance_norm(x: Tensor, weight: Optional[Tensor] = None, bias: Optional[Tensor] = None,
                  eps: float = 1e-5) -> Tensor:
    """``(x - mean) / sqrt(var + eps) [* weight + bias]`` per (sample, channel), biased variance."""
    return _InstanceNormFn.apply(x, weight, bias, eps)


class _InstanceNorm(nn.Module):
    _rank = 0

    def __init__(self, num_features: int, eps: float = 1e-5, momentum: Optional[float] = 0.1,
                 affine: bool = False, track_running_stats: bool = False, device=None,
                 dtype=None) -> None:
        super().__init__()
        if track_running_stats:
            raise NotImplementedError("deconver_b200: running statistics are not supported")
        self.num_features, self.eps, self.momentum, self.affine = num_features, eps, momentum, affine
        self.track_running_stats = False
        if affine:
            kw = dict(device=device, dtype=dtype)
            self.weight = nn.Parameter(torch.ones(num_features, **kw))
            self.bias = nn.Parameter(torch.zeros(num_features, **kw))
        else:
            self.register_parameter("weight", None)
            self.register_parameter("bias", None)

    def forward(self, x: Tensor) -> Tensor:
        if x.dim() != self._rank + 2:
            raise ValueError(f"expected a {self._rank + 2}-D input (got {x.dim()}-D)")
        if x.shape[1] != self.num_features:
            raise ValueError(f"expected {self.num_features} channels (got {x.shape[1]})")
        return instance_norm(x, self.weight, self.bias, self.eps)

    def extra_repr(self) -> str:
        return f"{self.num_features}, eps={self.eps}, affine={self.affine}"


class InstanceNorm1d(_InstanceNorm):
    _rank = 1


class InstanceNorm2d(_InstanceNorm):
    _rank = 2


class InstanceNorm3d(_InstanceNorm):
    _rank = 3
