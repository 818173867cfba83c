"""Autograd node for one multiplicative NDC update, on the sm_100a kernels.

Same interface as the reference's `deconver/deconvolution/functional.py`:
`DeconvUpdate.forward(ctx, x, z, h, bias, groups, m, sc, eps, relu_input)`,
`DeconvUpdate.backward(ctx, gout)` returning a 9-tuple, and
`deconv_update(x, z, h, bias, *, groups, m, sc, eps, relu_input)`
(`functional.py:97-207` there).  The arithmetic is

    s    = relu(z + b)
    t1   = K(s)
    out  = (s * (A(x) + eps)) / (A(t1) + eps)          A = K^T

and only `x`, `z` and `t1` are kept for backward.  There is no Triton, no backend selection
and no CPU path: tensors must live on a CUDA device and be float32 or bfloat16.
"""

import contextlib
import ctypes
import warnings
from typing import Optional, Sequence

import torch
from torch import Tensor

from . import _lib

__all__ = ["DeconvUpdate", "deconv_update", "kernels_apply", "gconv", "force_generic"]

_DTYPES = {torch.float32: _lib.NDC_F32, torch.bfloat16: _lib.NDC_BF16}

_flags = 0


@contextlib.contextmanager
def force_generic(enabled: bool = True):
    """Run the generic kernels even where the tiled depthwise ones apply (for cross-checks)."""
    global _flags
    old = _flags
    _flags = _lib.FLAG_FORCE_GENERIC if enabled else 0
    try:
        yield
    finally:
        _flags = old


_NO_SPAN = contextlib.nullcontext()


def _on_device(device):
    """Device guard for the C-ABI calls; free when `device` is already the current one."""
    if device.index is None or device.index == torch.cuda.current_device():
        return _NO_SPAN
    return torch.cuda.device(device)


class _Timing:
    """Optional CUDA-event timing of the C-ABI calls, on the stream they are issued on.

    Off by default.  `enable()` starts collecting; `disable_and_collect()` synchronises and
    returns ``{"ndc_fwd": [ms, ...], "ndc_bwd": [ms, ...]}``.
    """

    def __init__(self) -> None:
        self.enabled = False
        self._events = {"ndc_fwd": [], "ndc_bwd": []}

    def enable(self) -> None:
        self._events = {"ndc_fwd": [], "ndc_bwd": []}
        self.enabled = True

    def span(self, name: str):
        return self._span(name) if self.enabled else _NO_SPAN

    @contextlib.contextmanager
    def _span(self, name: str):
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            yield
        finally:
            stop.record()
            self._events[name].append((start, stop))

    def disable_and_collect(self):
        self.enabled = False
        torch.cuda.synchronize()
        return {k: [a.elapsed_time(b) for a, b in v] for k, v in self._events.items()}


timing = _Timing()


_kernels_apply_cache = {}


def kernels_apply(x: Tensor, m: int, sc: int, kernel_size: Sequence[int]) -> bool:
    """Whether the CUDA kernels cover this input and filter geometry.

    Takes the place of the reference's `fused_kernels_apply` (`functional.py:34-47`).
    """
    if not (x.is_cuda and x.dtype in _DTYPES and 1 <= x.dim() - 2 <= 3):
        return False
    if len(kernel_size) != x.dim() - 2 or any(k % 2 == 0 for k in kernel_size):
        return False
    # the answer depends on the geometry only: asked once per geometry, not once per call
    key = (x.dtype, x.shape[0], tuple(x.shape[2:]), m, sc, tuple(kernel_size))
    known = _kernels_apply_cache.get(key)
    if known is None:
        desc = _lib.make_desc(max(x.shape[0], 1), 1, m, sc, [max(v, 1) for v in x.shape[2:]],
                              kernel_size, 0.0, True, _DTYPES[x.dtype])
        known = _lib.load().ndc_query(desc, None) == _lib.NDC_OK
        if len(_kernels_apply_cache) < 4096:
            _kernels_apply_cache[key] = known
    return known


_warned_generic = set()
_checked_tiled = set()     # geometries already known to run on the tiled kernels


def _warn_if_generic(desc, flags: int) -> None:
    """Depthwise ratio-4 problems normally run on the tiled kernels; tell the user (once per
    geometry class) when one falls outside them and takes the much slower generic kernels."""
    if flags & _lib.FLAG_FORCE_GENERIC or desc.m != 1 or desc.sc != 4:
        return
    key = (desc.kD, desc.kH, desc.kW, desc.W > 256, desc.dtype)
    if key in _warned_generic:
        return
    seen = (desc.batch, desc.groups, desc.D, desc.H, desc.W, desc.kD, desc.kH, desc.kW, desc.dtype)
    if seen in _checked_tiled:
        return
    path = ctypes.c_int32(-1)
    status = _lib.load().ndc_query(desc, ctypes.byref(path))
    if status == _lib.NDC_OK and path.value != _lib.PATH_GENERIC and len(_checked_tiled) < 4096:
        _checked_tiled.add(seen)
    if status == _lib.NDC_OK and path.value == _lib.PATH_GENERIC:
        _warned_generic.add(key)
        warnings.warn(
            f"deconver_b200: depthwise ratio-4 update with kernel ({desc.kD},{desc.kH},{desc.kW}) on "
            f"({desc.D},{desc.H},{desc.W}) runs on the generic kernels (about 20x slower per voxel); "
            "the tiled kernels cover 3x3x3 volumes up to 256 columns and 5x5 / 3x3 images up to 512",
            RuntimeWarning, stacklevel=3)


def _require(t: Optional[Tensor], name: str, like: Tensor) -> None:
    if t is None:
        return
    if not t.is_cuda:
        raise RuntimeError(
            f"deconver_b200: `{name}` is on {t.device}; the NDC update runs on CUDA only "
            "(there is no CPU path)"
        )
    if t.device != like.device:
        raise RuntimeError(f"deconver_b200: `{name}` is on {t.device}, expected {like.device}")


def _ptr(t: Optional[Tensor]):
    return None if t is None else t.data_ptr()


def _f32(t: Optional[Tensor]) -> Optional[Tensor]:
    """Filter and bias are handed to the kernels in float32 whatever the model's dtype."""
    if t is None:
        return None
    t = t.detach()
    if t.dtype != torch.float32:
        t = t.to(torch.float32)
    return t if t.is_contiguous() else t.contiguous()


def _desc(x: Tensor, groups: int, m: int, sc: int, ks, eps: float, relu_input: bool,
          flags: Optional[int] = None):
    if x.dtype not in _DTYPES:
        raise NotImplementedError(
            f"deconver_b200: dtype {x.dtype} is not supported (float32 and bfloat16 are)"
        )
    return _lib.make_desc(x.shape[0], groups, m, sc, x.shape[2:], ks, eps, relu_input,
                          _DTYPES[x.dtype], _flags if flags is None else flags)


def _check_shapes(x, z, h, bias, groups, m, sc):
    if x.dim() != z.dim() or x.shape[0] != z.shape[0] or x.shape[2:] != z.shape[2:]:
        raise ValueError(f"x {tuple(x.shape)} and z {tuple(z.shape)} do not match")
    if x.shape[1] != groups * m or z.shape[1] != groups * sc:
        raise ValueError(
            f"channel counts {x.shape[1]}, {z.shape[1]} do not match groups={groups}, m={m}, sc={sc}"
        )
    if h.shape[0] != groups * m or h.shape[1] != sc or h.dim() != x.dim():
        raise ValueError(f"filter {tuple(h.shape)} does not match groups={groups}, m={m}, sc={sc}")
    if bias is not None and bias.numel() != groups * sc:
        raise ValueError(f"bias has {bias.numel()} elements, expected {groups * sc}")
    if z.dtype != x.dtype:
        raise ValueError(f"x is {x.dtype} but z is {z.dtype}")


class DeconvUpdate(torch.autograd.Function):
    """``out = relu(z + b) * (A(x) + eps) / (A(K(relu(z + b))) + eps)``."""

    @staticmethod
    def forward(ctx, x, z, h, bias, groups, m, sc, eps, relu_input):
        for name, t in (("x", x), ("z", z), ("h", h), ("bias", bias)):
            _require(t, name, x)
        _check_shapes(x, z, h, bias, groups, m, sc)
        x = x.contiguous()
        z = z.contiguous()
        ks = tuple(h.shape[2:])
        flags = _flags   # read once: backward runs later, on an autograd thread
        desc = _desc(x, groups, m, sc, ks, eps, relu_input, flags)
        _warn_if_generic(desc, flags)
        hf, bf = _f32(h), _f32(bias)
        out = torch.empty_like(z)
        t1 = torch.empty_like(x)
        if x.numel() and z.numel():
            with _on_device(x.device):
                stream = torch.cuda.current_stream().cuda_stream
                with timing.span("ndc_fwd"):
                    _lib.check(_lib.load().ndc_fwd(desc, _ptr(x), _ptr(z), _ptr(hf), _ptr(bf),
                                                   _ptr(out), _ptr(t1), stream))
        ctx.cfg = (groups, m, sc, eps, relu_input, flags)
        ctx.save_for_backward(x, z, t1, h, bias)
        return out

    @staticmethod
    def backward(ctx, gout):
        # The backward runs kernels autograd cannot see through, so it is not itself
        # differentiable; the engine enables grad here exactly when the caller asked for
        # create_graph=True (same refusal as the reference, functional.py:126-132).
        if torch.is_grad_enabled():
            raise RuntimeError(
                "double backward through the fused Deconv update is not supported"
            )
        x, z, t1, h, bias = ctx.saved_tensors
        groups, m, sc, eps, relu_input, flags = ctx.cfg
        need_x, need_z, need_h, need_b = ctx.needs_input_grad[:4]
        need_b = need_b and bias is not None
        if not (need_x or need_z or need_h or need_b):
            return (None,) * 9
        _require(gout, "gout", x)
        gout = gout.contiguous()
        if gout.dtype != x.dtype:
            gout = gout.to(x.dtype)
        ks = tuple(h.shape[2:])
        desc = _desc(x, groups, m, sc, ks, eps, relu_input, flags)
        hf, bf = _f32(h), _f32(bias)
        gx = torch.empty_like(x) if need_x else None
        gz = torch.empty_like(z) if (need_z or need_b) else None
        gh = torch.empty(h.shape, device=x.device, dtype=torch.float32) if need_h else None
        gb = torch.empty(bias.shape, device=x.device, dtype=torch.float32) if need_b else None
        if x.numel() and z.numel():
            lib = _lib.load()
            with _on_device(x.device):
                nbytes = lib.ndc_bwd_workspace_bytes(desc)
                ws = torch.empty(max(nbytes, 1), device=x.device, dtype=torch.uint8)
                stream = torch.cuda.current_stream().cuda_stream
                with timing.span("ndc_bwd"):
                    _lib.check(lib.ndc_bwd(desc, _ptr(x), _ptr(z), _ptr(t1), _ptr(hf), _ptr(bf),
                                           _ptr(gout), _ptr(gx), _ptr(gz), _ptr(gh), _ptr(gb),
                                           _ptr(ws), nbytes, stream))
                # `ws` is released to the caching allocator here; later work on this stream
                # is ordered after the kernels that use it
        else:
            for t in (gx, gz, gh, gb):
                if t is not None:
                    t.zero_()
        if gh is not None and gh.dtype != h.dtype:
            gh = gh.to(h.dtype)
        if gb is not None and gb.dtype != bias.dtype:
            gb = gb.to(bias.dtype)
        return gx, gz if need_z else None, gh, gb, None, None, None, None, None


def deconv_update(
    x: Tensor,
    z: Tensor,
    h: Tensor,
    bias: Optional[Tensor],
    *,
    groups: int,
    m: int,
    sc: int,
    eps: float,
    relu_input: bool,
) -> Tensor:
    """One multiplicative source update.

    Args:
        x: input, ``(B, C, *S)``.
        z: projection output, ``(B, groups * sc, *S)``, pre-bias and pre-ReLU.
        h: rectified filter, ``(C, sc, *k)``.
        bias: the projection's bias (or None), folded in by the kernels.
        eps: stabiliser added to the numerator and the denominator.
    """
    return DeconvUpdate.apply(x, z, h, bias, groups, m, sc, eps, relu_input)


def gconv(inp: Tensor, h: Tensor, *, groups: int, m: int, sc: int, adjoint: bool,
          relu_input: bool = False, bias: Optional[Tensor] = None) -> Tensor:
    """Grouped convolution ``K`` (``adjoint=False``) or its adjoint ``A``; no autograd.

    Counterpart of the reference's `kernels.gconv` (`kernels.py:728-759`).
    """
    _require(inp, "inp", inp)
    _require(h, "h", inp)
    inp = inp.contiguous()
    cout = sc if adjoint else m
    desc = _desc(inp, groups, m, sc, tuple(h.shape[2:]), 0.0, relu_input)
    out = torch.empty(inp.shape[0], groups * cout, *inp.shape[2:], device=inp.device,
                      dtype=inp.dtype)
    hf, bf = _f32(h), _f32(bias)
    if inp.numel():
        with torch.cuda.device(inp.device):
            stream = torch.cuda.current_stream().cuda_stream
            _lib.check(_lib.load().ndc_gconv(desc, _ptr(inp), _ptr(hf), _ptr(bf), int(adjoint),
                                             _ptr(out), stream))
    return out
