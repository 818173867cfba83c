"""Batch-sharded data parallelism for the NDC layer: one process per GPU, one flat gradient
bucket, one all-reduce.

The reference has no distributed code.  Every operator of the layer is per sample, so the
forward pass needs no exchange; a training step exchanges only the parameter gradients (the
filter gradient dK = `init.h0.grad`, and the projection's weight and bias gradients).

`GradBucket` keeps all gradients of a parameter list in one contiguous float32 buffer and
points each `param.grad` at its slice, so backward accumulates straight into the bucket and
the all-reduce moves one tensor.  It works with any `torch.distributed` backend (NCCL over
NVLink on GPUs; gloo on CPUs for tests).
"""

import os
from typing import Iterable, List, Optional

import torch
import torch.distributed as dist

__all__ = ["GradBucket", "init_from_env", "shard_batch"]


def init_from_env(backend: Optional[str] = None) -> tuple[int, int, int]:
    """Join the process group torchrun describes.  Returns ``(rank, world_size, local_rank)``.

    Without torchrun's environment this is a single-process run and no group is made.
    """
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(local)
            dist.init_process_group(backend, device_id=torch.device("cuda", local))
        else:
            dist.init_process_group(backend)
    return rank, world, local


def shard_batch(global_batch: int, rank: int, world: int) -> slice:
    """Contiguous slice of the global batch owned by `rank` (sizes differ by at most one)."""
    if not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    base, extra = divmod(global_batch, world)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


class GradBucket:
    """All gradients of `params` in one flat float32 buffer, reduced with one collective."""

    def __init__(self, params: Iterable[torch.nn.Parameter], group=None) -> None:
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        if not self.params:
            raise ValueError("GradBucket needs at least one parameter that requires grad")
        dev = self.params[0].device
        if any(p.device != dev for p in self.params):
            raise ValueError("all parameters of a bucket must live on one device")
        self.group = group
        sizes = [p.numel() for p in self.params]
        # 64-element (256-byte) alignment of every slice keeps vector accesses aligned
        self.offsets = []
        total = 0
        for n in sizes:
            self.offsets.append(total)
            total += (n + 63) // 64 * 64
        self.flat = torch.zeros(total, device=dev, dtype=torch.float32)
        self._views = [self.flat[o:o + n].view(p.shape)
                       for o, n, p in zip(self.offsets, sizes, self.params)]
        self.attach()

    def attach(self) -> None:
        """Point every float32 `param.grad` at its slice (others are copied in `gather`)."""
        for p, v in zip(self.params, self._views):
            if p.dtype == torch.float32:
                p.grad = v

    def zero(self) -> None:
        self.flat.zero_()
        self.attach()

    def gather(self) -> None:
        """Bring gradients that autograd placed elsewhere (or in another dtype) into the bucket:
        one multi-tensor copy, not one launch per parameter."""
        src, dst = [], []
        for p, v in zip(self.params, self._views):
            if p.grad is None:
                v.zero_()
            elif p.grad.data_ptr() != v.data_ptr():
                src.append(p.grad)
                dst.append(v)
        if dst:
            torch._foreach_copy_(dst, src)

    def scatter(self) -> None:
        """Write reduced values back to gradients that are not views of the bucket."""
        src, dst = [], []
        for p, v in zip(self.params, self._views):
            if p.grad is not None and p.grad.data_ptr() != v.data_ptr():
                src.append(v)
                dst.append(p.grad)
        if dst:
            torch._foreach_copy_(dst, src)

    def allreduce_mean(self, async_op: bool = False, gather: bool = True):
        """Average the bucket over the group (sum, then scale by 1/world).  `gather=False` when
        the caller has already gathered (e.g. inside a captured graph)."""
        if gather:
            self.gather()
        if not dist.is_initialized() or dist.get_world_size(self.group) == 1:
            return None
        world = dist.get_world_size(self.group)
        work = dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=self.group, async_op=async_op)
        if async_op:
            return _Pending(self, work, world)
        self.flat.mul_(1.0 / world)
        self.scatter()
        return None


class _Pending:
    def __init__(self, bucket: GradBucket, work, world: int) -> None:
        self.bucket, self.work, self.world = bucket, work, world

    def wait(self) -> None:
        self.work.wait()
        self.bucket.flat.mul_(1.0 / self.world)
        self.bucket.scatter()
