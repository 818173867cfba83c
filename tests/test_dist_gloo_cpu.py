"""The multi-rank path on CPU: two `gloo` ranks, batch sharding, one gradient bucket.

The layer itself has no CPU path, so each rank computes its shard's gradients with the CPU
oracle; what is tested is the product's sharding and bucket/all-reduce logic: the averaged
bucket must equal the gradient of the mean loss over the whole batch on one process."""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from deconver_b200.distributed import GradBucket, shard_batch


def test_shard_batch_partitions_exactly():
    for total in (1, 2, 7, 16, 32):
        for world in (1, 2, 4, 8):
            parts = [shard_batch(total, r, world) for r in range(world)]
            covered = [i for p in parts for i in range(p.start, p.stop)]
            assert covered == list(range(total))
            sizes = [p.stop - p.start for p in parts]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_batch(4, 4, 4)


def test_bucket_views_and_single_process():
    lin = torch.nn.Linear(5, 3)
    bucket = GradBucket(lin.parameters())
    assert lin.weight.grad.data_ptr() == bucket.flat.data_ptr()
    lin(torch.ones(2, 5)).sum().backward()
    assert torch.equal(bucket.flat[:15].view(3, 5), lin.weight.grad)
    assert float(bucket.flat[:15].sum()) == 30.0
    assert bucket.allreduce_mean() is None  # no process group: nothing to reduce
    bucket.zero()
    assert float(bucket.flat.abs().sum()) == 0.0 and lin.weight.grad.data_ptr() == bucket.flat.data_ptr()
    with pytest.raises(ValueError):
        GradBucket([])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _layer_params(seed):
    gen = torch.Generator().manual_seed(seed)
    C, sc, ks = 4, 4, (3, 3, 3)
    w = torch.nn.Parameter(torch.randn(C * sc, C, 1, generator=gen) * 0.3)
    b = torch.nn.Parameter(torch.rand(C * sc, generator=gen) + 0.5)
    h0 = torch.nn.Parameter(torch.rand(C, sc, *ks, generator=gen) / 27)
    return [w, b, h0]


def _loss(params, x, g):
    from oracle import ndc_oracle
    w, b, h0 = params
    y = ndc_oracle.ndc_layer(x, w, b, h0, groups=4)
    return (y * g).sum() / x.shape[0]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank),
                      WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        gen = torch.Generator().manual_seed(7)
        x = torch.rand(4, 4, 5, 6, 7, generator=gen)
        g = torch.randn(4, 16, 5, 6, 7, generator=gen)
        params = _layer_params(3)
        bucket = GradBucket(params)
        sl = shard_batch(x.shape[0], rank, world)
        _loss(params, x[sl], g[sl]).backward()
        pending = bucket.allreduce_mean(async_op=True)
        pending.wait()
        if rank == 0:
            torch.save([p.grad.clone() for p in params], out)
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_average_to_the_global_gradient(tmp_path):
    out = str(tmp_path / "grads.pt")
    port = _free_port()
    mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
    got = torch.load(out)
    gen = torch.Generator().manual_seed(7)
    x = torch.rand(4, 4, 5, 6, 7, generator=gen)
    g = torch.randn(4, 16, 5, 6, 7, generator=gen)
    params = _layer_params(3)
    _loss(params, x, g).backward()
    for a, p in zip(got, params):
        assert torch.allclose(a, p.grad, rtol=1e-4, atol=1e-6)
