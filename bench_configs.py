"""Secondary measurements: the reference's Triton path on the same GPU, and the full-network
configurations (2-D forward, 3-D training step, large 3-D inference).

    python bench_configs.py --config triton      # layer: reference Triton path vs this library
    python bench_configs.py --config 1           # 2-D layer forward: reference on the host cores vs this library
    python bench_configs.py --config 2           # full 2-D Deconver forward, fp32 and bf16
    python bench_configs.py --config 4 [--gpus N under torchrun]   # 3-D training step, bf16
    python bench_configs.py --config 5           # large 3-D inference, bf16, NDC share

The U-Net around the NDC layer is not part of this library.  These runs take it, unmodified,
from an installation of the reference under `baseline/_ref` (made with
`pip install --no-deps --target baseline/_ref <reference checkout>`) and swap this library's
`Deconv` in by the same monkey-patch the reference's own tests use.  Without that directory
every configuration prints an `unavailable` line.  One JSON line per measurement.
"""

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "baseline", "_ref")

import torch


def emit(**kw):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(kw), flush=True)


def load_reference():
    if not os.path.isdir(os.path.join(REF, "deconver")):
        return None
    if REF not in sys.path:
        sys.path.insert(0, REF)
    import deconver  # noqa: F401
    return deconver


def timed(fn, iters=7, warmup=2):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return statistics.median(out)


class LayerClock:
    """Sums the device time spent inside every module of class `cls` (forward only)."""

    def __init__(self, model, cls):
        self.pairs = []
        for m in model.modules():
            if isinstance(m, cls):
                m.register_forward_pre_hook(self._pre)
                m.register_forward_hook(self._post)

    def _pre(self, m, inp):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pairs.append([e, None])

    def _post(self, m, inp, out):
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        self.pairs[-1][1] = e

    def reset(self):
        self.pairs = []

    def total_ms(self):
        torch.cuda.synchronize()
        return sum(a.elapsed_time(b) for a, b in self.pairs if b is not None)


def build_model(dc, use_b200, spatial_dims, in_ch, out_ch, widths, strides, depths_dec, ks, own_norm=True):
    import deconver.deconver as dm
    import deconver_b200
    from deconver.deconvolution.deconv import Deconv as RefDeconv

    # The network's own convolutions (stem, strided down/up-sampling, 1x1 head) are library
    # calls; let the library time its algorithms once per shape instead of trusting its
    # heuristic, which picks a 4.6x slower kernel for the stem at a per-GPU batch of 2.
    torch.backends.cudnn.benchmark = True
    norm = torch.nn.InstanceNorm3d if spatial_dims == 3 else torch.nn.InstanceNorm2d
    if use_b200 and own_norm:   # the same operator on this library's kernels
        norm = deconver_b200.InstanceNorm3d if spatial_dims == 3 else deconver_b200.InstanceNorm2d
    dm.Deconv = deconver_b200.Deconv if use_b200 else RefDeconv
    import deconver.layers.mlp as mlp_module
    ref_linear, ref_mlp = dm.Linear, dm.MLP
    if use_b200 and own_norm:   # the reference's Linear / MLP with this library's bias kernels
        dm.Linear = mlp_module.Linear = deconver_b200.Linear
        dm.MLP = deconver_b200.MLP
    try:
        torch.manual_seed(0)
        model = dc.Deconver(
            in_channels=in_ch, out_channels=out_ch, spatial_dims=spatial_dims,
            encoder_depth=(1,) * len(widths), encoder_width=widths, strides=strides,
            decoder_depth=depths_dec, norm=norm, act=torch.nn.ReLU, kernel_size=ks,
            groups=-1, ratio=4, num_iters=1, mlp_ratio=4,
        )
    finally:
        dm.Deconv = RefDeconv
        dm.Linear = mlp_module.Linear = ref_linear
        dm.MLP = ref_mlp
    return model, (deconver_b200.Deconv if use_b200 else RefDeconv)


# ------------------------------------------------------------------------------- configs


TRITON_CASES = {
    "cfg3": ("cfg3 3D layer", dict(channels=64, ratio=4, groups=-1, kernel_size=(3, 3, 3)), (2, 64, 64, 64, 64)),
    "cfg1": ("cfg1 2D layer", dict(channels=32, ratio=4, groups=-1, kernel_size=(5, 5)), (1, 32, 256, 256)),
}


def triton_record(dc, case="cfg3", dev=None):
    """Layer-level: reference `Deconv` (its Triton fast path) vs this library, same weights, on
    one GPU.  Returns a dict (times in ms, CUDA events, median of 7 after 2 warm-ups)."""
    import deconver_b200
    from deconver.deconvolution.deconv import Deconv as RefDeconv

    dev = dev or torch.device("cuda", torch.cuda.current_device())
    name, kw, shape = TRITON_CASES[case]
    torch.manual_seed(0)
    ref = RefDeconv(**kw).to(dev)
    mine = deconver_b200.Deconv(**kw).to(dev)
    mine.load_state_dict(ref.state_dict())
    x = torch.rand(*shape, device=dev)
    g = torch.randn(shape[0], 4 * shape[1], *shape[2:], device=dev)
    vox = shape[0]
    for s in shape[2:]:
        vox *= s
    res = {}
    for tag, mod in (("reference_triton", ref), ("b200", mine)):
        fast = bool(mod.fast_path_applicable(x))

        def fwd():
            with torch.no_grad():
                mod(x)

        def fwdbwd():
            xi = x.detach().requires_grad_(True)
            mod.zero_grad(set_to_none=True)
            mod(xi).backward(g)

        res[tag] = dict(fast_path=fast, fwd_ms=timed(fwd), fwd_bwd_ms=timed(fwdbwd))
    with torch.no_grad():
        a, b = ref(x), mine(x)
    err = float((a.double() - b.double()).abs().max() / b.double().abs().max())
    return dict(case=name, voxels=vox, forward_max_norm_diff=err, **res,
                speedup_fwd=res["reference_triton"]["fwd_ms"] / res["b200"]["fwd_ms"],
                speedup_fwd_bwd=res["reference_triton"]["fwd_bwd_ms"] / res["b200"]["fwd_bwd_ms"])


def config_triton(dc, args):
    for case in TRITON_CASES:
        emit(config="triton", **triton_record(dc, case, torch.device("cuda", 0)))


def config_1(dc, args):
    """Config 1 as BASELINE states it: one 2-D layer forward, fp32, X (1,32,256,256), seed 0,
    K = |N(0,1)|/25 — the reference's own module on the host cores (its general PyTorch path)
    next to this library on the GPU, same weights, with the difference between the two."""
    import os

    import deconver_b200
    from deconver.deconvolution.deconv import Deconv as RefDeconv

    kw = dict(channels=32, ratio=4, groups=-1, kernel_size=(5, 5))
    torch.manual_seed(0)
    ref = RefDeconv(**kw)
    with torch.no_grad():
        ref.init.h0.copy_(torch.randn(32, 4, 5, 5).abs() / 25)
    x = torch.rand(1, 32, 256, 256)
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    with torch.no_grad():
        for _ in range(2):
            y_cpu = ref(x)
        import time
        ts = []
        for _ in range(5):
            t0 = time.perf_counter()
            ref(x)
            ts.append((time.perf_counter() - t0) * 1e3)
    cpu_ms = sorted(ts)[len(ts) // 2]
    dev = torch.device("cuda", 0)
    # fp32 config: the 1x1 projection (a library convolution) runs without TF32 here
    torch.backends.cudnn.allow_tf32 = False
    torch.backends.cuda.matmul.allow_tf32 = False
    mine = deconver_b200.Deconv(**kw).to(dev)
    mine.load_state_dict(ref.state_dict())
    xd = x.to(dev)

    def fwd():
        with torch.no_grad():
            mine(xd)

    gpu_ms = timed(fwd)
    with torch.no_grad():
        y = mine(xd).cpu()
    err = float((y.double() - y_cpu.double()).abs().max() / y_cpu.double().abs().max())
    vox = 256 * 256
    emit(config=1, voxels=vox, forward_max_norm_diff=err,
         reference_cpu=dict(ms=cpu_ms, voxels_per_s=vox / cpu_ms * 1e3, cores=cores,
                            path="reference Deconv, general PyTorch path, fp32"),
         b200=dict(ms=gpu_ms, voxels_per_s=vox / gpu_ms * 1e3))


def forward2d_records(dc, with_reference=True):
    """Full 2-D Deconver forward, batch 16 x 3 x 256 x 256, fp32 and bf16, on one GPU.  Returns a
    list of records (this library in both dtypes; the reference's Triton path in fp32)."""
    dev = torch.device("cuda", torch.cuda.current_device())
    x0 = torch.rand(16, 3, 256, 256, device=dev)
    vox = 16 * 256 * 256
    out = []
    for dtype in (torch.float32, torch.bfloat16):
        for use_b200 in (True, False):
            if not use_b200 and (dtype != torch.float32 or not with_reference):
                continue  # the reference's Triton path is float32 only
            model, cls = build_model(dc, use_b200, 2, 3, 1, (32, 64, 128, 256, 512),
                                     (1, 2, 2, 2, 2), (1, 1, 1, 1), (5, 5))
            model = model.to(device=dev, dtype=dtype).eval()
            clock = LayerClock(model, cls)
            x = x0.to(dtype)

            def fwd():
                with torch.no_grad():
                    model(x)

            ms = timed(fwd)
            clock.reset()
            fwd()
            ndc = clock.total_ms()
            out.append(dict(impl="b200" if use_b200 else "reference_triton",
                            dtype=str(dtype).split(".")[-1], ms=ms, voxels_per_s=vox / ms * 1e3,
                            ndc_layers=len(clock.pairs), ndc_ms=ndc, ndc_share=ndc / ms))
            del model
    return out


def config_2(dc, args):
    for rec in forward2d_records(dc):
        emit(config=2, **rec)


def train_step_record(dc, steps=10, graph=False, per_gpu_batch=0):
    """Full 3-D training step (fwd + bwd + SGD), bf16, global batch 16 of 2 x 64^3, batch
    sharded over the ranks of the current process group (strong scaling), NCCL all-reduce of
    all parameter gradients.  The reference has no loss or optimizer: BCE-with-logits and plain
    SGD stand in.  Returns a dict; ms_per_step is the maximum over ranks (CUDA events)."""
    import torch.distributed as dist
    from deconver_b200.distributed import GradBucket, init_from_env, shard_batch

    rank, world, local = init_from_env("nccl")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    model, cls = build_model(dc, True, 3, 2, 1, (64, 128, 256, 512), (1, 2, 2, 2), (1, 1, 1), (3, 3, 3))
    model = model.to(device=dev, dtype=torch.bfloat16).train()
    sl = shard_batch(16, rank, world)
    gen = torch.Generator(device=dev).manual_seed(100 + rank)
    nb = per_gpu_batch or (sl.stop - sl.start)
    x = torch.rand(nb, 2, 64, 64, 64, device=dev, generator=gen).to(torch.bfloat16)
    y = (torch.rand(nb, 1, 64, 64, 64, device=dev, generator=gen) < 0.05).to(torch.bfloat16)
    params = [p for p in model.parameters() if p.requires_grad]
    bucket = GradBucket(params)
    opt = torch.optim.SGD(params, lr=1e-2, momentum=0.0)
    clock = LayerClock(model, cls)

    def fwd_bwd():
        out = model(x)
        # mean over the local shard; equal shards, so the rank average is the global-batch mean
        loss = torch.nn.functional.binary_cross_entropy_with_logits(out.float(), y.float())
        loss.backward()
        return loss

    def eager_step():
        for p in params:
            p.grad = None
        loss = fwd_bwd()
        bucket.allreduce_mean()
        opt.step()
        return loss

    step = eager_step
    if graph:
        # forward + backward + gradient gather replayed as one CUDA graph (x, y and the
        # gradients keep their addresses); the all-reduce and the optimizer stay outside
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                eager_step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        for p in params:
            p.grad = None
        cuda_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cuda_graph):
            static_loss = fwd_bwd()
            bucket.gather()

        def step():
            cuda_graph.replay()
            bucket.allreduce_mean(gather=False)
            opt.step()
            return static_loss

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = step()
    b.record()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    clock.reset()
    with torch.no_grad():
        model(x)
    ndc_fwd = clock.total_ms()
    return dict(n_gpus=world, global_batch=16, per_gpu_batch=nb, dtype="bfloat16",
                cuda_graph=bool(graph), cudnn_benchmark=bool(torch.backends.cudnn.benchmark),
                steps=steps, ms_per_step=ms, voxels_per_s=16 * 64 ** 3 / ms * 1e3, loss=float(loss.detach()),
                ndc_forward_ms_per_rank=ndc_fwd, params=sum(p.numel() for p in params))


def config_4(dc, args):
    import torch.distributed as dist

    emit(config=4, **train_step_record(dc, args.steps, args.graph, args.per_gpu_batch))
    if dist.is_initialized():
        dist.destroy_process_group()


def inference_record(dc, chunk=4):
    """Large 3-D inference, bf16: batch 32 of 4 x 128^3 (relu(N(0,1))), batch-sharded over the
    ranks of the current process group with no collective, processed in chunks of `chunk`
    samples per GPU; reports the NDC share of the end-to-end time."""
    from deconver_b200.distributed import init_from_env, shard_batch
    import torch.distributed as dist

    rank, world, local = init_from_env("nccl")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    model, cls = build_model(dc, True, 3, 4, 3, (64, 128, 256, 512), (1, 2, 2, 2), (1, 1, 1), (3, 3, 3))
    model = model.to(device=dev, dtype=torch.bfloat16).eval()
    clock = LayerClock(model, cls)
    sl = shard_batch(32, rank, world)
    nb = sl.stop - sl.start
    gen = torch.Generator(device=dev).manual_seed(7 + rank)
    chunk = min(chunk, nb)
    xs = [torch.relu(torch.randn(chunk, 4, 128, 128, 128, device=dev, generator=gen)).to(torch.bfloat16)
          for _ in range(2)]

    def run():
        with torch.no_grad():
            for i in range(0, nb, chunk):
                model(xs[(i // chunk) % 2])

    ms = timed(run, iters=3, warmup=1)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    clock.reset()
    run()
    ndc = clock.total_ms()
    return dict(n_gpus=world, batch=32, per_gpu_batch=nb, chunk=chunk, dtype="bfloat16", ms=ms,
                voxels_per_s=32 * 128 ** 3 / ms * 1e3, ndc_ms_per_rank=ndc, ndc_share=ndc / ms)


def config_5(dc, args):
    import torch.distributed as dist

    emit(config=5, **inference_record(dc, args.chunk))
    if dist.is_initialized():
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--config", required=True, choices=["triton", "1", "2", "4", "5"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--chunk", type=int, default=4)
    ap.add_argument("--graph", action="store_true",
                    help="config 4: replay forward+backward as one CUDA graph")
    ap.add_argument("--per-gpu-batch", type=int, default=0,
                    help="config 4: override the per-GPU batch (single-GPU experiments)")
    args = ap.parse_args()
    dc = load_reference()
    if dc is None:
        emit(config=args.config, unavailable="baseline/_ref (an installation of the reference) is not present")
        return
    if not torch.cuda.is_available():
        emit(config=args.config, unavailable="no CUDA device")
        return
    {"triton": config_triton, "1": config_1, "2": config_2, "4": config_4, "5": config_5}[args.config](dc, args)


if __name__ == "__main__":
    main()
