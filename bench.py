"""Benchmark of the NDC mixer layer (forward + backward) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

One JSON line is printed by rank 0.  A "step" is one forward + backward of a single 3-D NDC
layer on one batch of synthetic input resident in HBM:

    NDC(channels=64, ratio=4, groups=-1, kernel_size=(3,3,3)), fp32,
    X = rand(2, 64, 64, 64, 64), h0 = |randn|/27, upstream gradient randn(2, 256, 64, 64, 64)

`value` is voxels/s (one voxel = one spatial site of one sample), aggregated over all ranks.
With N > 1 every rank works on its own batch of 2 (weak scaling, batch sharding) and the
parameter gradients (dK, projection weight and bias) are averaged with one NCCL all-reduce
inside the step.  `e2e` is the same step through the public `Deconv` module with pinned HOST
input and upstream gradient, host<->device copies inside the timed region.

`--impl reference` times the reference's own CPU implementation of the same layer
(`ReferenceDeconv`, imported from an installation of the reference under `baseline/_ref`;
the oracle's port of it when that directory is absent) on all host cores.

Sub-records ride along on the GPU arm when `baseline/_ref` is importable: `train_step` (the
full 3-D network's training step, global batch 16 split over the ranks) and `inference` (the
large 3-D inference configuration, batch 32 split over the ranks) at every N; `triton` (the
reference's own Triton kernels on the same GPU and layer) and `forward_2d` (the full 2-D
network's forward) at N = 1 only.

`--profile-case` runs a few update calls on a small case and nothing else: the command the
ncu summaries under `profiles/` were captured with.
"""

import argparse
import ctypes
import json
import math
import os
import re
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "baseline", "_ref")

import torch

METRIC = "ndc_mixer_fwd_bwd_voxels_per_sec"
UNIT = "voxels/s"
WORKLOAD = dict(channels=64, ratio=4, kernel_size=(3, 3, 3), batch=2, spatial=(64, 64, 64))
WORKLOAD_NAME = ("single 3D NDC mixer layer fwd+bwd (dX, dK), fp32, X (2,64,64,64,64), "
                 "source 256 ch, K (256,1,3,3,3)")
# DRAM traffic of one backward call, from an ncu capture at batch 1 (traffic is proportional to
# voxels: every CTA works on its own slab); the capture's summary carries the figure
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "ndc_bwd_cfg3_b1_dram_traffic.txt")


def config_of(world):
    """The `config` object: the same for both arms, so their lines compare like with like."""
    B = WORKLOAD["batch"]
    return {
        "workload": WORKLOAD_NAME, "per_gpu_batch": B, "global_batch": B * world,
        "parallelism": f"batch-sharded x{world}" + (", NCCL grad all-reduce" if world > 1 else ""),
        "l2": "inputs larger than L2 (x 134 MB, z/out/gout 537 MB each vs 126 MB L2)",
    }


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def load_traffic(batch):
    """(bytes per backward call at `batch`, provenance) from the tracked ncu summary, or
    (None, reason)."""
    try:
        text = open(TRAFFIC_FILE).read()
        per_b1 = int(re.search(r"^dram_bytes_per_call_batch1\s*=\s*(\d+)", text, re.M).group(1))
        return per_b1 * batch, os.path.relpath(TRAFFIC_FILE, ROOT) + " (ncu, batch 1, scaled by batch)"
    except Exception as exc:  # missing or unreadable summary: no figure rather than a stale one
        return None, f"unavailable: {exc}"


# ----------------------------------------------------------------------------- clocks


class ClockSampler:
    """Samples SM clock and throttle reasons (read-only NVML queries) while a region runs."""

    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap",
        0x8: "hw_slowdown", 0x10: "sync_boost", 0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _loop(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                bits = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if bits & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.01)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.samples) if self.samples else None,
            "sm_max_mhz": self.max_mhz,
            "reasons": sorted(self.reasons),
            "samples": len(self.samples),
        }


# ------------------------------------------------------------------------- CPU arm


class CpuLayer:
    """The layer's forward + backward on the host cores: the reference's own `ReferenceDeconv`
    when an installation of the reference is present, else the oracle's port of the same
    eager path."""

    def __init__(self):
        self.threads = os.cpu_count() or 1
        torch.set_num_threads(self.threads)
        C, r, ks = WORKLOAD["channels"], WORKLOAD["ratio"], WORKLOAD["kernel_size"]
        self.mod = None
        if os.path.isdir(os.path.join(REF, "deconver")):
            try:
                if REF not in sys.path:
                    sys.path.insert(0, REF)
                from deconver.deconvolution.reference import ReferenceDeconv
                torch.manual_seed(0)
                self.mod = ReferenceDeconv(channels=C, ratio=r, groups=-1, kernel_size=ks)
                with torch.no_grad():
                    self.mod.init.h0.copy_(torch.randn(C, r, *ks).abs() / 27)
            except Exception as exc:
                print(f"bench.py: reference installation not importable ({exc}); "
                      "timing the oracle port", file=sys.stderr)
                self.mod = None
        self.kind = "reference" if self.mod is not None else "port"
        self.what = ("reference ReferenceDeconv (general PyTorch path)" if self.mod is not None
                     else "oracle port of the reference's general PyTorch path")

    def step(self, batch, spatial, seed=0):
        """One forward+backward; returns seconds."""
        C, r, ks = WORKLOAD["channels"], WORKLOAD["ratio"], WORKLOAD["kernel_size"]
        gen = torch.Generator().manual_seed(seed)
        x = torch.rand(batch, C, *spatial, generator=gen).requires_grad_(True)
        g = torch.randn(batch, C * r, *spatial, generator=gen)
        if self.mod is not None:
            self.mod.zero_grad(set_to_none=True)
            t0 = time.perf_counter()
            self.mod(x).backward(g)
            return time.perf_counter() - t0
        from oracle import ndc_oracle
        w = (torch.randn(C * r, C, 1, generator=gen) / C ** 0.5).requires_grad_(True)
        b = torch.zeros(C * r).requires_grad_(True)
        h0 = (torch.randn(C, r, *ks, generator=gen).abs() / 27).requires_grad_(True)
        t0 = time.perf_counter()
        ndc_oracle.ndc_layer(x, w, b, h0, groups=C).backward(g)
        return time.perf_counter() - t0

    def sample_for(self, budget_s):
        """Largest sample of the workload (whole, or a depth slab of one sample) whose step is
        estimated to fit `budget_s`: (batch, spatial)."""
        self.step(1, (4, 16, 16))          # thread-pool warm-up
        per_voxel = self.step(1, (8, 64, 64)) / (8 * 64 * 64)
        B, S = WORKLOAD["batch"], WORKLOAD["spatial"]
        if per_voxel * B * S[0] * S[1] * S[2] <= budget_s:
            return B, S
        depth = int(max(4, min(S[0], budget_s / (per_voxel * S[1] * S[2]))))
        return 1, (depth, S[1], S[2])


def cpu_baseline(budget_s=25.0):
    """Bounded CPU sample for the GPU arm's line: one step."""
    cpu = CpuLayer()
    batch, spatial = cpu.sample_for(budget_s)
    t = cpu.step(batch, spatial)
    vox = batch * spatial[0] * spatial[1] * spatial[2]
    return {
        "value": vox / t, "unit": UNIT, "cores": cpu.threads, "kind": cpu.kind,
        "sample": f"1 fwd+bwd of the layer on X ({batch},64,{spatial[0]},64,64), fp32, "
                  f"{cpu.what}, torch {torch.__version__} CPU, {t:.2f} s",
    }


def run_reference(args):
    """`--impl reference`: the reference's CPU implementation of the layer on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = max(1, args.gpus)
    cpu = CpuLayer()
    total_steps = args.steps + args.warmup
    batch, spatial = cpu.sample_for(240.0 / max(total_steps, 1))
    for _ in range(args.warmup):
        cpu.step(batch, spatial)
    times = [cpu.step(batch, spatial) for _ in range(args.steps)]
    total = sum(times)
    vox = batch * spatial[0] * spatial[1] * spatial[2]
    value = vox * args.steps / total
    whole = (batch, tuple(spatial)) == (WORKLOAD["batch"], tuple(WORKLOAD["spatial"]))
    sample = (f"{args.steps} fwd+bwd steps of the layer on X ({batch},64,{spatial[0]},64,64) "
              f"({'the whole workload' if whole else 'a depth slab of the workload'}), fp32, "
              f"{cpu.what}, {cpu.threads} threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * total / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": config_of(world),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cpu.threads, "kind": cpu.kind,
                         "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------- GPU arm


def measure_fp32_fma_peak(lib, dev):
    """TFLOP/s of register-only float32 multiply-add chains on this GPU, measured now with the
    library's probe kernel (plain `fmaf` and packed `fma.rn.f32x2`; the better of the two)."""
    sms = torch.cuda.get_device_properties(dev).multi_processor_count
    out = torch.empty(sms * 4 * 256, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    best = {}
    for packed in (0, 1):
        n = ctypes.c_uint64(0)
        iters = 4096
        for _ in range(2):   # warm-up
            st = lib.ndc_probe_fp32_fma(packed, iters, out.data_ptr(), out.numel(), ctypes.byref(n), stream)
            if st != 0:
                return None
        times = []
        for _ in range(5):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            lib.ndc_probe_fp32_fma(packed, iters, out.data_ptr(), out.numel(), ctypes.byref(n), stream)
            b.record()
            b.synchronize()
            times.append(a.elapsed_time(b))
        best["packed" if packed else "scalar"] = 2.0 * n.value / (min(times) * 1e-3) / 1e12
    return best


def sub_records(args, world, rank):
    """`train_step` and `inference` (every N), `triton` and `forward_2d` (N = 1): measured
    through bench_configs.py's code with the reference's own network around this library's
    layer, norm and Linear."""
    out = {}
    if args.no_sub_records:
        return out
    try:
        import bench_configs
        dc = bench_configs.load_reference()
    except Exception as exc:
        dc, why = None, f"reference installation not importable: {exc}"
    else:
        why = "baseline/_ref (an installation of the reference) is not present"
    if dc is None:
        out["train_step"] = {"unavailable": why}
        out["inference"] = {"unavailable": why}
        if world == 1:
            out["triton"] = {"unavailable": why}
            out["forward_2d"] = {"unavailable": why}
        return out
    try:
        # forward + backward replayed as one CUDA graph; the plain launch sequence beside it
        rec = bench_configs.train_step_record(dc, steps=8, graph=True)
        eager = bench_configs.train_step_record(dc, steps=8, graph=False)
        rec["ms_per_step_without_cuda_graph"] = eager["ms_per_step"]
        rec["workload"] = ("full 3D Deconver training step (fwd+bwd+SGD), bf16, global batch 16 "
                           "of 2x64^3 split over the ranks (strong scaling); the reference's "
                           "network with this library's NDC layer, InstanceNorm3d, Linear and MLP")
        out["train_step"] = rec
    except Exception as exc:
        out["train_step"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    try:
        rec = bench_configs.inference_record(dc)
        rec["workload"] = ("large 3D Deconver inference, bf16, batch 32 of 4x128^3 split over the "
                           "ranks, no collective; NDC share of the end-to-end time")
        out["inference"] = rec
    except Exception as exc:
        out["inference"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    if world == 1:
        try:
            out["triton"] = bench_configs.triton_record(dc, "cfg3")
        except Exception as exc:
            out["triton"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
        try:
            out["forward_2d"] = {"workload": "full 2D Deconver forward, batch 16x3x256x256",
                                 "runs": bench_configs.forward2d_records(dc)}
        except Exception as exc:
            out["forward_2d"] = {"unavailable": f"{type(exc).__name__}: {exc}"}
    return out


def run_b200(args):
    import torch.distributed as dist

    import deconver_b200 as dcb
    from deconver_b200 import _lib
    from deconver_b200 import functional as Fn
    from deconver_b200.distributed import GradBucket, init_from_env

    rank, world, local = init_from_env("nccl")
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    lib = dcb.load_library()  # raises if the CUDA library is missing

    C, r, ks = WORKLOAD["channels"], WORKLOAD["ratio"], WORKLOAD["kernel_size"]
    B, S = WORKLOAD["batch"], WORKLOAD["spatial"]
    torch.manual_seed(rank)
    layer = dcb.NDC(channels=C, ratio=r, groups=-1, kernel_size=ks).to(dev)
    with torch.no_grad():
        layer.init.h0.copy_(torch.randn(C, r, *ks, device=dev).abs() / 27)
    x = torch.rand(B, C, *S, device=dev)
    gout = torch.randn(B, C * r, *S, device=dev)
    bucket = GradBucket(layer.parameters())
    vox_per_step = B * S[0] * S[1] * S[2]

    def step(xin, gin):
        bucket.zero()
        xin.grad = None
        y = layer(xin)
        y.backward(gin)
        bucket.allreduce_mean()
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    x.requires_grad_(True)
    for _ in range(max(args.warmup, 3)):
        step(x, gout)
    barrier()

    # ---- timed region: K steps, device-resident inputs (each tensor is larger than L2)
    launches0 = lib.ndc_launch_count()
    Fn.timing.enable()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as clocks:
        barrier()
        ev0.record()
        for _ in range(args.steps):
            step(x, gout)
        ev1.record()
        barrier()
    ms_total = ev0.elapsed_time(ev1)
    kernel_ms = Fn.timing.disable_and_collect()
    launches = lib.ndc_launch_count() - launches0
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    value = world * vox_per_step * args.steps / (ms_total * 1e-3)

    # ---- e2e: pinned host tensors in, results back to pinned host memory, every step
    x_host = torch.rand(B, C, *S).pin_memory()
    g_host = torch.randn(B, C * r, *S).pin_memory()
    y_host = torch.empty(B, C * r, *S).pin_memory()
    gx_host = torch.empty(B, C, *S).pin_memory()
    grads_host = torch.empty_like(bucket.flat, device="cpu").pin_memory()

    # Every step copies its own inputs in and its own results out; the copies of neighbouring
    # steps overlap with compute on separate streams (device input buffers are double-buffered).
    s_main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_dev = [torch.empty(B, C, *S, device=dev) for _ in range(2)]
    g_dev = [torch.empty(B, C * r, *S, device=dev) for _ in range(2)]
    in_done = [torch.cuda.Event() for _ in range(2)]
    comp_done = [torch.cuda.Event() for _ in range(2)]
    grads_out = torch.cuda.Event()
    out_done = torch.cuda.Event()
    state = {"i": 0}

    def e2e_step():
        i = state["i"]
        b = i % 2
        state["i"] = i + 1
        with torch.cuda.stream(s_in):
            if i >= 2:
                s_in.wait_event(comp_done[b])       # the step that last used this buffer is done
            x_dev[b].copy_(x_host, non_blocking=True)
            g_dev[b].copy_(g_host, non_blocking=True)
            in_done[b].record(s_in)
        s_main.wait_event(in_done[b])
        if i >= 1:
            s_main.wait_event(grads_out)            # the bucket was read out before it is zeroed
        xd = x_dev[b].detach().requires_grad_(True)
        y = step(xd, g_dev[b])
        gx = xd.grad
        comp_done[b].record(s_main)
        with torch.cuda.stream(s_out):
            s_out.wait_event(comp_done[b])
            grads_host.copy_(bucket.flat, non_blocking=True)
            grads_out.record(s_out)
            y_host.copy_(y.detach(), non_blocking=True)
            gx_host.copy_(gx, non_blocking=True)
            out_done.record(s_out)
        y.record_stream(s_out)
        gx.record_stream(s_out)

    for _ in range(2):
        e2e_step()
    s_main.wait_event(out_done)
    barrier()
    e2e_steps = max(1, min(args.steps, 40))   # enough steps that pipeline fill and drain stay small
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    s_main.wait_event(out_done)                     # the last step's results are on the host
    e1.record()
    barrier()
    te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_value = world * vox_per_step * e2e_steps / (float(te.item()) * 1e-3)
    h2d = x_host.numel() * 4 + g_host.numel() * 4
    d2h = y_host.numel() * 4 + gx_host.numel() * 4 + grads_host.numel() * 4
    del x_dev, g_dev, x_host, g_host, y_host, gx_host
    fma_peak = measure_fp32_fma_peak(lib, dev) if rank == 0 else None
    del x, gout, layer, bucket
    torch.cuda.empty_cache()

    extra = sub_records(args, world, rank)   # collective: every rank takes part
    if rank != 0:
        return

    # ---- roofline of the dominant call (ndc_bwd), from live CUDA-event timings
    peak, peak_kind = load_peaks()
    e = 4  # bytes per element (fp32 storage)
    bwd_bytes = 14 * C * e * vox_per_step  # read x, z, gout; write gx, gz (ratio 4)
    fwd_bytes = 9 * C * e * vox_per_step   # read x, z; write out
    bwd_ms = statistics.mean(kernel_ms["ndc_bwd"]) if kernel_ms["ndc_bwd"] else None
    fwd_ms = statistics.mean(kernel_ms["ndc_fwd"]) if kernel_ms["ndc_fwd"] else None
    taps = ks[0] * ks[1] * ks[2]
    bwd_flops = 2 * 8 * r * taps * C * vox_per_step
    fwd_flops = 2 * 3 * r * taps * C * vox_per_step
    achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9 if bwd_ms else None
    fma_tflops = max(fma_peak.values()) if fma_peak else None
    traffic, traffic_source = load_traffic(B)

    def fma_frac(flops, ms):
        return flops / (ms * 1e-3) / 1e12 / fma_tflops if (ms and fma_tflops) else None

    roofline = {
        "bound": "hbm", "kernel": "ndc_bwd (all launches of one backward call)",
        "achieved": achieved, "peak": peak, "unit": "GB/s",
        "frac": achieved / peak if achieved else None, "peak_kind": peak_kind,
        "traffic": traffic, "traffic_source": traffic_source,
        "algorithmic_bytes": bwd_bytes, "ms": bwd_ms,
        "fp32_fma": {
            "achieved_tflops": bwd_flops / (bwd_ms * 1e-3) / 1e12 if bwd_ms else None,
            "peak_tflops": fma_tflops, "peak_kind": "measured by this run (ndc_probe_fp32_fma)",
            "peak_detail": fma_peak, "frac": fma_frac(bwd_flops, bwd_ms),
        },
        "fwd": {
            "ms": fwd_ms, "algorithmic_bytes": fwd_bytes,
            "achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9 if fwd_ms else None,
            "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak if fwd_ms else None,
            "fp32_fma_frac": fma_frac(fwd_flops, fwd_ms),
        },
        "fwd_bwd_frac": (fwd_bytes + bwd_bytes) / ((fwd_ms + bwd_ms) * 1e-3) / 1e9 / peak
        if fwd_ms and bwd_ms else None,
        "fwd_bwd_fp32_fma_frac": fma_frac(fwd_flops + bwd_flops, (fwd_ms or 0) + (bwd_ms or 0))
        if fwd_ms and bwd_ms else None,
    }

    pth = ctypes.c_int32(-1)
    lib.ndc_query(_lib.make_desc(B, C, 1, r, S, ks, 1e-16, True, _lib.NDC_F32), ctypes.byref(pth))

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": config_of(world),
        "kernel_path": {0: "generic", 1: "depthwise4", 2: "depthwise4_rows"}.get(pth.value, "?"),
        "roofline": roofline,
        "clocks": clocks.summary(),
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "steps": e2e_steps},
        "gpu_launches": int(launches),
    }
    line.update(extra)
    if world == 1 and not args.no_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline()
    print(json.dumps(line), flush=True)


def run_profile_case(args):
    """A small, bounded run of the update for `ncu`: the benchmark geometry at batch
    `--batch` (default 1), `--steps` forward+backward calls, nothing else."""
    import deconver_b200 as dcb

    dev = torch.device("cuda", 0)
    dcb.load_library()
    C, r, ks, S = WORKLOAD["channels"], WORKLOAD["ratio"], WORKLOAD["kernel_size"], WORKLOAD["spatial"]
    if args.channels:
        C = args.channels
    if args.ksize:
        ks = tuple(int(v) for v in args.ksize.split(","))
        S = S[:len(ks)]
    if args.size:
        S = (args.size,) * len(ks)
    B = args.batch
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float32
    gen = torch.Generator(device=dev).manual_seed(0)
    x = torch.rand(B, C, *S, device=dev, generator=gen).to(dt).requires_grad_(True)
    z = (torch.randn(B, C * r, *S, device=dev, generator=gen) * 0.5 + 0.3).to(dt).requires_grad_(True)
    h = (torch.randn(C, r, *ks, device=dev, generator=gen).abs() / math.prod(ks)).requires_grad_(True)
    b = (torch.randn(C * r, device=dev, generator=gen) * 0.1).requires_grad_(True)
    g = torch.randn(B, C * r, *S, device=dev, generator=gen).to(dt)
    from deconver_b200 import functional as Fn
    Fn.timing.enable()
    for _ in range(args.steps):
        out = dcb.deconv_update(x, z, h, b, groups=C, m=1, sc=r, eps=1e-16, relu_input=True)
        out.backward(g)
        x.grad = z.grad = h.grad = b.grad = None
    ms = Fn.timing.disable_and_collect()
    print(json.dumps({"profile_case": True, "batch": B, "channels": C, "spatial": list(S),
                      "steps": args.steps, "dtype": args.dtype,
                      "ndc_fwd_ms": [round(v, 4) for v in ms["ndc_fwd"]],
                      "ndc_bwd_ms": [round(v, 4) for v in ms["ndc_bwd"]]}))


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    ap.add_argument("--no-cpu-baseline", action="store_true",
                    help="skip the CPU-baseline leg (profiling runs)")
    ap.add_argument("--no-sub-records", action="store_true",
                    help="skip the train_step and triton sub-records")
    ap.add_argument("--profile-case", action="store_true",
                    help="run only a few update calls at --batch (for an ncu capture)")
    ap.add_argument("--batch", type=int, default=1, help="batch of --profile-case")
    ap.add_argument("--dtype", choices=["f32", "bf16"], default="f32", help="dtype of --profile-case")
    ap.add_argument("--channels", type=int, default=0, help="channels of --profile-case (default 64)")
    ap.add_argument("--size", type=int, default=0, help="extent per axis of --profile-case (default 64)")
    ap.add_argument("--ksize", default="", help="kernel size of --profile-case, e.g. 5,5 (default 3,3,3)")
    args = ap.parse_args()
    if args.profile_case:
        run_profile_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_b200(args)
        import torch.distributed as dist
        if dist.is_initialized():
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
