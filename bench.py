#!/usr/bin/env python3
"""Headline benchmark: ResNet-18 (CIFAR stem) data-parallel training throughput with PowerSGD.

Configuration: ResNet-18 with 3x3 stem and no max-pool (11.2 M parameters,
BatchNorm), float32, synthetic 3x32x32 N(0,1) images with labels uniform over 10 classes,
batch 128 per GPU, PowerSGD rank 2 with 2 half-iterations per step, SGD lr 0.1 with nesterov
momentum 0.9 and weight decay 1e-4. One process per GPU; weak scaling.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line on rank 0. `value` is device-timed (CUDA events around exactly K steps,
max over ranks) with the inputs already resident on the GPU; `e2e.value` times the same K
steps through the public API including, every step, the host->device copy of that step's
batch from pinned memory and the device->host read of the loss. `aggregate_ms_per_step` is
the second half of the metric (compress + reduce + optimizer update): the device time from
the end of backward to the end of the parameter update, averaged over further steps after the
two timed regions, max over ranks - for this library read from two event-record nodes inside
the replayed CUDA graph, for the reference from an event pair around its `optimizer_step`.

`--impl reference` runs the unmodified upstream package (installed under baseline/_ref) with
the upstream model definition and `powersgd.optimizer_step`; nothing of this repository's
models, kernels or engine is on that path.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
BATCH_PER_GPU = 128
RANK, ITERS = 2, 2
LR, MOMENTUM, WD = 0.1, 0.9, 1e-4


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-graph", action="store_true", help="ours: run eagerly instead of replaying a CUDA graph")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""

    FIELDS = (
        "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
        "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
        "clocks_event_reasons.sw_power_cap"
    )

    def __init__(self, index: int, enabled: bool = True):
        self.index = index
        self.proc = None
        # one sampler per job (rank 0): every nvidia-smi query takes driver locks, and one poller
        # per rank visibly perturbs an 8-GPU run
        self.enabled = enabled

    def start(self):
        if not self.enabled:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200"],
                stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL,
                text=True,
            )
        except OSError:
            self.proc = None

    def stop(self):
        if not self.enabled:
            return None
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples taken under load are the upper half of the clock readings' power draw; keep it simple:
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "samples": len(sm),
            "reasons": sorted(reasons),
        }


def setup_dist(n_gpus: int):
    import torch
    import torch.distributed as dist

    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world != n_gpus:
        raise SystemExit(f"--gpus {n_gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    return local, world


def synthetic_batches(device, count: int, seed: int):
    """Pinned host batches (different per rank and per slot) of the config's shape."""
    import torch

    g = torch.Generator().manual_seed(seed)
    xs, ys = [], []
    for _ in range(count):
        xs.append(torch.randn(BATCH_PER_GPU, 3, 32, 32, generator=g).pin_memory())
        ys.append(torch.randint(0, 10, (BATCH_PER_GPU,), generator=g).pin_memory())
    return xs, ys


def build_ours(device, use_graph: bool):
    import torch

    sys.path.insert(0, ROOT)
    from powersgd_b200 import Config, PowerSGD
    from powersgd_b200.engine import TrainStep
    from powersgd_b200.models import ResNet18

    torch.manual_seed(0)
    model = ResNet18().to(device)
    params = list(model.parameters())
    optimizer = torch.optim.SGD(params, lr=LR, momentum=MOMENTUM, nesterov=True, weight_decay=WD)
    aggregator = PowerSGD(
        params,
        Config(rank=RANK, min_compression_rate=2, num_iters_per_step=ITERS, start_compressing_after_num_steps=0),
    )
    step = TrainStep(model, torch.nn.functional.cross_entropy, optimizer, aggregator, cuda_graph=use_graph)
    return step


def build_reference(device):
    import torch

    ref_root = os.path.join(ROOT, "baseline", "_ref")
    arch_dir = os.path.join(ref_root, "paper_code", "tasks", "cifar_architectures")
    if not os.path.isdir(os.path.join(ref_root, "powersgd")) or not os.path.exists(os.path.join(arch_dir, "resnet.py")):
        return None
    sys.path.insert(0, ref_root)
    import importlib.util

    import powersgd as ref  # the unmodified upstream package

    spec = importlib.util.spec_from_file_location("_ref_resnet", os.path.join(arch_dir, "resnet.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)

    torch.manual_seed(0)
    model = mod.ResNet18().to(device)
    params = list(model.parameters())
    optimizer = torch.optim.SGD(params, lr=LR, momentum=MOMENTUM, nesterov=True, weight_decay=WD)
    aggregator = ref.PowerSGD(
        params,
        ref.Config(rank=RANK, min_compression_rate=2, num_iters_per_step=ITERS, start_compressing_after_num_steps=0),
    )

    class Step:
        launches_per_step = 0
        time_aggregate = False   # switched on for the separate aggregate-timing pass only
        _pair = None

        @property
        def aggregate_ms(self):
            if self._pair is None:
                return None
            a, b = self._pair
            b.synchronize()
            return a.elapsed_time(b)

        def __call__(self, x, y):
            loss = torch.nn.functional.cross_entropy(model(x), y)
            loss.backward()
            if self.time_aggregate:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                ref.optimizer_step(optimizer, aggregator)
                b.record()
                self._pair = (a, b)
            else:
                ref.optimizer_step(optimizer, aggregator)
            return loss.detach()

    return Step()


def measure_aggregate(step, xs, ys, is_reference: bool, max_over_ranks, graph: bool, bursts: int = 20, burst_len: int = 10):
    """Device time from the end of backward to the end of the parameter update, in steady state.

    Bursts of steps are enqueued back to back (no host synchronisation inside a burst, so the
    ranks' GPUs stay coupled as they are in training); the event pair of the LAST step of every
    burst is read after the burst. Mean over bursts, max over ranks. Returns (ms, description)."""
    import torch

    if is_reference:
        step.time_aggregate = True
    samples = []
    k = 0
    for _ in range(bursts):
        for _ in range(burst_len):
            step(xs[k % len(xs)], ys[k % len(ys)])
            k += 1
        torch.cuda.synchronize()
        ms = step.aggregate_ms
        if ms is not None:
            samples.append(ms)
    if not samples:
        return None, "not measured"
    how = (
        f"device time from the end of backward to the end of the parameter update: last step of each of {len(samples)} "
        f"bursts of {burst_len} back-to-back steps after the timed regions, mean, max over ranks; "
        + ("event-record nodes inside the replayed CUDA graph" if graph else "CUDA-event pair around the aggregation + optimizer call")
    )
    return max_over_ranks(sum(samples) / len(samples)), how


def main():
    args = parse_args()
    if args.impl == "reference":
        ref_root = os.path.join(ROOT, "baseline", "_ref")
        if not os.path.isdir(os.path.join(ref_root, "powersgd")):
            print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"}))
            return 0

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device"}))
        return 0

    local, world = setup_dist(args.gpus)
    device = torch.device("cuda", local)
    rank = int(os.environ.get("RANK", "0"))

    if args.impl == "ours":
        step = build_ours(device, use_graph=not args.no_graph)
    else:
        step = build_reference(device)
        if step is None:
            if rank == 0:
                print(json.dumps({"impl": "reference", "unavailable": "upstream model definition not found under baseline/_ref"}))
            return 0

    n_slots = 8
    xs_host, ys_host = synthetic_batches(device, n_slots, seed=1234 + rank)
    xs_dev = [x.to(device) for x in xs_host]
    ys_dev = [y.to(device) for y in ys_host]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- warm-up (also builds descriptors / captures the graph) -----------------------------
    # at least 3 untimed steps: two run eagerly (cuDNN autotuning, lazy buffers), the third records the graph
    for i in range(max(args.warmup, 3)):
        loss = step(xs_dev[i % n_slots], ys_dev[i % n_slots])
    barrier()

    # ---- device-timed region: inputs resident, no host read-back ----------------------------
    sampler = ClockSampler(local, enabled=rank == 0)
    sampler.start()
    time.sleep(0.3)
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    start.record()
    for i in range(args.steps):
        loss = step(xs_dev[i % n_slots], ys_dev[i % n_slots])
    stop.record()
    barrier()
    dev_ms = max_over_ranks(start.elapsed_time(stop))

    # ---- end-to-end region: pinned H2D of the batch and D2H of the loss every step ----------
    x_stage = torch.empty_like(xs_dev[0])
    y_stage = torch.empty_like(ys_dev[0])
    barrier()
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e_start.record()
    # Every step copies its batch from pinned host memory and its loss back to pinned host memory.
    # The loss of step i is READ on the host after step i + 1 has been enqueued (asynchronous
    # logging), so the host wait does not drain the GPU between steps.
    last = 0.0
    loss_host = [torch.empty((), dtype=torch.float32).pin_memory() for _ in range(2)]
    pending = None
    for i in range(args.steps):
        x_stage.copy_(xs_host[i % n_slots], non_blocking=True)
        y_stage.copy_(ys_host[i % n_slots], non_blocking=True)
        loss = step(x_stage, y_stage)
        slot = loss_host[i % 2]
        slot.copy_(loss, non_blocking=True)
        landed = torch.cuda.Event()
        landed.record()
        if pending is not None:
            pending[1].synchronize()
            last = float(pending[0])
        pending = (slot, landed)
    pending[1].synchronize()
    last = float(pending[0])
    e_stop.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(e_start.elapsed_time(e_stop), 0.0))
    clocks = sampler.stop()

    # ---- compress + reduce + update time per step, steady state (outside both timed regions) ----
    agg_ms, agg_how = measure_aggregate(step, xs_dev, ys_dev, args.impl == "reference", max_over_ranks,
                                        graph=args.impl == "ours" and not args.no_graph)
    barrier()

    images = BATCH_PER_GPU * world * args.steps
    h2d = xs_host[0].numel() * xs_host[0].element_size() + ys_host[0].numel() * ys_host[0].element_size()
    launches = getattr(step, "launches_per_step", 0) * args.steps
    if rank == 0:
        out = {
            "metric": "ResNet-18 imgs/s @1/2/4/8 B200; compress+reduce ms/step vs ref NCCL",
            "impl": args.impl,
            "value": images / (dev_ms / 1e3),
            "unit": "images/s",
            "n_gpus": world,
            "steps": args.steps,
            "warmup": max(args.warmup, 3),
            "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": "fp32",
            "data": "synthetic N(0,1) 3x32x32 images, uniform labels, random-init weights",
            "config": {
                "model": "ResNet-18 (CIFAR stem, no max-pool, BatchNorm, 11.17M params)",
                "global_batch": BATCH_PER_GPU * world,
                "seq_len": None,
                "parallelism": f"dp{world}",
                "powersgd": {"rank": RANK, "num_iters_per_step": ITERS, "min_compression_rate": 2,
                             "start_compressing_after_num_steps": 0},
                "optimizer": {"sgd_lr": LR, "momentum": MOMENTUM, "nesterov": True, "weight_decay": WD},
                "l2": "per-step working set (activations + gradients, > 1 GB at batch 128) exceeds the 126 MB L2; no explicit flush",
            },
            "engine": {"cuda_graph": bool(args.impl == "ours" and not args.no_graph), "host_cpus": os.cpu_count()},
            "clocks": clocks,
            "e2e": {
                "value": images / (e2e_ms / 1e3),
                "unit": "images/s",
                "ms_per_step": e2e_ms / args.steps,
                "wall_ms_per_step": wall_ms / args.steps,
                "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": 4,
                "loss_read": "copied to pinned host memory every step, read on the host after the next step is enqueued",
                "last_loss": last,
            },
            "gpu_launches": launches,
            "aggregate_ms_per_step": agg_ms,
            "aggregate_how": agg_how,
        }
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
