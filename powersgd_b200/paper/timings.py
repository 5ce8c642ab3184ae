#!/usr/bin/env python3
"""Collective micro-benchmark: all_reduce / all_gather / gather / broadcast at 14 message sizes
(4 B ... 256 MiB), plus this library's in-kernel all-reduces beside NCCL's: the one-shot
flag-in-data kernel up to 4 MiB and the two-shot bulk kernel above.

Protocol of paper-code/timings.py:16-39, 65-115 (barrier before every repetition, `repetitions`
samples per size, summary table and JSON). Timing differs on purpose: on CUDA every sample is a
CUDA-event pair on the launching stream (no host synchronisation inside the sample), reported
as the max over ranks; the host-clock `Timer` of the original serialises the GPU and measures
launch overhead for small messages.

    python -m torch.distributed.run --nproc-per-node 8 -m powersgd_b200.paper.timings
"""
from __future__ import annotations

import datetime
import json
import os
import time

import torch
import torch.distributed as dist

config = dict(
    distributed_backend="nccl",
    device="cuda",
    rank=0,
    n_workers=1,
    distributed_init_file=None,
    message_sizes=[4 ** i for i in range(1, 15)],  # bytes: 4 ... 268 435 456
    repetitions=4,
    in_kernel_limit_bytes=4 << 20,  # largest message given to the one-shot peer all-reduce
    nvls_from_bytes=1 << 20,        # smallest message given to the in-switch (multimem) all-reduce
)

output_dir = "./output.tmp"


def _init():
    if dist.is_initialized():
        return
    if "RANK" in os.environ:
        config["rank"], config["n_workers"] = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        kwargs = {}
        if config["distributed_backend"] == "nccl":
            local = int(os.environ.get("LOCAL_RANK", "0"))
            torch.cuda.set_device(local)
            kwargs["device_id"] = torch.device("cuda", local)
        dist.init_process_group(config["distributed_backend"], timeout=datetime.timedelta(seconds=1800), **kwargs)
    else:
        if config["distributed_init_file"] is None:
            config["distributed_init_file"] = os.path.join(output_dir, "dist_init")
        os.makedirs(os.path.dirname(os.path.abspath(config["distributed_init_file"])), exist_ok=True)
        dist.init_process_group(config["distributed_backend"], init_method="file://" + os.path.abspath(config["distributed_init_file"]),
                                timeout=datetime.timedelta(seconds=1800), world_size=config["n_workers"], rank=config["rank"])


class _Samples:
    def __init__(self, cuda: bool):
        self.cuda = cuda
        self.data = {}

    def time(self, label, fn):
        dist.barrier()
        if self.cuda:
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            seconds = a.elapsed_time(b) * 1e-3
        else:
            t0 = time.perf_counter()
            fn()
            seconds = time.perf_counter() - t0
        t = torch.tensor([seconds], dtype=torch.float64, device="cuda" if self.cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        self.data.setdefault(label, []).append(float(t.item()))

    def summary(self, skip_first=True):
        out = {}
        for label, values in self.data.items():
            kept = values[1:] if (skip_first and len(values) > 1) else values
            out[label] = {"label": label, "average_duration": sum(kept) / len(kept), "n_events": len(kept),
                          "total_time": sum(kept)}
        return out


def main():
    _init()
    cuda = config["device"] == "cuda" and torch.cuda.is_available()
    device = torch.device("cuda", torch.cuda.current_device()) if cuda else torch.device("cpu")
    world = dist.get_world_size()
    samples = _Samples(cuda)
    reps = config["repetitions"]

    channel = None
    if cuda and world > 1:
        try:
            from ..parallel.symm import Channel

            channel = Channel(config["in_kernel_limit_bytes"] // 4)
        except Exception as exc:  # library not built: NCCL numbers only
            metric("in_kernel_allreduce_unavailable", {"value": 0.0}, {"reason": str(exc)[:80]})

    nvls_ok = [os.environ.get("PSGD_B200_TIMINGS_NVLS", "1") != "0"]
    for size in config["message_sizes"]:
        data = torch.randn(max(size // 4, 1), device=device)
        for _ in range(reps):
            samples.time(f"all_reduce_{size}", lambda: dist.all_reduce(data))
        if channel is not None and size <= config["in_kernel_limit_bytes"]:
            for _ in range(reps):
                samples.time(f"in_kernel_all_reduce_{size}", lambda: channel.all_reduce_(data))
            channel.check()
        elif channel is not None:
            from ..parallel.symm import BulkAllReduce

            bulk = BulkAllReduce(data.numel())
            bulk.buffer.copy_(data)
            for _ in range(reps):
                samples.time(f"in_kernel_all_reduce_{size}", bulk.all_reduce_)
            bulk.check()
            bulk.close()
        if channel is not None and size >= config["nvls_from_bytes"] and nvls_ok[0]:
            from ..parallel.nvls import NvlsAllReduce, NvlsUnavailable

            try:
                nvls = NvlsAllReduce(data.numel())
            except NvlsUnavailable as exc:
                nvls_ok[0] = False
                metric("nvls_allreduce_unavailable", {"value": 0.0}, {"reason": str(exc)[:80]})
            else:
                nvls.buffer[: data.numel()].copy_(data)
                for _ in range(reps):
                    samples.time(f"nvls_all_reduce_{size}", nvls.all_reduce_)
                nvls.check()
                nvls.close()
    for size in config["message_sizes"]:
        data = torch.randn(max(size // 4, 1), device=device)
        outs = [torch.empty_like(data) for _ in range(world)]
        for _ in range(reps):
            samples.time(f"all_gather_{size}", lambda: dist.all_gather(outs, data))
    if config["distributed_backend"] != "nccl":
        for size in config["message_sizes"]:
            data = torch.randn(max(size // 4, 1), device=device)
            outs = [torch.empty_like(data) for _ in range(world)] if dist.get_rank() == 0 else None
            for _ in range(reps):
                samples.time(f"gather_{size}", lambda: dist.gather(data, outs, dst=0))
    for size in config["message_sizes"]:
        data = torch.randn(max(size // 4, 1), device=device)
        for _ in range(reps):
            samples.time(f"broadcast_{size}", lambda: dist.broadcast(data, src=0))

    summary = samples.summary()
    if dist.get_rank() == 0:
        print("--- Collective timings (max over ranks) ---------------------------")
        for label in sorted(summary, key=lambda s: (s.rsplit("_", 1)[0], int(s.rsplit("_", 1)[1]))):
            row = summary[label]
            size = int(label.rsplit("_", 1)[1])
            print(f"- {label:34s} | {row['n_events']:3d} | {row['average_duration'] * 1e6:12.1f} us | "
                  f"{size / row['average_duration'] / 1e9:9.3f} GB/s")
        os.makedirs(output_dir, exist_ok=True)
        with open(os.path.join(output_dir, "timer_summary.json"), "w") as fp:
            json.dump(summary, fp)
    if channel is not None:
        dist.barrier()
        channel.close()
    return summary


def log_metric(name, values, tags={}):
    print(f"{name:30s} - {values} ({tags})")


def metric(*args, **kwargs):
    if config["rank"] == 0:
        log_metric(*args, **kwargs)


if __name__ == "__main__":
    main()
    if dist.is_initialized():
        dist.destroy_process_group()
