#!/usr/bin/env python3
"""Comparison harness on PyTorch DistributedDataParallel with communication hooks.

Restates paper-code/train_pytorch.py:88-224: the task's model wrapped in DDP, one of the
built-in hooks — `powerSGD_hook` (PowerSGDState with `matrix_approximation_rank`,
`start_powerSGD_iter`), `fp16_compress_hook`, `allreduce_hook` — `torch.optim.SGD` with
per-parameter groups (conv / BatchNorm / other weight decay and learning rates) and a
`LambdaLR` following the same schedule, bits counted by wrapping `dist.all_reduce`.

    from powersgd_b200.paper import train_ddp
    train_ddp.config["optimizer_reducer"] = "PowerSGD"      # or "fp16" / "allreduce"
    train_ddp.main()
"""
from __future__ import annotations

import torch
import torch.distributed as dist
from torch.distributed.algorithms.ddp_comm_hooks import default_hooks
from torch.distributed.algorithms.ddp_comm_hooks import powerSGD_hook as powersgd_hooks
from torch.nn.parallel import DistributedDataParallel

from . import tasks
from . import train as base
from ..utils import MeanAccumulator, Timer

config = dict(base.config, optimizer_reducer="PowerSGD", optimizer_reducer_rank=2, start_powerSGD_iter=10)
output_dir = base.output_dir


class BitCounter:
    """Counts the payload of every all-reduce issued while it is installed."""

    def __init__(self):
        self.bits = 0
        self._orig = None

    def __enter__(self):
        self._orig = dist.all_reduce

        def counted(tensor, *args, **kwargs):
            self.bits += 8 * tensor.nelement() * tensor.element_size()
            return self._orig(tensor, *args, **kwargs)

        dist.all_reduce = counted
        return self

    def __exit__(self, *exc):
        dist.all_reduce = self._orig


def register_hook(model: DistributedDataParallel):
    name = config["optimizer_reducer"]
    if name == "PowerSGD":
        state = powersgd_hooks.PowerSGDState(process_group=None, matrix_approximation_rank=config["optimizer_reducer_rank"],
                                             start_powerSGD_iter=config["start_powerSGD_iter"])
        model.register_comm_hook(state, powersgd_hooks.powerSGD_hook)
    elif name == "fp16":
        model.register_comm_hook(None, default_hooks.fp16_compress_hook)
    elif name == "allreduce":
        model.register_comm_hook(None, default_hooks.allreduce_hook)
    else:
        raise ValueError(f"unknown DDP hook {name!r}")


def param_groups(task):
    groups = []
    for name, p in zip(task.parameter_names, task.state):
        base.config.update({k: config[k] for k in base.config if k in config})
        groups.append({"params": [p], "lr": base.get_learning_rate(0.0, name), "weight_decay": base.get_weight_decay(0, name),
                       "name": name})
    return groups


def main():
    base.config.update({k: v for k, v in config.items() if k in base.config})
    base.init_distributed()
    if not dist.is_initialized():
        raise RuntimeError("DistributedDataParallel needs a process group (launch with torch.distributed.run)")
    device = base.pick_device()
    timer = Timer(verbosity_level=config["log_verbosity"], log_fn=base.metric)
    kwargs = {k: v for k, v in config.items() if k not in ("device", "seed", "task")}
    task = tasks.build(task_name=config["task"], seed=config["seed"], device=device, timer=timer, **kwargs)
    ddp = DistributedDataParallel(task._model, device_ids=[device.index] if device.type == "cuda" else None)
    register_hook(ddp)
    task._model = ddp
    groups = param_groups(task)
    optimizer = torch.optim.SGD(groups, lr=config["optimizer_learning_rate"], momentum=config["optimizer_momentum"],
                                nesterov=config["optimizer_momentum_type"] == "nesterov")
    base_lrs = [g["lr"] for g in groups]
    names = [g["name"] for g in groups]
    progress = {"epoch": 0.0}
    scheduler = torch.optim.lr_scheduler.LambdaLR(
        optimizer, [lambda _s, n=n, b=b: base.get_learning_rate(progress["epoch"], n) / b for n, b in zip(names, base_lrs)])

    with BitCounter() as counter:
        for epoch in range(config["num_epochs"]):
            metrics_acc = MeanAccumulator()
            loader = task.train_iterator(config["optimizer_batch_size"])
            for i, batch in enumerate(loader):
                if config["max_batches_per_epoch"] is not None and i >= config["max_batches_per_epoch"]:
                    break
                progress["epoch"] = epoch + i / len(loader)
                with timer("batch", progress["epoch"]):
                    _, _, metrics = task.batch_loss_and_gradient(batch)  # backward runs the hooks
                    metrics_acc.add(metrics)
                    with timer("batch.step", progress["epoch"], verbosity=2):
                        optimizer.step()
                        scheduler.step()
            metrics_acc.reduce()
            for key, value in (metrics_acc.value() or {}).items():
                base.metric(key, {"value": float(value), "epoch": epoch + 1.0, "bits": counter.bits}, tags={"split": "train"})
            print(timer.summary())
    return task, counter.bits


if __name__ == "__main__":
    main()
