#!/usr/bin/env python3
"""Research training loop: data-parallel SGD with a pluggable gradient reducer.

Restates paper-code/train.py (config dict :31-65, main loop :70-300, schedules :317-349,
reducer factory :382-440, logging hooks :451-479) for this library:

    from powersgd_b200.paper import train
    train.config["optimizer_reducer"] = "RankKReducer"
    train.config["optimizer_reducer_rank"] = 2
    train.main()

Per batch: gradients -> (optional wd / momentum before the reducer) -> send = grad + memory
(error feedback) -> `reducer.reduce(send, grads, memories)` -> weight decay, momentum
(heavy-ball / nesterov / EMA), SGD step, running-average model, sampled diagnostics. Per epoch:
metric reduction over workers, test of the last and of the running-average model, optional
checkpoint, timer summary.

Differences from the original, all additive: the rendezvous may come from the environment
(`torchrun`) instead of a shared file; checkpoints hold EVERYTHING needed to resume (reducer
factors, error memories, momenta, RNG, running average) and `config["resume_from"]` loads one;
no dataset is downloaded (tasks fall back to synthetic data).
"""
from __future__ import annotations

import datetime
import os
import re

import numpy as np
import torch
import torch.distributed as dist

from . import reducers as gradient_reducers
from . import tasks
from ..utils import MeanAccumulator, Timer

config = dict(
    average_reset_epoch_interval=30,
    distributed_backend="nccl",
    fix_conv_weight_norm=False,
    num_epochs=300,
    checkpoints=[],
    num_train_tracking_batches=1,
    optimizer_batch_size=128,  # per worker
    optimizer_conv_learning_rate=0.1,
    optimizer_decay_at_epochs=[150, 250],
    optimizer_decay_with_factor=10.0,
    optimizer_learning_rate=0.1,
    optimizer_memory=True,
    optimizer_momentum_type="nesterov",
    optimizer_momentum=0.9,
    optimizer_reducer="ExactReducer",
    optimizer_reducer_reuse_query=True,
    optimizer_reducer_rank=2,
    optimizer_reducer_compression=1 / 244,
    optimizer_reducer_n_power_iterations=0,
    optimizer_scale_lr_with_factor=None,
    optimizer_scale_lr_with_warmup_epochs=5,
    optimizer_mom_before_reduce=False,
    optimizer_wd_before_reduce=False,
    optimizer_weight_decay_conv=0.0001,
    optimizer_weight_decay_other=0.0001,
    optimizer_weight_decay_bn=0.0,
    task="Cifar",
    task_architecture="ResNet18",
    seed=42,
    rank=0,
    n_workers=1,
    distributed_init_file=None,
    log_verbosity=2,
    # additions
    max_batches_per_epoch=None,  # cut epochs short (smoke runs, benchmarks)
    resume_from=None,  # path of a checkpoint written by `save`
    device=None,  # default: cuda:LOCAL_RANK when available, else cpu
)

output_dir = "./output.tmp"  # a launcher may overwrite this


def _world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def init_distributed() -> None:
    """Join the process group: from torchrun's environment when present, else through the
    shared-file rendezvous of the original (train.py:78-93)."""
    if not dist.is_available() or dist.is_initialized():
        return
    if "RANK" in os.environ and "WORLD_SIZE" in os.environ:
        config["rank"], config["n_workers"] = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29500")
        dist.init_process_group(config["distributed_backend"], timeout=datetime.timedelta(seconds=120))
        return
    if config["n_workers"] == 1 and config["distributed_init_file"] is None:
        return  # single process: every collective in this package degrades to a no-op
    if config["distributed_init_file"] is None:
        config["distributed_init_file"] = os.path.join(output_dir, "dist_init")
    os.makedirs(os.path.dirname(os.path.abspath(config["distributed_init_file"])), exist_ok=True)
    dist.init_process_group(
        backend=config["distributed_backend"],
        init_method="file://" + os.path.abspath(config["distributed_init_file"]),
        timeout=datetime.timedelta(seconds=120),
        world_size=config["n_workers"],
        rank=config["rank"],
    )


def pick_device() -> torch.device:
    if config["device"] is not None:
        return torch.device(config["device"])
    if torch.cuda.is_available() and config["distributed_backend"] != "gloo":
        local = int(os.environ.get("LOCAL_RANK", "0"))
        torch.cuda.set_device(local)
        return torch.device("cuda", local)
    return torch.device("cpu")


def main():
    torch.manual_seed(config["seed"] + config["rank"])
    np.random.seed(config["seed"] + config["rank"])
    init_distributed()
    device = pick_device()
    timer = Timer(verbosity_level=config["log_verbosity"], log_fn=metric)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()

    task_kwargs = {k: v for k, v in config.items() if k not in ("device", "seed", "task")}
    task = tasks.build(task_name=config["task"], seed=config["seed"], device=device, timer=timer, **task_kwargs)
    reducer = get_reducer(device, timer)

    bits_communicated = 0
    runavg_model = MeanAccumulator()
    memories = [torch.zeros_like(p) for p in task.state]
    momenta = [torch.empty_like(p) for p in task.state]  # initialised at the first step
    send_buffers = [torch.zeros_like(p) for p in task.state]
    first_step_done = False
    start_epoch = 0
    if config["resume_from"]:
        ckpt = torch.load(config["resume_from"], map_location=device, weights_only=False)
        start_epoch, bits_communicated, first_step_done = load_checkpoint(ckpt, task, reducer, memories, momenta, runavg_model)

    for epoch in range(start_epoch, config["num_epochs"]):
        epoch_metrics = MeanAccumulator()
        info({"state.progress": float(epoch) / config["num_epochs"], "state.current_epoch": epoch})
        wds = [get_weight_decay(epoch, name) for name in task.parameter_names]
        if epoch % config["average_reset_epoch_interval"] == 0:
            runavg_model.reset()

        train_loader = task.train_iterator(config["optimizer_batch_size"])
        for i, batch in enumerate(train_loader):
            if config["max_batches_per_epoch"] is not None and i >= config["max_batches_per_epoch"]:
                break
            epoch_frac = epoch + i / len(train_loader)
            lrs = [get_learning_rate(epoch_frac, name) for name in task.parameter_names]

            with timer("batch", epoch_frac):
                _, grads, metrics = task.batch_loss_and_gradient(batch)
                epoch_metrics.add(metrics)
                report_lr_and_grad_norm(timer, task, grads, lrs, epoch_frac)

                if config["optimizer_wd_before_reduce"]:
                    with timer("batch.weight_decay", epoch_frac, verbosity=2):
                        apply_weight_decay(grads, task.state, wds)
                if config["optimizer_mom_before_reduce"]:
                    with timer("batch.momentum", epoch_frac, verbosity=2):
                        apply_momentum(grads, momenta, first_step=not first_step_done)

                with timer("batch.accumulate", epoch_frac, verbosity=2):
                    # multi-tensor launches (one per operation, not one per parameter)
                    torch._foreach_copy_(send_buffers, grads)
                    if config["optimizer_memory"]:
                        torch._foreach_add_(send_buffers, memories)

                with timer("batch.reduce", epoch_frac):
                    # `grads` now receive the aggregate that every worker applies
                    bits_communicated += reducer.reduce(send_buffers, grads, memories)

                if config["optimizer_memory"]:
                    report_compression_error(timer, task, memories, send_buffers, epoch_frac)

                if not config["optimizer_wd_before_reduce"]:
                    with timer("batch.wd", epoch_frac, verbosity=2):
                        apply_weight_decay(grads, task.state, wds)
                if not config["optimizer_mom_before_reduce"]:
                    with timer("batch.mom", epoch_frac, verbosity=2):
                        apply_momentum(grads, momenta, first_step=not first_step_done)
                first_step_done = True

                with timer("batch.step", epoch_frac, verbosity=2):
                    # one multi-tensor launch per distinct learning rate (usually one)
                    for lr in sorted(set(lrs)):
                        picked = [k for k, value in enumerate(lrs) if value == lr]
                        torch._foreach_add_([task.state[k].data for k in picked], [grads[k] for k in picked], alpha=-lr)

                if config["fix_conv_weight_norm"]:
                    with timer("batch.normfix", epoch_frac, verbosity=2):
                        for name, param in zip(task.parameter_names, task.state):
                            if is_conv_param(name):
                                param.data.div_(l2norm(param))

                with timer("batch.update_runavg", epoch_frac, verbosity=2):
                    runavg_model.add(task.state_dict())

                if config["optimizer_memory"]:
                    report_memory_norm(timer, task, memories, epoch_frac)

        with timer("epoch_metrics.collect", epoch + 1.0, verbosity=2):
            epoch_metrics.reduce()
            for key, value in (epoch_metrics.value() or {}).items():
                for name in (key, f"last_{key}"):
                    metric(name, {"value": float(value), "epoch": epoch + 1.0, "bits": bits_communicated}, tags={"split": "train"})

        with timer("test.last", epoch):
            test_stats = task.test()
            for key, value in test_stats.items():
                metric(f"last_{key}", {"value": float(value), "epoch": epoch + 1.0, "bits": bits_communicated}, tags={"split": "test"})
        with timer("test.runavg", epoch):
            if runavg_model.value() is not None:
                test_stats = task.test(state_dict=runavg_model.value())
                for key, value in test_stats.items():
                    metric(f"runavg_{key}", {"value": float(value), "epoch": epoch + 1.0, "bits": bits_communicated}, tags={"split": "test"})

        if epoch in config["checkpoints"] and config["rank"] == 0:
            with timer("checkpointing"):
                os.makedirs(output_dir, exist_ok=True)
                save(os.path.join(output_dir, "epoch_{:03d}".format(epoch)), task.state_dict(), epoch + 1.0, test_stats,
                     extra=checkpoint_extras(reducer, memories, momenta, runavg_model, bits_communicated, first_step_done))

        print(timer.summary())
        if config["rank"] == 0:
            os.makedirs(output_dir, exist_ok=True)
            timer.save_summary(os.path.join(output_dir, "timer_summary.json"))

    info({"state.progress": 1.0})
    return task, reducer, bits_communicated


# ---- optimizer pieces ---------------------------------------------------------------------
def apply_weight_decay(grads, params, wds) -> None:
    for grad, param, wd in zip(grads, params, wds):
        if wd > 0:
            grad.add_(param.detach(), alpha=wd)


def apply_momentum(grads, momenta, first_step: bool) -> None:
    mu, kind = config["optimizer_momentum"], config["optimizer_momentum_type"]
    for grad, momentum in zip(grads, momenta):
        if first_step:
            momentum.copy_(grad.detach())
        elif kind == "exponential_moving_average":
            momentum.mul_(mu).add_(grad, alpha=1 - mu)
        else:
            momentum.mul_(mu).add_(grad)
        replace_grad_by_momentum(grad, momentum)


def replace_grad_by_momentum(grad, momentum) -> None:
    kind = config["optimizer_momentum_type"]
    if kind in ("heavy-ball", "exponential_moving_average"):
        grad.copy_(momentum)
    elif kind == "nesterov":
        grad.add_(momentum)
    else:
        raise ValueError("Unknown momentum type")


def get_weight_decay(epoch, parameter_name):
    if is_conv_param(parameter_name):
        return config["optimizer_weight_decay_conv"]
    if is_batchnorm_param(parameter_name):
        return config["optimizer_weight_decay_bn"]
    return config["optimizer_weight_decay_other"]


def get_learning_rate(epoch, parameter_name):
    """Base rate (conv / other), linear warm-up towards `world_size x` over the first epochs,
    then division by the decay factor at every milestone that has passed."""
    lr = config["optimizer_conv_learning_rate"] if is_conv_param(parameter_name) else config["optimizer_learning_rate"]
    warmup = config["optimizer_scale_lr_with_warmup_epochs"]
    if warmup:
        top = config.get("optimizer_scale_lr_with_factor", None)
        if top is None:
            top = float(_world_size())
        lr *= 1.0 + (top - 1.0) * min(epoch / warmup, 1.0)
    for milestone in config["optimizer_decay_at_epochs"]:
        if epoch >= milestone:
            lr /= config["optimizer_decay_with_factor"]
        else:
            break
    return lr


def is_conv_param(parameter_name) -> bool:
    return "conv" in parameter_name and "weight" in parameter_name


def is_batchnorm_param(parameter_name):
    return re.match(r""".*\.bn\d+\.(weight|bias)""", parameter_name)


def l2norm(tensor):
    return torch.sqrt(torch.sum(tensor ** 2))


def get_reducer(device, timer):
    """Build the reducer named in the config with the options it understands."""
    name = config["optimizer_reducer"]
    cls = getattr(gradient_reducers, name)
    common = dict(random_seed=config["seed"], device=device, timer=timer)
    if name == "RankKReducer":
        return cls(**common, n_power_iterations=config["optimizer_reducer_n_power_iterations"],
                   reuse_query=config["optimizer_reducer_reuse_query"], rank=config["optimizer_reducer_rank"])
    if name in ("AtomoReducer", "RandomSparseReducer", "RandomSparseBlockReducer", "HalfRankKReducer", "SVDReducer"):
        return cls(**common, rank=config["optimizer_reducer_rank"])
    if name in ("GlobalTopKReducer", "TopKReducer", "UniformRandomSparseBlockReducer", "UniformRandomSparseReducer"):
        return cls(**common, compression=config["optimizer_reducer_compression"])
    return cls(**common)


# ---- sampled diagnostics (train.py:136-152, 188-200, 238-254) -------------------------------
def report_lr_and_grad_norm(timer, task, grads, lrs, epoch_frac, probability=0.001) -> None:
    with timer("batch.reporting.lr", epoch_frac, verbosity=2):
        for name, param, grad, lr in zip(task.parameter_names, task.state, grads, lrs):
            if np.random.rand() < probability:
                tags = {"weight": name.replace("module.", "")}
                metric("effective_lr", {"epoch": epoch_frac, "value": lr / max(l2norm(param).item() ** 2, 1e-8)}, tags)
                metric("grad_norm", {"epoch": epoch_frac, "value": l2norm(grad).item()}, tags)


def report_compression_error(timer, task, memories, send_buffers, epoch_frac, probability=0.001) -> None:
    with timer("batch.reporting.compr_err", verbosity=2):
        for name, memory, send in zip(task.parameter_names, memories, send_buffers):
            if np.random.rand() < probability:
                value = (l2norm(memory) / l2norm(send)).item()
                metric("rel_compression_error", {"epoch": epoch_frac, "value": value}, {"weight": name.replace("module.", "")})


def report_memory_norm(timer, task, memories, epoch_frac, probability=0.001) -> None:
    with timer("batch.reporting.memory_norm", epoch_frac, verbosity=2):
        if np.random.rand() < probability:
            total = 0.0
            for name, memory in zip(task.parameter_names, memories):
                norm = l2norm(memory)
                total = total + norm
                metric("memory_norm", {"epoch": epoch_frac, "value": norm.item()}, {"weight": name.replace("module.", "")})
            metric("compression_error", {"epoch": epoch_frac, "value": float(torch.sqrt(torch.as_tensor(total)))})


# ---- checkpoints --------------------------------------------------------------------------
def checkpoint_extras(reducer, memories, momenta, runavg_model, bits, first_step_done):
    """Everything beyond the model that a faithful resume needs (the original saved none of it)."""
    return {
        "memories": [m.detach().cpu() for m in memories],
        "momenta": [m.detach().cpu() for m in momenta],
        "first_step_done": first_step_done,
        "bits_communicated": bits,
        "reducer": {
            "p_memory": None if getattr(reducer, "p_memory", None) is None else reducer.p_memory.detach().cpu(),
            "q_memory": None if getattr(reducer, "q_memory", None) is None else reducer.q_memory.detach().cpu(),
            "next_operation": getattr(reducer, "next_operation", None),
            "rng_state": reducer.rng.get_state(),
        },
        "runavg": {"average": runavg_model.value(), "counter": runavg_model.counter},
        "torch_rng": torch.get_rng_state(),
        "numpy_rng": np.random.get_state(),
    }


def save(destination_path, model_state, epoch, test_stats, extra=None):
    payload = {"epoch": epoch, "test_stats": test_stats, "model_state_dict": model_state}
    if extra is not None:
        payload["resume"] = extra
    torch.save(payload, destination_path)


def load_checkpoint(ckpt, task, reducer, memories, momenta, runavg_model):
    task._model.load_state_dict(ckpt["model_state_dict"])
    extra = ckpt.get("resume")
    if extra is None:
        return int(ckpt["epoch"]), 0, False
    for dst, src in zip(memories, extra["memories"]):
        dst.copy_(src)
    for dst, src in zip(momenta, extra["momenta"]):
        dst.copy_(src)
    state = extra["reducer"]
    if state["p_memory"] is not None:
        reducer.p_memory = state["p_memory"].to(memories[0].device)
        reducer.q_memory = state["q_memory"].to(memories[0].device)
    if state["next_operation"] is not None:
        reducer.next_operation = state["next_operation"]
    reducer.rng.set_state(state["rng_state"])
    if extra["runavg"]["average"] is not None:
        runavg_model.reset()
        runavg_model.add(extra["runavg"]["average"], weight=extra["runavg"]["counter"])
    torch.set_rng_state(extra["torch_rng"])
    np.random.set_state(extra["numpy_rng"])
    return int(ckpt["epoch"]), extra["bits_communicated"], extra["first_step_done"]


# ---- logging hooks: a launcher may replace log_info / log_metric --------------------------
def log_info(info_dict):
    pass


def log_metric(name, values, tags={}):
    value_list = [f"{key}:{values[key]:7.3f}" for key in sorted(values.keys())]
    tag_list = [f"{key}:{tag}" for key, tag in tags.items()]
    print("{name:30s} - {values} ({tags})".format(name=name, values=", ".join(value_list), tags=", ".join(tag_list)))


def info(*args, **kwargs):
    if config["rank"] == 0:
        log_info(*args, **kwargs)


def metric(*args, **kwargs):
    if config["rank"] == 0:
        log_metric(*args, **kwargs)


def check_model_consistency_across_workers(model, epoch):
    """True when every parameter is bit-identical on all workers (the original only printed
    the first element of each parameter per worker, train.py:496-503)."""
    if _world_size() == 1:
        return True
    same = True
    for _, p in model.named_parameters():
        gathered = [torch.empty_like(p) for _ in range(_world_size())]
        dist.all_gather(gathered, p.detach().contiguous())
        same = same and all(torch.equal(gathered[0], g) for g in gathered)
    return same


if __name__ == "__main__":
    main()
