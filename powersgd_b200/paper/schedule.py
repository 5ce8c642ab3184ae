"""Experiment definitions of the paper as plain data, and a local launcher.

The reference drives its experiments through a MongoDB-backed job monitor on a Kubernetes /
Slurm cluster (paper-code/schedule/neurips19/*.py, paper-code/environment/cluster.py). On one
8 x B200 box none of that is needed: an experiment is a list of `Job`s (name, worker count,
config overrides, script) that `launch()` runs with `torch.distributed.run`, one process per
GPU, and `slurm_script()` renders as an sbatch file for multi-node clusters.

`optimizer_config(name)` maps the display names used throughout the paper ("Rank 2 (EF)",
"Signum", "Top K (136x) (EF)", ...) to config overrides (schedule/neurips19/shared.py:71-256).
Names whose reducers never existed in the published tree (ShuffledRankKReducer,
FasterRank1Reducer, StratifiedTopKReducer, the SuperResolution task) raise `KeyError`.
"""
from __future__ import annotations

import os
import re
import subprocess
import sys
from dataclasses import dataclass, field
from typing import Dict, Iterator, List


def sgd_config(lr: float, momentum: float, weight_decay: float) -> Dict:
    return {
        "optimizer_learning_rate": lr,
        "optimizer_conv_learning_rate": lr,
        "optimizer_weight_decay_other": weight_decay,
        "optimizer_weight_decay_conv": weight_decay,
        "optimizer_momentum": momentum,
    }


def language_modeling_base() -> Dict:
    return {
        "task": "LanguageModeling",
        "optimizer_weight_decay_other": 0,
        "optimizer_weight_decay_conv": 0,
        "optimizer_batch_size": 64,
        "optimizer_learning_rate": 20,
        "optimizer_decay_at_epochs": [60, 80],
        "optimizer_momentum": 0,
        "num_epochs": 90,
    }


_PATTERNS = [
    (r"Rank (\d+) \(EF\)$", lambda m: dict(optimizer_reducer="RankKReducer", optimizer_reducer_rank=int(m[1]),
                                          optimizer_reducer_reuse_query=True, optimizer_reducer_n_power_iterations=0,
                                          optimizer_memory=True)),
    (r"Rank (\d+) w/o reuse \(EF\)$", lambda m: dict(optimizer_reducer="RankKReducer", optimizer_reducer_rank=int(m[1]),
                                                     optimizer_reducer_reuse_query=False,
                                                     optimizer_reducer_n_power_iterations=0, optimizer_memory=True)),
    (r"Half Rank (\d+) \(EF\)$", lambda m: dict(optimizer_reducer="HalfRankKReducer", optimizer_reducer_rank=int(m[1]),
                                               optimizer_memory=True)),
    (r"Unbiased Rank (\d+)$", lambda m: dict(optimizer_reducer="HalfRankKReducer", optimizer_reducer_rank=int(m[1]),
                                            optimizer_memory=False)),
    (r"SVD Rank (\d+) \(EF\)$", lambda m: dict(optimizer_reducer="SVDReducer", optimizer_reducer_rank=int(m[1]),
                                              optimizer_memory=True)),
    (r"Atomo \(rank (\d+)\)$", lambda m: dict(optimizer_reducer="AtomoReducer", optimizer_reducer_rank=int(m[1]),
                                             optimizer_memory=False)),
    (r"Random K \((\d+)x\) \(EF\)$", lambda m: dict(optimizer_reducer="UniformRandomSparseReducer",
                                                   optimizer_reducer_compression=1 / int(m[1]), optimizer_memory=True)),
    (r"Random Block \((\d+)x\) \(EF\)$", lambda m: dict(optimizer_reducer="UniformRandomSparseBlockReducer",
                                                       optimizer_reducer_compression=1 / int(m[1]), optimizer_memory=True)),
    (r"Random K \(rank (\d+)\) \(EF\)$", lambda m: dict(optimizer_reducer="RandomSparseReducer",
                                                       optimizer_reducer_rank=int(m[1]), optimizer_memory=True)),
    (r"Random Block \(rank (\d+)\) \(EF\)$", lambda m: dict(optimizer_reducer="RandomSparseBlockReducer",
                                                           optimizer_reducer_rank=int(m[1]), optimizer_memory=True)),
    (r"Top K \((\d+)x\) \(EF\)$", lambda m: dict(optimizer_reducer="TopKReducer",
                                                optimizer_reducer_compression=1 / int(m[1]), optimizer_memory=True)),
    (r"Global Top K \((\d+)x\) \(EF\)$", lambda m: dict(optimizer_reducer="GlobalTopKReducer",
                                                       optimizer_reducer_compression=1 / int(m[1]), optimizer_memory=True)),
]
_FIXED = {
    "SGD": dict(optimizer_reducer="ExactReducer", optimizer_memory=False),
    "Top K (EF)": dict(optimizer_reducer="TopKReducer", optimizer_reducer_compression=1 / 244, optimizer_memory=True),
    "Signum": dict(optimizer_reducer="SignSGDwithMajorityVoteReducer", optimizer_memory=False,
                   optimizer_mom_before_reduce=True, optimizer_wd_before_reduce=True,
                   optimizer_momentum_type="exponential_moving_average"),
    "Sign+Norm (EF)": dict(optimizer_reducer="SignAndNormReducer", optimizer_memory=True),
    "Sign (EF)": dict(optimizer_reducer="SignReducer", optimizer_memory=True),
}


def optimizer_config(reducer: str) -> Dict:
    if reducer in _FIXED:
        return dict(_FIXED[reducer], reducer_name=reducer)
    for pattern, build in _PATTERNS:
        match = re.match(pattern, reducer)
        if match:
            return dict(build(match), reducer_name=reducer)
    raise KeyError(f"no reducer of this library matches the name {reducer!r}")


@dataclass
class Job:
    name: str
    n_workers: int
    config_overrides: Dict = field(default_factory=dict)
    script: str = "train"  # "train" (research loop) or "timings" (collective sweep)


def scaling_controlled(workers=(1, 2, 4, 8), seeds=(1, 2, 3), backends=("nccl",)) -> Iterator[Job]:
    """Timing / scaling protocol: ResNet-18, batch 128 per worker, SGD vs Rank 2 vs Signum, each
    at timer verbosity 1 and 2 (schedule/neurips19/scaling_controlled.py:48-79)."""
    for backend in backends:
        for reducer in ["SGD", "Rank 2 (EF)", "Signum"]:
            for log_level in [1, 2]:
                for seed in seeds:
                    for n in workers:
                        yield Job(f"{reducer}_{n:02d}workers_{backend}_l{log_level}_s{seed}", n, {
                            "seed": 10000 + seed, "optimizer_scale_lr_with_factor": n, "distributed_backend": backend,
                            "log_verbosity": log_level, "num_epochs": 10,
                            **sgd_config(0.1, momentum=0.9, weight_decay=0.0001), **optimizer_config(reducer)})


def rank_tuning(n_workers: int = 8) -> Iterator[Job]:
    for rank in [2, 4]:
        for lr in [0.2, 0.1, 0.05]:
            yield Job(f"rank{rank}_lr{lr}", n_workers, {"seed": 42, "num_epochs": 300, "task_architecture": "ResNet18",
                                                         **sgd_config(lr, 0.9, 0.0001), **optimizer_config(f"Rank {rank} (EF)")})


def ef_compressors(n_workers: int = 8, lr: float = 0.1) -> Iterator[Job]:
    """Error-feedback compressors at the communication budget of rank-2 / rank-7 PowerSGD."""
    names = ["Rank 2 (EF)", "Random Block (136x) (EF)", "Random K (136x) (EF)", "Top K (136x) (EF)", "Sign+Norm (EF)",
             "Rank 7 (EF)", "Random Block (32x) (EF)", "Random K (32x) (EF)", "Top K (32x) (EF)", "SGD"]
    for name in names:
        yield Job(name, n_workers, {"seed": 1, "num_epochs": 300, **sgd_config(lr, 0.9, 0.0001), **optimizer_config(name)})


def lm_rank(n_workers: int = 8) -> Iterator[Job]:
    for lr in [2.5, 1.25, 0.6]:
        for rank in [1, 2, 4]:
            yield Job(f"lm_rank{rank}_lr{lr}", n_workers, {"seed": 42, **language_modeling_base(),
                                                            **sgd_config(lr, 0.0, 0.0), **optimizer_config(f"Rank {rank} (EF)")})


def warm_start(n_workers: int = 8, lr: float = 0.1) -> Iterator[Job]:
    for name in ["Rank 1 (EF)", "Rank 1 w/o reuse (EF)", "Rank 2 (EF)", "Rank 2 w/o reuse (EF)"]:
        yield Job(name, n_workers, {"seed": 42, "num_epochs": 300, **sgd_config(lr, 0.9, 0.0001), **optimizer_config(name)})


def system_characterization(workers=(2, 4, 8), backends=("nccl", "gloo"), repetitions: int = 20) -> Iterator[Job]:
    for backend in backends:
        for n in workers:
            yield Job(f"timings_{backend}_{n:02d}", n, {"distributed_backend": backend, "repetitions": repetitions,
                                                        "device": "cuda" if backend == "nccl" else "cpu"}, script="timings")


def _cifar_job(name: str, reducer: str, n_workers: int, lr: float, seed: int, **extra) -> Job:
    """A 300-epoch ResNet-18 / CIFAR-10 run with the paper's base optimizer settings."""
    return Job(name, n_workers, {"seed": seed, "distributed_backend": "nccl", "optimizer_scale_lr_with_factor": n_workers,
                                 "num_epochs": 300, "log_verbosity": 1, **sgd_config(lr, momentum=0.9, weight_decay=0.0001),
                                 **optimizer_config(reducer), **extra})


def _lr_sweep(reducer: str, rates, n_workers: int) -> Iterator[Job]:
    for lr in rates:
        yield _cifar_job(f"{reducer}_{n_workers:02d}workers_lr{lr}", reducer, n_workers, lr, seed=42)


def sgd_tuning(n_workers: int = 8) -> Iterator[Job]:
    """Learning rate of the uncompressed baseline (schedule/neurips19/sgd_tuning.py)."""
    return _lr_sweep("SGD", [0.2, 0.1, 0.05, 0.025], n_workers)


def signum_tuning(n_workers: int = 8) -> Iterator[Job]:
    """(schedule/neurips19/signum_tuning.py)"""
    return _lr_sweep("Signum", [0.0001, 0.0002, 0.00005, 0.000025], n_workers)


def atomo_tuning(n_workers: int = 8) -> Iterator[Job]:
    """(schedule/neurips19/atomo_tuning.py)"""
    return _lr_sweep("Atomo (rank 2)", [0.2, 0.1, 0.05, 0.025], n_workers)


def xvvt_tuning(n_workers: int = 8) -> Iterator[Job]:
    """Unbiased rank-1 compression without error feedback (schedule/neurips19/xvvt_tuning.py)."""
    return _lr_sweep("Unbiased Rank 1", [0.1, 0.05, 0.025, 0.0125, 0.00625], n_workers)


def xvvt_rank2_tuning(n_workers: int = 8) -> Iterator[Job]:
    """(schedule/neurips19/xvvt_rank2_tuning.py)"""
    return _lr_sweep("Unbiased Rank 2", [0.1, 0.05, 0.025, 0.0125, 0.00625], n_workers)


def top_k_tuning(n_workers: int = 8) -> Iterator[Job]:
    """Top-K with error feedback at the budgets of rank 1 / 4 / 7 (schedule/neurips19/top_k_tuning.py)."""
    for compression in [244, 72, 32]:
        for lr in [0.1, 0.05]:
            yield _cifar_job(f"Top K (EF)_{n_workers:02d}workers_lr{lr}_{compression}x", "Top K (EF)", n_workers, lr, seed=42,
                             optimizer_reducer_compression=1 / compression)


def right_rank(n_workers: int = 8) -> Iterator[Job]:
    """Full against half power-iteration steps at ranks 1, 2, 4 (schedule/neurips19/right_rank.py)."""
    for rank in [1, 2, 4]:
        for name in (f"Half Rank {rank} (EF)", f"Rank {rank} (EF)"):
            yield _cifar_job(name, name, n_workers, 0.1, seed=1000)


QUALITY_VARIANCE_REDUCERS = [
    "SGD", "Rank 1 (EF)", "Rank 2 (EF)", "Rank 4 (EF)", "Rank 7 (EF)", "Rank 2 w/o reuse (EF)", "HQ Rank 2 w/o reuse (EF)",
    "Random K (rank 2) (EF)", "Random K (rank 7) (EF)", "Random Block (rank 2) (EF)", "Random Block (rank 7) (EF)",
    "Sign+Norm (EF)", "Top K (136x) (EF)", "Top K (32x) (EF)", "Top K (rank 2) (EF)", "Top K (rank 7) (EF)", "Signum",
    "Unbiased Rank 1", "Unbiased Rank 2", "Atomo (rank 2)", "Atomo (rank 1)",
]


def quality_variance(n_workers: int = 8, seeds=(1, 2, 3)) -> Iterator[Job]:
    """Every compressor of the main results table at its tuned learning rate, three seeds
    (schedule/neurips19/quality_variance.py). The original list also names compressors whose
    classes were never published (`HQ Rank 2 w/o reuse`: two extra power iterations, which the
    rank-k reducer refuses; `Top K (rank N)`: a stratified top-k); those entries are skipped."""
    tuned = {"Signum": 0.00005, "Unbiased Rank 1": 0.0125, "Unbiased Rank 2": 0.0125}
    for reducer in QUALITY_VARIANCE_REDUCERS:
        try:
            optimizer_config(reducer)
        except KeyError:
            continue
        for seed in seeds:
            yield _cifar_job(f"{reducer}_{n_workers:02d}workers_seed{seed}", reducer, n_workers, tuned.get(reducer, 0.1), seed)


def _lm_job(name: str, reducer: str, n_workers: int, lr: float, momentum: float, seed: int) -> Job:
    return Job(name, n_workers, {"seed": seed, "distributed_backend": "nccl", "optimizer_scale_lr_with_factor": n_workers,
                                 "log_verbosity": 1, **language_modeling_base(), **sgd_config(lr, momentum=momentum, weight_decay=0.0),
                                 **optimizer_config(reducer)})


def lm_sgd_tuning(n_workers: int = 8) -> Iterator[Job]:
    """(schedule/neurips19/lm_sgd_tuning.py)"""
    for lr in [2.5, 1.25, 0.6]:
        yield _lm_job(f"SGD_{n_workers:02d}workers_lr{lr}", "SGD", n_workers, lr, 0.0, seed=42)


def lm_signum_tuning(n_workers: int = 8) -> Iterator[Job]:
    """(schedule/neurips19/lm_signum_tuning.py)"""
    for lr in [0.0001, 0.0002, 0.00005, 1e-5, 1e-6]:
        yield _lm_job(f"Signum_{n_workers:02d}workers_lr{lr}", "Signum", n_workers, lr, 0.9, seed=42)


def lm_quality_variance(n_workers: int = 8, seeds=(1, 2, 3)) -> Iterator[Job]:
    """(schedule/neurips19/lm_quality_variance.py)"""
    for reducer in ["SGD", "Rank 1 (EF)", "Rank 2 (EF)", "Rank 4 (EF)", "Signum"]:
        lr, momentum = (1e-5, 0.9) if reducer == "Signum" else (1.25, 0.0)
        for seed in seeds:
            yield _lm_job(f"{reducer}_{n_workers:02d}workers_seed{seed}", reducer, n_workers, lr, momentum, seed)


def varying_rank_ours(n_workers: int = 8, seeds=(1, 2)) -> Iterator[Job]:
    """This code base's rank 4 / 2 / 1 against plain all-reduce (schedule/pytorch/varying_rank_ours.py)."""
    for seed in seeds:
        for label, reducer in [("powersgd-rank4", "Rank 4 (EF)"), ("powersgd-rank2", "Rank 2 (EF)"),
                               ("powersgd-rank1", "Rank 1 (EF)"), ("all-reduce", "SGD")]:
            yield _cifar_job(f"{n_workers:02d}workers_{label}_seed{seed}", reducer, n_workers, 0.1, seed)


def varying_rank_ddp(n_workers: int = 8, seeds=(2,)) -> Iterator[Job]:
    """The same comparison through PyTorch DDP's built-in communication hooks
    (schedule/pytorch/varying_rank.py): PowerSGD hook at ranks 4 / 2 / 1, fp16 compression, plain
    all-reduce. Runs `paper/train_ddp.py`."""
    for seed in seeds:
        for label, hook, rank in [("powersgd-rank4", "PowerSGD", 4), ("powersgd-rank2", "PowerSGD", 2),
                                  ("powersgd-rank1", "PowerSGD", 1), ("fp16", "fp16", None), ("all-reduce", "allreduce", None)]:
            cfg = {"seed": seed, "distributed_backend": "nccl", "optimizer_scale_lr_with_factor": n_workers, "log_verbosity": 1,
                   **sgd_config(0.1, momentum=0.9, weight_decay=0.0001), "optimizer_reducer": hook}
            if rank is not None:
                cfg["optimizer_reducer_rank"] = rank
            yield Job(f"{n_workers:02d}workers_{label}_seed{seed}", n_workers, cfg, script="train_ddp")


EXPERIMENTS = {f.__name__: f for f in (
    scaling_controlled, system_characterization, sgd_tuning, signum_tuning, atomo_tuning, xvvt_tuning, xvvt_rank2_tuning,
    top_k_tuning, rank_tuning, right_rank, warm_start, ef_compressors, quality_variance, lm_sgd_tuning, lm_signum_tuning,
    lm_rank, lm_quality_variance, varying_rank_ours, varying_rank_ddp)}

_RUNNER = (
    "import json,sys;from powersgd_b200.paper import {mod} as m;"
    "m.config.update(json.loads(sys.argv[1]));m.output_dir=sys.argv[2];m.main()"
)


def command(job: Job, output_dir: str, master_port: int = 29555) -> List[str]:
    """The `torch.distributed.run` command line that runs `job` on this machine."""
    import json

    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={job.n_workers}",
            "--master-addr", "127.0.0.1", "--master-port", str(master_port), "--no-python", sys.executable, "-c",
            _RUNNER.format(mod=job.script), json.dumps(job.config_overrides), output_dir]


def launch(job: Job, output_dir: str, master_port: int = 29555, timeout=None) -> subprocess.CompletedProcess:
    os.makedirs(output_dir, exist_ok=True)
    return subprocess.run(command(job, output_dir, master_port), capture_output=True, text=True, timeout=timeout)


def slurm_script(job: Job, output_dir: str, gpus_per_node: int = 8, partition: str = "b200") -> str:
    """An sbatch file for the same job on a Slurm cluster (replaces the GCP/Slurm provisioning of
    paper-code/environment/cluster.py with the scheduler the site already runs)."""
    import json

    nodes = max(1, -(-job.n_workers // gpus_per_node))
    per_node = min(job.n_workers, gpus_per_node)
    payload = json.dumps(job.config_overrides).replace("'", "'\\''")
    return "\n".join([
        "#!/bin/bash",
        f"#SBATCH --job-name={re.sub(r'[^A-Za-z0-9_.-]', '_', job.name)}",
        f"#SBATCH --partition={partition}", f"#SBATCH --nodes={nodes}", f"#SBATCH --ntasks-per-node=1",
        f"#SBATCH --gres=gpu:{per_node}", f"#SBATCH --output={output_dir}/slurm-%j.out", "",
        "head=$(scontrol show hostnames $SLURM_JOB_NODELIST | head -n 1)",
        f"srun python -m torch.distributed.run --nnodes={nodes} --nproc-per-node={per_node} \\",
        "  --rdzv-backend=c10d --rdzv-endpoint=$head:29500 --no-python python -c \\",
        f"  '{_RUNNER.format(mod=job.script)}' '{payload}' {output_dir}", "",
    ])


def hyperparameter_record(max_rows: int = 1000) -> str:
    """Markdown record of every experiment's jobs and overrides (what the reference keeps as
    config dumps in paper-code/hyperparameters.md), generated from the definitions above:
    `python -m powersgd_b200.paper.schedule > powersgd_b200/paper/HYPERPARAMETERS.md`."""
    from . import train

    lines = [
        "# Hyper-parameters of the experiment definitions", "",
        "Generated by `python -m powersgd_b200.paper.schedule` from `powersgd_b200/paper/schedule.py` (the reference keeps the",
        "same information as config dumps in paper-code/hyperparameters.md). Every job starts from the defaults of",
        "`paper/train.py::config` and applies the overrides listed here.", "", "## Defaults", "", "| key | value |", "|---|---|",
    ]
    lines += [f"| `{k}` | `{v}` |" for k, v in train.config.items()]
    for name, gen in EXPERIMENTS.items():
        jobs = list(gen())
        lines += ["", f"## {name} ({len(jobs)} jobs)", "", " ".join((gen.__doc__ or "").split()), "",
                  "| job | workers | script | overrides |", "|---|---|---|---|"]
        for job in jobs[:max_rows]:
            overrides = ", ".join(f"{k}={v}" for k, v in job.config_overrides.items())
            lines.append(f"| {job.name} | {job.n_workers} | {job.script} | {overrides} |")
        if len(jobs) > max_rows:
            lines.append(f"| ... {len(jobs) - max_rows} more (same pattern) | | | |")
    return "\n".join(lines) + "\n"


if __name__ == "__main__":
    sys.stdout.write(hyperparameter_record())
