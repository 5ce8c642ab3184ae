"""Experiment definitions, launcher command lines and the collective benchmark (gloo)."""
import json
import os

import pytest

from powersgd_b200.paper import reducers, schedule

from test_dist_cpu import run_scenario  # noqa: F401  (keeps the shared port counter in one place)


def test_optimizer_config_names():
    cfg = schedule.optimizer_config("Rank 2 (EF)")
    assert cfg["optimizer_reducer"] == "RankKReducer" and cfg["optimizer_reducer_rank"] == 2 and cfg["optimizer_memory"]
    assert schedule.optimizer_config("Top K (136x) (EF)")["optimizer_reducer_compression"] == pytest.approx(1 / 136)
    assert schedule.optimizer_config("Signum")["optimizer_momentum_type"] == "exponential_moving_average"
    assert schedule.optimizer_config("Unbiased Rank 4")["optimizer_memory"] is False
    assert schedule.optimizer_config("Rank 2 w/o reuse (EF)")["optimizer_reducer_reuse_query"] is False
    with pytest.raises(KeyError):
        schedule.optimizer_config("Shuffled rank 2 (EF)")
    for job in list(schedule.ef_compressors()) + list(schedule.scaling_controlled(workers=(1, 2), seeds=(1,))):
        assert job.config_overrides["optimizer_reducer"] in reducers.REDUCERS


def test_every_experiment_generates_jobs_and_commands(tmp_path):
    for name, gen in schedule.EXPERIMENTS.items():
        jobs = list(gen())
        assert jobs, name
        cmd = schedule.command(jobs[0], str(tmp_path))
        assert "torch.distributed.run" in cmd and f"--nproc-per-node={jobs[0].n_workers}" in cmd
        json.loads(cmd[-2])
        text = schedule.slurm_script(jobs[0], str(tmp_path))
        assert text.startswith("#!/bin/bash") and "#SBATCH --nodes=" in text


def test_hyperparameter_record_is_current():
    """The committed record is what the definitions generate (regenerate with
    `python -m powersgd_b200.paper.schedule > powersgd_b200/paper/HYPERPARAMETERS.md`)."""
    path = os.path.join(os.path.dirname(schedule.__file__), "HYPERPARAMETERS.md")
    with open(path) as fp:
        assert fp.read() == schedule.hyperparameter_record()
    assert len(schedule.EXPERIMENTS) == 19  # 17 scripts under schedule/neurips19 + 2 under schedule/pytorch


def test_launch_timings_job_on_two_gloo_ranks(tmp_path):
    job = schedule.Job("timings_gloo_02", 2, {"distributed_backend": "gloo", "device": "cpu", "repetitions": 2,
                                             "message_sizes": [4, 1024, 65536]}, script="timings")
    res = schedule.launch(job, str(tmp_path), master_port=29431 + os.getpid() % 100, timeout=240)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    with open(os.path.join(tmp_path, "timer_summary.json")) as fp:
        summary = json.load(fp)
    for kind in ("all_reduce", "all_gather", "gather", "broadcast"):
        assert f"{kind}_1024" in summary and summary[f"{kind}_1024"]["average_duration"] > 0


def test_launch_train_job_on_two_gloo_ranks(tmp_path):
    job = schedule.Job("rank2", 2, dict(schedule.optimizer_config("Rank 2 (EF)"), distributed_backend="gloo", device="cpu",
                                        num_epochs=1, max_batches_per_epoch=3, optimizer_batch_size=8, task_architecture="LeNet",
                                        train_size=64, test_size=32, log_verbosity=0))
    job.config_overrides.pop("reducer_name")
    res = schedule.launch(job, str(tmp_path), master_port=29531 + os.getpid() % 100, timeout=300)
    assert res.returncode == 0, res.stdout[-1500:] + res.stderr[-3000:]
    assert "last_accuracy" in res.stdout
