"""Multi-rank semantics on CPU ranks (gloo, world size 2)."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
WORKER = os.path.join(ROOT, "tests", "dist_worker.py")
_port = [29600 + (os.getpid() % 200)]


def run_scenario(name, nproc=2, timeout=240, env=None):
    _port[0] += 1
    cmd = [
        sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
        "--master-addr", "127.0.0.1", "--master-port", str(_port[0]), WORKER, name,
    ]
    full_env = dict(os.environ)
    full_env.update(env or {})
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=full_env)
    return res


@pytest.mark.parametrize("name", ["mlp_gloo", "ef_identity_gloo", "ddp_hooks_gloo", "preflight_gloo", "plan_mismatch_gloo", "mean_accumulator_gloo"])
def test_gloo_scenarios(name):
    res = run_scenario(name)
    assert "SCENARIO-OK" in res.stdout, res.stdout[-2000:] + res.stderr[-4000:]


def test_rank_failure_is_detected_not_hung():
    res = run_scenario("rank_failure_gloo", timeout=120)
    assert "SCENARIO-OK-FAILING-RANK-LEFT" in res.stdout, res.stdout[-2000:] + res.stderr[-3000:]
    assert "SCENARIO-OK\n" in res.stdout or res.stdout.rstrip().endswith("SCENARIO-OK"), res.stdout[-2000:] + res.stderr[-3000:]
