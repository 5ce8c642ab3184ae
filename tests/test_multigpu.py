"""In-kernel collectives and the multi-GPU training path (2 ranks, one per GPU)."""
import pytest
import torch

from test_dist_cpu import run_scenario

pytestmark = pytest.mark.gpu

needs_two = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
# plain peer stores only; keep the library's in-switch multicast out of these runs
ENV = {"NCCL_NVLS_ENABLE": "0"}


@needs_two
@pytest.mark.parametrize("name", ["channel_allreduce", "powersgd_native", "train_step_graph", "channel_timeout"])
def test_two_gpu_scenarios(name):
    res = run_scenario(name, nproc=2, timeout=600, env=ENV)
    assert "SCENARIO-OK" in res.stdout, res.stdout[-3000:] + res.stderr[-6000:]
