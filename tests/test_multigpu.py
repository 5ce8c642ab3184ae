"""In-kernel collectives and the multi-GPU training path (2 ranks, one per GPU)."""
import pytest
import torch

from test_dist_cpu import run_scenario

pytestmark = pytest.mark.gpu

needs_two = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
# plain peer stores only; keep the library's NVLS (in-switch reduction) path out of these runs
ENV = {"NCCL_NVLS_ENABLE": "0"}


@needs_two
@pytest.mark.parametrize("name", ["channel_allreduce", "flat_twoshot", "powersgd_native", "train_step_graph", "channel_timeout", "preflight", "reducers_native", "sparse_reducers_native", "nvls_allreduce", "paper_train_native"])
def test_two_gpu_scenarios(name):
    res = run_scenario(name, nproc=2, timeout=600, env=ENV)
    assert "SCENARIO-OK" in res.stdout, res.stdout[-3000:] + res.stderr[-6000:]


@needs_two
def test_two_gpu_tensor_core_path_with_peer_push():
    """The tcgen05 product kernels push their epilogue to the peers too."""
    res = run_scenario("powersgd_native", nproc=2, timeout=600, env=dict(ENV, PSGD_B200_GEMM="tc"))
    assert "SCENARIO-OK" in res.stdout, res.stdout[-3000:] + res.stderr[-6000:]


@needs_two
def test_two_gpu_library_allreduce_path():
    """PSGD_B200_COMM=nccl: same kernels, factors and flat buffer reduced by the library (eager)."""
    res = run_scenario("powersgd_native_nccl", nproc=2, timeout=600, env=dict(ENV, PSGD_B200_COMM="nccl"))
    assert "SCENARIO-OK" in res.stdout, res.stdout[-3000:] + res.stderr[-6000:]


@needs_two
def test_two_gpu_training_step_raises_when_a_peer_stays_away():
    """Failure detection in the product: 300 ms limit on device-side waits, library NVLS off, the
    in-kernel collectives on plain peer stores."""
    res = run_scenario("train_step_timeout", nproc=2, timeout=600, env=dict(ENV, PSGD_B200_COMM_TIMEOUT_MS="300"))
    assert "SCENARIO-OK" in res.stdout, res.stdout[-3000:] + res.stderr[-6000:]
