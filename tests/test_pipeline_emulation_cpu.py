"""The kernel pipeline's algebra (Gram orthonormalisation + algebraic deflation), restated in
PyTorch, must reproduce the batched reference formulation."""
import pytest
import torch

from powersgd_b200 import BasicConfig, BasicPowerSGD
from powersgd_b200.ops.emulate import emulated_aggregate
from powersgd_b200.orthogonalization import cholesky_qr2_, gram_schmidt_, orthogonalize

# every min(n, m) exceeds rank * iters, so no residual is exhausted (a regime where the factors are rounding noise)
SHAPES = [(24, 3, 3, 3), (24, 24, 3, 3), (24, 24, 3, 3), (40, 24, 1, 1), (20, 64), (33, 65)]


def _rel(a, b):
    return ((a - b).norm() / b.norm().clamp_min(1e-30)).item()


@pytest.mark.parametrize("rank,iters", [(1, 1), (1, 2), (2, 2), (3, 3), (4, 4), (2, 1)])
def test_emulated_pipeline_matches_batched_formulation(rank, iters):
    torch.set_default_dtype(torch.float64)
    torch.manual_seed(0)
    params = [torch.zeros(s) for s in SHAPES]
    a = BasicPowerSGD(params, BasicConfig(rank=rank, num_iters_per_step=iters))
    b = BasicPowerSGD(params, BasicConfig(rank=rank, num_iters_per_step=iters))
    ga = [torch.randn(s) for s in SHAPES]
    gb = [g.clone() for g in ga]
    for _ in range(3):
        oa = emulated_aggregate(a, ga)
        a.step_counter += 1
        ob = b.aggregate(gb)
        for x, y in zip(oa, ob):
            assert _rel(x, y) < 1e-9
        for x, y in zip(ga, gb):
            assert _rel(x, y) < 1e-9
        n = [torch.randn(s) for s in SHAPES]
        for x, y, z in zip(ga, gb, n):
            x.add_(z)
            y.add_(z)


def test_three_orthonormalisations_span_the_same_space():
    torch.manual_seed(0)
    x = torch.randn(2, 300, 5, dtype=torch.float64)
    q1 = orthogonalize(x.clone())
    q2 = cholesky_qr2_(x.clone())
    q3 = torch.stack([gram_schmidt_(x[i].clone(), eps=0.0) for i in range(2)])
    for q in (q1, q2, q3):
        eye = torch.eye(5, dtype=torch.float64)
        assert torch.allclose(q.transpose(1, 2) @ q, eye.expand(2, 5, 5), atol=1e-10)
    p1, p2, p3 = (q @ q.transpose(1, 2) for q in (q1, q2, q3))
    assert torch.allclose(p1, p2, atol=1e-9) and torch.allclose(p1, p3, atol=1e-9)


def test_cholesky_qr_handles_zero_and_dependent_columns():
    x = torch.zeros(1, 50, 3)
    q = cholesky_qr2_(x.clone())
    assert torch.isfinite(q).all()
    assert torch.allclose(q[0].T @ q[0], torch.eye(3), atol=1e-6)
    y = torch.randn(1, 50, 3)
    y[0, :, 2] = y[0, :, 0] * 2.0
    q = cholesky_qr2_(y.clone())
    assert torch.isfinite(q).all()
    assert torch.allclose(q[0].T @ q[0], torch.eye(3), atol=1e-5)
