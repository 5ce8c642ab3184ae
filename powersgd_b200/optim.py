"""Optimizer glue (powersgd/__init__.py:7-25)."""
from __future__ import annotations

import torch

from .aggregators import Aggregator
from .utils import params_in_optimizer


def optimizer_step(optimizer: torch.optim.Optimizer, aggregator: Aggregator) -> None:
    """Aggregate the gradients over workers, step the optimizer with the aggregate, and
    leave each parameter's `.grad` holding its local residual.

    The next `backward()` accumulates onto that residual, which is how error feedback is
    realised — so the caller must NOT call `optimizer.zero_grad()` between steps.
    """
    params = params_in_optimizer(optimizer)
    residuals = [p.grad.data for p in params]
    averaged = aggregator.aggregate(residuals)  # `residuals` now hold what was not sent
    for p, g in zip(params, averaged):
        p.grad = g
    optimizer.step()
    for p, g in zip(params, residuals):
        p.grad = g
