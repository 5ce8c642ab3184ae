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

    With the native back end and a plain `torch.optim.SGD`, aggregation, error feedback and
    the parameter update run as one fused sequence of kernels (`PowerSGD.fused_step`).
    """
    fused = getattr(aggregator, "supports_fused_step", None)
    if fused is not None and fused(optimizer):
        aggregator.fused_step(optimizer)
        return
    params = params_in_optimizer(optimizer)
    residuals = [p.grad.data for p in params]
    averaged = aggregator.aggregate(residuals)  # `residuals` now hold what was not sent
    for p, g in zip(params, averaged):
        p.grad = g
    optimizer.step()
    for p, g in zip(params, residuals):
        p.grad = g
