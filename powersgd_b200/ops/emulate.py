"""Pure-PyTorch restatement of the native kernel pipeline (same bookkeeping, same algebra).

Runs anywhere (CPU included). It exists to pin down, independently of CUDA, the formulation
that the kernels implement: Gram-matrix orthonormalisation, algebraic deflation through
r x r cross products, and the single decompression pass. Tests compare it with the batched
reference formulation in `aggregators.BasicPowerSGD._aggregate_torch`.
"""
from __future__ import annotations

from typing import List

import torch

from ..orthogonalization import cholesky_qr2_
from ..utils import world_size


def _orth_units(core, side: str, buf: torch.Tensor) -> None:
    for g in core.plan.groups:
        length = g.n if side == "p" else g.m
        off = g.p_offset if side == "p" else g.q_offset
        block = buf[off : off + g.batch * length * g.r].view(g.batch, length, g.r)
        if g.r == 1:
            block.div_(torch.clamp(block.norm(), min=1e-16))
        else:
            cholesky_qr2_(block, passes=1)


def emulated_aggregate(core, gradients: List[torch.Tensor], allreduce=None) -> List[torch.Tensor]:
    """Same contract as `BasicPowerSGD.aggregate` (without the step-counter increment)."""
    plan, T = core.plan, core.config.num_iters_per_step
    W = world_size()
    mats = [g.view(g.shape[0], -1) for g in gradients]
    h_in, h_loc, h_sum, sides = [], [], [], []
    for t in range(T):
        left = (core.step_counter * T + t) % 2 == 0
        sides.append(left)
        state_in = core._ps_buffer if left else core._qs_buffer
        state_out = core._qs_buffer if left else core._ps_buffer
        _orth_units(core, "p" if left else "q", state_in)
        basis = state_in.clone()
        fresh = torch.zeros_like(state_out)
        for g in plan.groups:
            for pos, idx in enumerate(g.members):
                M = mats[idx]
                po, qo = g.p_offset + pos * g.n * g.r, g.q_offset + pos * g.m * g.r
                P = lambda b: b[po : po + g.n * g.r].view(g.n, g.r)  # noqa: E731
                Q = lambda b: b[qo : qo + g.m * g.r].view(g.m, g.r)  # noqa: E731
                if left:
                    out = M.t() @ P(basis)
                    for i in range(t):
                        Lloc = P(h_in[i]) if sides[i] else P(h_loc[i])
                        Rloc = Q(h_loc[i]) if sides[i] else Q(h_in[i])
                        out -= Rloc @ (Lloc.t() @ P(basis))
                    Q(fresh).copy_(out)
                else:
                    out = M @ Q(basis)
                    for i in range(t):
                        Lloc = P(h_in[i]) if sides[i] else P(h_loc[i])
                        Rloc = Q(h_loc[i]) if sides[i] else Q(h_in[i])
                        out -= Lloc @ (Rloc.t() @ Q(basis))
                    P(fresh).copy_(out)
        summed = fresh.clone()
        if allreduce is not None and W > 1:
            allreduce(summed)
        state_out.copy_(summed)
        h_in.append(basis)
        h_loc.append(fresh)
        h_sum.append(summed)

    outputs = [torch.empty_like(g) for g in gradients]
    for g in plan.groups:
        for pos, idx in enumerate(g.members):
            po, qo = g.p_offset + pos * g.n * g.r, g.q_offset + pos * g.m * g.r
            P = lambda b: b[po : po + g.n * g.r].view(g.n, g.r)  # noqa: E731
            Q = lambda b: b[qo : qo + g.m * g.r].view(g.m, g.r)  # noqa: E731
            approx = torch.zeros_like(mats[idx])
            for t, left in enumerate(sides):
                if left:
                    mats[idx].sub_(P(h_in[t]) @ Q(h_loc[t]).t())
                    approx.add_(P(h_in[t]) @ Q(h_sum[t]).t())
                else:
                    mats[idx].sub_(P(h_loc[t]) @ Q(h_in[t]).t())
                    approx.add_(P(h_sum[t]) @ Q(h_in[t]).t())
            outputs[idx].view_as(approx).copy_(approx / W)
    return outputs
