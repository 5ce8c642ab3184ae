"""Checkpointable state of an aggregator.

The reference library has no resume path: its warm-start factors, its two step counters,
its generator and the error-feedback residuals (which live in `p.grad`) are lost on
restart (powersgd/powersgd.py:52, 123-144; powersgd/__init__.py:24-25). This module
defines the format that captures all of them:

    {
      "format": 1,
      "config": {...}, "is_compressed_mask": [...],
      "step_counter": int,                 # policy wrapper: counts every aggregate() call
      "compressor": {
          "step_counter": int,             # counts compressed steps only; sets the parity
          "generator_state": ByteTensor,
          "groups": [ {"shape": [n, m], "rank": r, "members": [...],
                       "p": [B, n, r], "q": [B, m, r],
                       "error": [B, n, m] or None}, ... ] },
      "plain_error": [tensor, ...] or None   # residuals of uncompressed tensors (zeros)
    }

Factors and residuals are stored per shape group, which is also how the kernels see them.
"""
from __future__ import annotations

import warnings
from typing import Dict, Optional, Sequence

import torch

FORMAT = 1


def compressor_state_dict(core, gradients: Optional[Sequence[torch.Tensor]] = None) -> Dict:
    groups = []
    for gi, g in enumerate(core.plan.groups):
        entry = {
            "shape": [g.n, g.m],
            "rank": g.r,
            "members": list(g.members),
            "p": core._ps[gi].detach().clone().cpu(),
            "q": core._qs[gi].detach().clone().cpu(),
            "error": None,
        }
        if gradients is not None:
            # logical order ([shape[0], rest] of the contiguous view), whatever the memory format
            entry["error"] = torch.stack(
                [gradients[i].detach().reshape(g.n, g.m) for i in g.members]
            ).cpu()
        groups.append(entry)
    return {
        "step_counter": core.step_counter,
        "generator_state": core.generator.get_state().clone().cpu(),
        "rank": core.config.rank,
        "num_iters_per_step": core.config.num_iters_per_step,
        "groups": groups,
    }


def load_compressor_state_dict(core, state: Dict, gradients: Optional[Sequence[torch.Tensor]] = None) -> None:
    if len(state["groups"]) != len(core.plan.groups):
        raise ValueError("checkpoint has a different number of shape groups")
    if int(state["rank"]) != int(core.config.rank) or int(state["num_iters_per_step"]) != int(
        core.config.num_iters_per_step
    ):
        raise ValueError("checkpoint was written with a different rank / num_iters_per_step")
    for gi, (g, entry) in enumerate(zip(core.plan.groups, state["groups"])):
        if list(entry["shape"]) != [g.n, g.m] or int(entry["rank"]) != g.r or list(entry["members"]) != list(g.members):
            raise ValueError(f"shape group {gi} of the checkpoint does not match the model")
        core._ps[gi].copy_(entry["p"].to(core.device))
        core._qs[gi].copy_(entry["q"].to(core.device))
        if gradients is not None and entry.get("error") is not None:
            for pos, idx in enumerate(g.members):
                # write through the tensor itself: `reshape` of a channels_last gradient would
                # return a copy and the restored residual would be lost
                dst = gradients[idx]
                dst.copy_(entry["error"][pos].to(dst.device).view(dst.shape))
    core.step_counter = int(state["step_counter"])
    native = getattr(core, "_native", None)
    if native is not None:
        native._early = None  # a basis orthonormalised ahead of time came from the factors just replaced
    try:
        core.generator.set_state(state["generator_state"].cpu())
    except RuntimeError as exc:
        # a generator state only restores onto the device type that produced it; the generator is
        # only used to draw the initial factors, which the checkpoint has just overwritten
        warnings.warn(f"PowerSGD checkpoint: generator state not restored ({exc})")


def aggregator_state_dict(agg, gradients: Optional[Sequence[torch.Tensor]] = None) -> Dict:
    lowrank = plain = None
    if gradients is not None:
        lowrank, plain = agg._split(list(gradients))
    return {
        "format": FORMAT,
        "config": dict(agg.config._asdict()),
        "is_compressed_mask": list(agg.is_compressed_mask),
        "step_counter": agg.step_counter,
        "compressor": compressor_state_dict(agg._powersgd, lowrank),
        "plain_error": None if plain is None else [t.detach().clone().cpu() for t in plain],
    }


def load_aggregator_state_dict(agg, state: Dict, gradients: Optional[Sequence[torch.Tensor]] = None) -> None:
    if state.get("format") != FORMAT:
        raise ValueError(f"unsupported checkpoint format {state.get('format')!r}")
    if list(state["is_compressed_mask"]) != list(agg.is_compressed_mask):
        raise ValueError("checkpoint's compression mask does not match this model / config")
    for key, value in state["config"].items():
        if getattr(agg.config, key) != value:
            raise ValueError(f"checkpoint config differs in {key!r}: {value} != {getattr(agg.config, key)}")
    lowrank = plain = None
    if gradients is not None:
        lowrank, plain = agg._split(list(gradients))
    load_compressor_state_dict(agg._powersgd, state["compressor"], lowrank)
    if plain is not None and state.get("plain_error") is not None:
        for dst, src in zip(plain, state["plain_error"]):
            dst.copy_(src.to(dst.device))
    agg.step_counter = int(state["step_counter"])
