"""Running means over nested containers (paper-code/mean_accumulator.py:5-98)."""
from __future__ import annotations

from copy import deepcopy

import torch
import torch.distributed as dist


def _world() -> int:
    return dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1


class MeanAccumulator:
    """Weighted running mean of floats, tensors, or dicts / lists of them.

    `update_weight > 1` biases the mean towards recent samples, as in the harness. `reduce()`
    merges the accumulators of all workers (count-weighted) with two async all-reduces.
    """

    def __init__(self, update_weight: float = 1):
        self.update_weight = update_weight
        self.reset()

    def reset(self) -> None:
        self.average = None
        self.counter = 0

    def value(self):
        avg = self.average
        if isinstance(avg, dict):
            return {k: child.value() for k, child in avg.items()}
        if isinstance(avg, list):
            return [child.value() for child in avg]
        return avg

    def add(self, value, weight: float = 1.0) -> None:
        self.counter += weight
        if self.average is None:
            self._start(value, weight)
        elif isinstance(self.average, dict):
            for k, v in value.items():
                self.average[k].add(v, weight)
        elif isinstance(self.average, list):
            for child, v in zip(self.average, value):
                child.add(v, weight)
        else:
            self._blend(value, weight)

    def _start(self, value, weight: float) -> None:
        if isinstance(value, dict):
            self.average = {}
            for k, v in value.items():
                child = MeanAccumulator()
                child.add(v, weight)
                self.average[k] = child
        elif isinstance(value, (list, tuple)):
            self.average = []
            for v in value:
                child = MeanAccumulator()
                child.add(v, weight)
                self.average.append(child)
        else:
            self.average = deepcopy(value)

    def _blend(self, value, weight: float) -> None:
        alpha = float(self.update_weight * weight) / float(self.counter + self.update_weight - 1)
        if isinstance(self.average, torch.Tensor):
            self.average = self.average.float()
            self.average.mul_(1.0 - alpha).add_(value, alpha=alpha)
        elif isinstance(self.average, (float, int)):
            self.average = (1.0 - alpha) * self.average + alpha * float(value)
        else:
            raise ValueError(f"cannot average values of type {type(self.average)}")

    def reduce(self) -> None:
        if _world() == 1:
            return
        if isinstance(self.average, dict):
            for key in sorted(self.average):
                self.average[key].reduce()
            return
        if isinstance(self.average, list):
            for child in self.average:
                child.reduce()
            return
        device = "cuda" if dist.get_backend() == "nccl" else "cpu"
        count = torch.tensor(float(self.counter), dtype=torch.float32, device=device)
        h_count = dist.all_reduce(count, async_op=True)
        if isinstance(self.average, torch.Tensor):
            weighted = self.average.detach().clone().to(device)
        else:
            weighted = torch.tensor(float(self.average), dtype=torch.float32, device=device)
        weighted.mul_(self.counter)
        h_sum = dist.all_reduce(weighted, async_op=True)
        h_count.wait()
        h_sum.wait()
        self.counter = count.item()
        merged = weighted / count
        if isinstance(self.average, torch.Tensor):
            self.average = merged.to(self.average.device)
        else:
            self.average = merged.item()
