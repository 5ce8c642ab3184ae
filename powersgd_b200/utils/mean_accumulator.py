"""Running means over nested containers (paper-code/mean_accumulator.py:5-98)."""
from __future__ import annotations

import os
from copy import deepcopy

import torch
import torch.distributed as dist


def _world() -> int:
    return dist.get_world_size() if (dist.is_available() and dist.is_initialized()) else 1


class MeanAccumulator:
    """Weighted running mean of floats, tensors, or dicts / lists of them.

    `update_weight > 1` biases the mean towards recent samples, as in the harness. `reduce()`
    merges the accumulators of all workers (count-weighted) with one all-reduce over all leaves.
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

    def _leaves(self, out: list) -> None:
        """Leaf accumulators of this tree in a deterministic order (dict keys sorted)."""
        if isinstance(self.average, dict):
            for key in sorted(self.average):
                self.average[key]._leaves(out)
        elif isinstance(self.average, list):
            for child in self.average:
                child._leaves(out)
        else:
            out.append(self)

    def reduce(self) -> None:
        """Merges the accumulators of all workers, count-weighted. The original issues two
        all-reduces per leaf (mean_accumulator.py:67-98); here every leaf's count and weighted sum
        sit in ONE float32 buffer that is summed once: by the one-launch in-kernel all-reduce on
        CUDA, by the library collective elsewhere."""
        if _world() == 1:
            return
        leaves: list = []
        self._leaves(leaves)
        leaves = [leaf for leaf in leaves if leaf.average is not None]
        if not leaves:
            return
        on_gpu = dist.get_backend() == "nccl"
        device = torch.device("cuda", torch.cuda.current_device()) if on_gpu else torch.device("cpu")
        parts = []
        for leaf in leaves:
            if isinstance(leaf.average, torch.Tensor):
                value = leaf.average.detach().to(device=device, dtype=torch.float32).reshape(-1) * float(leaf.counter)
            else:
                value = torch.tensor([float(leaf.average) * float(leaf.counter)], dtype=torch.float32, device=device)
            parts.append(torch.tensor([float(leaf.counter)], dtype=torch.float32, device=device))
            parts.append(value)
        flat = torch.cat(parts)
        done = False
        if on_gpu and os.environ.get("PSGD_B200_COMM", "p2p") == "p2p":
            from ..ops import native

            if native.use_for_cuda():
                from ..parallel.symm import native_all_reduce_

                native_all_reduce_(flat)
                done = True
        if not done:
            dist.all_reduce(flat)
        host = flat.cpu() if on_gpu else flat
        at = 0
        for leaf in leaves:
            count = float(host[at])
            at += 1
            if isinstance(leaf.average, torch.Tensor):
                n = leaf.average.numel()
                merged = flat[at : at + n].view(leaf.average.shape) / count
                leaf.average = merged.to(leaf.average.device)
                at += n
            else:
                leaf.average = float(host[at]) / count
                at += 1
            leaf.counter = count
