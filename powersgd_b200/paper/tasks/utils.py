"""Data sharding helpers of the research harness.

`DistributedSampler` restates paper-code/tasks/utils.py:8-61: an epoch-seeded permutation that
each rank strides through; padding to equal shard sizes can be switched off (used for the test
split), and iterating advances the epoch by itself.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


class DistributedSampler(torch.utils.data.Sampler):
    def __init__(self, dataset, add_extra_samples: bool = True):
        self._dataset = dataset
        self._num_replicas, self._rank = _world()
        self._add_extra_samples = add_extra_samples
        self._epoch = 0
        n = len(dataset)
        if add_extra_samples:
            self._num_samples = int(math.ceil(n / self._num_replicas))
            self._total_size = self._num_samples * self._num_replicas
        else:
            self._total_size = n
            base, rest = divmod(n, self._num_replicas)
            self._num_samples = base + (1 if self._rank < rest else 0)

    def __iter__(self):
        g = torch.Generator()
        g.manual_seed(self._epoch)
        order = torch.randperm(len(self._dataset), generator=g).tolist()
        if self._add_extra_samples:
            order += order[: self._total_size - len(order)]
        shard = order[self._rank : self._total_size : self._num_replicas]
        assert len(shard) == self._num_samples
        self.set_epoch(self._epoch + 1)
        return iter(shard)

    def __len__(self) -> int:
        return self._num_samples

    def set_epoch(self, epoch: int) -> None:
        self._epoch = epoch


class SyntheticImages(torch.utils.data.Dataset):
    """N(0,1) images with labels uniform over the classes, generated once from a seed.

    Stands in for CIFAR-10 (no network on the build machines); shapes and label space match
    (3 x 32 x 32, 10 classes)."""

    def __init__(self, size: int, seed: int, shape=(3, 32, 32), classes: int = 10):
        g = torch.Generator().manual_seed(seed)
        self.x = torch.randn(size, *shape, generator=g)
        self.y = torch.randint(0, classes, (size,), generator=g)

    def __len__(self) -> int:
        return self.x.shape[0]

    def __getitem__(self, i):
        return self.x[i], self.y[i]


def zipf_tokens(count: int, vocab: int, seed: int, s: float = 1.0) -> torch.Tensor:
    """`count` token ids drawn from a Zipf(s) law over `vocab` symbols."""
    g = torch.Generator().manual_seed(seed)
    weights = 1.0 / torch.arange(1, vocab + 1, dtype=torch.float64) ** s
    return torch.multinomial(weights / weights.sum(), count, replacement=True, generator=g)
