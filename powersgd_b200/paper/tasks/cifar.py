"""Image-classification task (paper-code/tasks/cifar.py:19-228) on CIFAR-shaped data.

Same task interface — `state`, `buffers`, `parameter_names`, `train_iterator`, `batch_loss`,
`batch_loss_and_gradient`, `test`, `state_dict` — and the same metrics (cross entropy, top-1,
top-5). The data is synthetic unless a real CIFAR-10 copy is found under `$DATA/data` by
torchvision (nothing is ever downloaded).
"""
from __future__ import annotations

import os
from copy import deepcopy
from typing import Dict, Iterable, List

import torch
from torch.utils.data import DataLoader

from ... import models as zoo
from ...utils import MeanAccumulator
from .utils import DistributedSampler, SyntheticImages


class Batch:
    def __init__(self, x, y):
        self.x, self.y = x, y


class BatchLoader:
    """Moves (x, y) pairs of a DataLoader to the device and wraps them in `Batch`."""

    def __init__(self, dataloader, device):
        self._dataloader, self._device = dataloader, device

    def __len__(self):
        return len(self._dataloader)

    def __iter__(self):
        for x, y in self._dataloader:
            yield Batch(x.to(self._device, non_blocking=True), y.to(self._device, non_blocking=True))


class CifarTask:
    def __init__(self, device, timer, architecture: str, seed: int, train_size: int = 50_000, test_size: int = 10_000,
                 num_workers: int = 0):
        self._device, self._timer, self._seed, self._architecture = device, timer, seed, architecture
        self._num_workers = num_workers
        self._train_set, self._test_set = self._create_dataset(train_size, test_size)
        self._model = self._create_model()
        self._criterion = torch.nn.CrossEntropyLoss().to(device)
        self._epoch = 0

    # -- task interface ---------------------------------------------------------------------
    @property
    def state(self) -> List[torch.Tensor]:
        return list(self._model.parameters())

    @property
    def buffers(self) -> List[torch.Tensor]:
        return list(self._model.buffers())

    @property
    def parameter_names(self) -> List[str]:
        return [name for name, _ in self._model.named_parameters()]

    def train_iterator(self, batch_size: int) -> Iterable[Batch]:
        sampler = DistributedSampler(self._train_set, add_extra_samples=True)
        sampler.set_epoch(self._epoch)
        loader = DataLoader(self._train_set, batch_size=batch_size, sampler=sampler, pin_memory=self._device.type == "cuda",
                            drop_last=True, num_workers=self._num_workers)
        self._epoch += 1
        return BatchLoader(loader, self._device)

    def batch_loss(self, batch: Batch):
        with torch.no_grad():
            with self._timer("batch.forward", float(self._epoch)):
                prediction = self._model(batch.x)
                loss = self._criterion(prediction, batch.y)
            with self._timer("batch.evaluate", float(self._epoch)):
                metrics = self.evaluate_prediction(prediction, batch.y)
        return loss.item(), metrics

    def batch_loss_and_gradient(self, batch: Batch):
        self._model.zero_grad()
        with self._timer("batch.forward", float(self._epoch)):
            prediction = self._model(batch.x)
            loss = self._criterion(prediction, batch.y)
        with self._timer("batch.backward", float(self._epoch)):
            loss.backward()
        with self._timer("batch.evaluate", float(self._epoch)):
            metrics = self.evaluate_prediction(prediction, batch.y)
        return loss.detach(), [p.grad for p in self._model.parameters()], metrics

    def evaluate_prediction(self, output: torch.Tensor, target: torch.Tensor) -> Dict[str, torch.Tensor]:
        with torch.no_grad():
            top5 = output.topk(min(5, output.shape[1])).indices
            n = len(target)
            return {
                "cross_entropy": self._criterion(output, target).detach(),
                "accuracy": (top5[:, 0] == target).sum().float() / n,
                "top5_accuracy": (top5 == target.unsqueeze(1)).sum().float() / n,
            }

    def test(self, state_dict=None):
        loader = BatchLoader(
            DataLoader(self._test_set, batch_size=250, drop_last=False, num_workers=0,
                       sampler=DistributedSampler(self._test_set, add_extra_samples=False)),
            self._device,
        )
        model = self._create_test_model(state_dict) if state_dict else self._model
        model.eval()
        mean = MeanAccumulator()
        for batch in loader:
            with torch.no_grad():
                mean.add(self.evaluate_prediction(model(batch.x), batch.y))
        mean.reduce()
        model.train()
        return mean.value()

    def state_dict(self):
        return self._model.state_dict()

    # -- internals --------------------------------------------------------------------------
    def _create_model(self):
        torch.random.manual_seed(self._seed)  # identical initial weights on every worker
        model = getattr(zoo, self._architecture)()
        return model.to(self._device).train()

    def _create_test_model(self, state_dict):
        model = deepcopy(self._model)
        model.load_state_dict(state_dict)
        return model.eval()

    def _create_dataset(self, train_size: int, test_size: int):
        root = os.path.join(os.environ.get("DATA", ""), "data")
        if os.environ.get("DATA") and os.path.isdir(os.path.join(root, "cifar-10-batches-py")):
            import torchvision
            import torchvision.transforms as T

            norm = T.Normalize((0.4914, 0.4822, 0.4465), (0.2023, 0.1994, 0.2010))
            train_tf = T.Compose([T.RandomCrop(32, padding=4), T.RandomHorizontalFlip(), T.ToTensor(), norm])
            test_tf = T.Compose([T.ToTensor(), norm])
            ds = torchvision.datasets.CIFAR10
            return ds(root, train=True, download=False, transform=train_tf), ds(root, train=False, download=False, transform=test_tf)
        return SyntheticImages(train_size, seed=1000), SyntheticImages(test_size, seed=2000)
