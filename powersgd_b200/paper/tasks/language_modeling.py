"""Language-modelling task (paper-code/tasks/language_modeling/__init__.py:27-325).

Truncated back-propagation through time over a token stream: the global batch is
`batch_size x n_workers` columns, every rank takes its own column slice, the hidden state is
carried from window to window and detached, and gradients are clipped to norm 0.4 before they
are handed to the reducer. The corpus is a synthetic Zipf(s = 1) token stream over a
33 278-word vocabulary (WikiText-2's size) — the tokenizer / download stack of the original
(torchtext, spaCy) is not needed for that and is not a dependency.
"""
from __future__ import annotations

from copy import deepcopy
from typing import Dict, Iterable, List

import torch

from ...models.lstm import RNNModel
from ...utils import MeanAccumulator
from .utils import _world, zipf_tokens


class Batch:
    def __init__(self, x, y, hidden):
        self.x, self.y, self.hidden = x, y, hidden


class BPTTStream:
    """[steps, global_batch] token matrix cut into windows of `bptt_len` (+1 shifted targets)."""

    def __init__(self, tokens: torch.Tensor, global_batch: int, bptt_len: int):
        steps = tokens.numel() // global_batch
        self.data = tokens[: steps * global_batch].view(global_batch, steps).t().contiguous()
        self.bptt_len = bptt_len

    def __len__(self) -> int:
        return max((self.data.shape[0] - 1) // self.bptt_len, 0)

    def __iter__(self):
        for i in range(len(self)):
            lo = i * self.bptt_len
            yield self.data[lo : lo + self.bptt_len], self.data[lo + 1 : lo + 1 + self.bptt_len]


class SplitBatchLoader:
    """Gives each rank its column slice of the global batch and a detached hidden state."""

    def __init__(self, stream, device, rank, batch_size, model, hidden_container):
        self._stream, self._device, self._rank, self._batch_size = stream, device, rank, batch_size
        self._model, self._hidden_container = model, hidden_container

    def __len__(self):
        return len(self._stream)

    def __iter__(self):
        lo, hi = self._rank * self._batch_size, (self._rank + 1) * self._batch_size
        for text, target in self._stream:
            hidden = self._model.repackage_hidden(self._hidden_container["hidden"])
            yield Batch(text[:, lo:hi].to(self._device), target[:, lo:hi].to(self._device), hidden)


class LanguageModelingTask:
    def __init__(self, device, timer, seed: int, batch_size: int, vocab: int = 33278, train_tokens: int = 2_000_000,
                 valid_tokens: int = 200_000, bptt_len: int = 30, hidden: int = 650, layers: int = 3, dropout: float = 0.4):
        self._device, self._timer, self._seed, self._batch_size = device, timer, seed, batch_size
        self._epoch = 0
        workers, _ = _world()
        self._vocab = vocab
        self._train = BPTTStream(zipf_tokens(train_tokens, vocab, seed=11), batch_size * workers, bptt_len)
        self._valid = BPTTStream(zipf_tokens(valid_tokens, vocab, seed=12), batch_size * workers, bptt_len)
        torch.random.manual_seed(seed)
        self._model = RNNModel("LSTM", vocab, hidden, hidden, layers, dropout=dropout, tie_weights=True).to(device).train()
        self._criterion = torch.nn.CrossEntropyLoss().to(device)
        self._hidden_container = {"hidden": None}

    @property
    def state(self) -> List[torch.Tensor]:
        return list(self._model.parameters())

    @property
    def buffers(self) -> List[torch.Tensor]:
        return list(self._model.buffers())

    @property
    def parameter_names(self) -> List[str]:
        return [name for name, _ in self._model.named_parameters()]

    def _loader(self, stream, batch_size):
        _, rank = _world()
        self._hidden_container["hidden"] = self._model.init_hidden(batch_size)
        return SplitBatchLoader(stream, self._device, rank, batch_size, self._model, self._hidden_container)

    def train_iterator(self, batch_size: int) -> Iterable[Batch]:
        self._epoch += 1
        return self._loader(self._train, batch_size)

    def _forward(self, batch: Batch):
        prediction, hidden = self._model(batch.x, batch.hidden)
        self._hidden_container["hidden"] = hidden
        return prediction, self._criterion(prediction.view(-1, self._vocab), batch.y.reshape(-1))

    def batch_loss(self, batch: Batch):
        with torch.no_grad():
            with self._timer("batch.forward", float(self._epoch)):
                prediction, loss = self._forward(batch)
            with self._timer("batch.evaluate", float(self._epoch)):
                metrics = self.evaluate_prediction(prediction, batch.y)
        return loss.item(), metrics

    def batch_loss_and_gradient(self, batch: Batch, rnn_clip: float = 0.4):
        self._model.zero_grad()
        with self._timer("batch.forward", float(self._epoch)):
            prediction, loss = self._forward(batch)
        with self._timer("batch.backward", float(self._epoch)):
            loss.backward()
        with self._timer("batch.evaluate", float(self._epoch)):
            metrics = self.evaluate_prediction(prediction, batch.y)
        torch.nn.utils.clip_grad_norm_(self._model.parameters(), rnn_clip)
        return loss.detach(), [p.grad for p in self._model.parameters()], metrics

    def evaluate_prediction(self, output, target) -> Dict[str, torch.Tensor]:
        with torch.no_grad():
            ce = self._criterion(output.view(-1, self._vocab), target.reshape(-1))
            return {"cross_entropy": ce.detach(), "perplexity": torch.exp(ce).detach()}

    def test(self, state_dict=None):
        model = self._model
        if state_dict:
            model = deepcopy(self._model)
            model.load_state_dict(state_dict)
        model.eval()
        mean = MeanAccumulator()
        for batch in self._loader(self._valid, self._batch_size):
            with torch.no_grad():
                prediction, hidden = model(batch.x, batch.hidden)
                self._hidden_container["hidden"] = hidden
                mean.add(self.evaluate_prediction(prediction, batch.y))
        mean.reduce()
        self._model.train()
        return mean.value()

    def state_dict(self):
        return self._model.state_dict()
