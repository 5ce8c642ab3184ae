"""Word-level recurrent language model: embedding -> multi-layer LSTM/GRU/RNN -> decoder whose
weight can be tied to the embedding.

Architecture and initialisation parity with paper-code/tasks/language_modeling/model.py:9-75
(`encoder`, `rnn`, `decoder` parameter names; uniform(-0.1, 0.1) embedding / decoder weights,
zero decoder bias). The benchmark configuration is 3 x LSTM(650), dropout 0.4, tied weights,
vocabulary 33 278 (language_modeling/__init__.py:277-301).
"""
from __future__ import annotations

import torch
import torch.nn as nn


class RNNModel(nn.Module):
    def __init__(self, rnn_type: str, ntoken: int, ninp: int, nhid: int, nlayers: int, dropout: float = 0.5,
                 tie_weights: bool = False):
        super().__init__()
        self.drop = nn.Dropout(dropout)
        self.encoder = nn.Embedding(ntoken, ninp)
        if rnn_type in ("LSTM", "GRU"):
            self.rnn = getattr(nn, rnn_type)(ninp, nhid, nlayers, dropout=dropout)
        elif rnn_type in ("RNN_TANH", "RNN_RELU"):
            self.rnn = nn.RNN(ninp, nhid, nlayers, nonlinearity=rnn_type.split("_")[1].lower(), dropout=dropout)
        else:
            raise ValueError("rnn_type must be one of LSTM, GRU, RNN_TANH, RNN_RELU")
        self.decoder = nn.Linear(nhid, ntoken)
        if tie_weights:
            if nhid != ninp:
                raise ValueError("tied weights need nhid == ninp")
            self.decoder.weight = self.encoder.weight
        self.rnn_type, self.nhid, self.nlayers, self.ntokens = rnn_type, nhid, nlayers, ntoken
        self.init_weights()

    def init_weights(self, initrange: float = 0.1) -> None:
        with torch.no_grad():
            self.encoder.weight.uniform_(-initrange, initrange)
            self.decoder.bias.zero_()
            self.decoder.weight.uniform_(-initrange, initrange)

    def forward(self, tokens: torch.Tensor, hidden):
        emb = self.drop(self.encoder(tokens))
        output, hidden = self.rnn(emb, hidden)
        output = self.drop(output)
        steps, batch, width = output.shape
        decoded = self.decoder(output.reshape(steps * batch, width))
        return decoded.view(steps, batch, -1), hidden

    def init_hidden(self, bsz: int):
        ref = next(self.parameters())
        zeros = lambda: ref.new_zeros(self.nlayers, bsz, self.nhid)  # noqa: E731
        return (zeros(), zeros()) if self.rnn_type == "LSTM" else zeros()

    def repackage_hidden(self, h):
        """Cut the graph: carried hidden state becomes a constant for the next BPTT window."""
        if isinstance(h, torch.Tensor):
            return h.detach()
        return tuple(self.repackage_hidden(v) for v in h)


def wikitext2_lstm(ntoken: int = 33278) -> RNNModel:
    """The paper's language-model configuration."""
    return RNNModel("LSTM", ntoken, 650, 650, 3, dropout=0.4, tie_weights=True)
