"""LSTM / GRU (ghostflow-nn/src/rnn.rs): ``LSTM(input, hidden, num_layers, bidirectional, dropout)`` with the
fused ``[4*hidden]`` gate projection in the order i, f, g, o (rnn.rs:73-78). Unlike the reference, which shares
one cell across all "layers" (rnn.rs:142-149), every layer and direction has its own weights."""
from __future__ import annotations

import torch

from .layers import Dropout, Linear
from .module import Module, ModuleList


class LSTMCell(Module):
    def __init__(self, input_size: int, hidden_size: int, bias: bool = True):
        super().__init__()
        self.input_size, self.hidden_size = input_size, hidden_size
        self.ih = Linear(input_size, 4 * hidden_size, bias)
        self.hh = Linear(hidden_size, 4 * hidden_size, bias)

    def forward(self, x, state=None):
        B = x.shape[0]
        if state is None:
            z = x.new_zeros(B, self.hidden_size)
            state = (z, z)
        h, c = state
        i, f, g, o = (self.ih(x) + self.hh(h)).chunk(4, dim=-1)
        c = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        h = torch.sigmoid(o) * torch.tanh(c)
        return h, c


class GRUCell(Module):
    def __init__(self, input_size: int, hidden_size: int, bias: bool = True):
        super().__init__()
        self.input_size, self.hidden_size = input_size, hidden_size
        self.ih = Linear(input_size, 3 * hidden_size, bias)
        self.hh = Linear(hidden_size, 3 * hidden_size, bias)

    def forward(self, x, h=None):
        if h is None:
            h = x.new_zeros(x.shape[0], self.hidden_size)
        ir, iz, in_ = self.ih(x).chunk(3, -1)
        hr, hz, hn = self.hh(h).chunk(3, -1)
        r = torch.sigmoid(ir + hr)
        z = torch.sigmoid(iz + hz)
        n = torch.tanh(in_ + r * hn)
        return (1 - z) * n + z * h


class _Recurrent(Module):
    cell_cls = LSTMCell

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bidirectional: bool = False,
                 dropout: float = 0.0):
        super().__init__()
        self.input_size, self.hidden_size, self.num_layers = input_size, hidden_size, num_layers
        self.bidirectional = bidirectional
        dirs = 2 if bidirectional else 1
        self.cells = ModuleList()
        for layer in range(num_layers):
            inp = input_size if layer == 0 else hidden_size * dirs
            for _ in range(dirs):
                self.cells.append(self.cell_cls(inp, hidden_size))
        self.drop = Dropout(dropout)

    def _run(self, cell, x, reverse):
        """x: [B, S, F] -> outputs [B, S, H], final state."""
        S = x.shape[1]
        state = None
        outs = [None] * S
        steps = range(S - 1, -1, -1) if reverse else range(S)
        for t in steps:
            state = cell(x[:, t], state)
            outs[t] = state[0] if isinstance(state, tuple) else state
        return torch.stack(outs, dim=1), state

    def forward(self, x):
        """x: ``[B, S, input_size]``. Returns ``(outputs [B, S, H*dirs], final_states per layer/direction)``."""
        dirs = 2 if self.bidirectional else 1
        finals = []
        for layer in range(self.num_layers):
            outs = []
            for d in range(dirs):
                o, st = self._run(self.cells[layer * dirs + d], x, reverse=(d == 1))
                outs.append(o)
                finals.append(st)
            x = torch.cat(outs, dim=-1) if dirs == 2 else outs[0]
            if layer + 1 < self.num_layers:
                x = self.drop(x)
        return x, finals


class LSTM(_Recurrent):
    cell_cls = LSTMCell


class GRU(_Recurrent):
    cell_cls = GRUCell
