"""Recurrent layers (ferrum-nn/src/rnn.rs:9-504): RNNCell / LSTMCell / GRUCell and the sequence modules.

Input is sequence-first ``[T, B, F]``.  The reference executes only layer 0 in the forward direction and computes
the LSTM / GRU gates on host vectors without autograd; here every layer runs, the per-step projections are GEMMs
of this package (the input projection of a whole sequence is one GEMM), the gate arithmetic of an LSTM / GRU step
is one fused kernel forward and one backward, and everything is differentiable.
"""
from __future__ import annotations

import enum
import math

import torch

from ..core import ShapeMismatch, Tensor, _as_device, _unwrap
from ..ops import functional as F
from .modules import Module, _param, _wrap_out


class Nonlinearity(enum.Enum):
    Tanh = "tanh"
    ReLU = "relu"


def _uniform(shape, k, dev):
    return _param(torch.empty(*shape, device=dev).uniform_(-k, k))


class _CellBase(Module):
    gates = 1

    def __init__(self, input_size, hidden_size, bias=True, device=None):
        super().__init__()
        self.input_size, self._hidden = int(input_size), int(hidden_size)
        dev = _as_device(device).to_torch()
        k = 1.0 / math.sqrt(hidden_size)
        g = self.gates
        self.weight_ih = _uniform((g * hidden_size, input_size), k, dev)
        self.weight_hh = _uniform((g * hidden_size, hidden_size), k, dev)
        if bias:
            self.bias_ih = _uniform((g * hidden_size,), k, dev)
            self.bias_hh = _uniform((g * hidden_size,), k, dev)
        else:
            self.register_parameter("bias_ih", None)
            self.register_parameter("bias_hh", None)

    @classmethod
    def new(cls, input_size, hidden_size):
        return cls(input_size, hidden_size)

    @classmethod
    def with_bias(cls, input_size, hidden_size, bias):
        return cls(input_size, hidden_size, bias)

    def hidden_size(self) -> int:
        return self._hidden

    def _check(self, x):
        if x.shape[-1] != self.input_size:
            raise ShapeMismatch(type(self).__name__, f"[B, {self.input_size}]", list(x.shape))

    def input_projection(self, x):
        return F.linear(x, self.weight_ih, self.bias_ih)


def _chunks(t, n):
    h = t.shape[-1] // n
    return [t[..., i * h:(i + 1) * h] for i in range(n)]


class RNNCell(_CellBase):
    gates = 1

    def __init__(self, input_size, hidden_size, bias=True, nonlinearity=Nonlinearity.Tanh, device=None):
        super().__init__(input_size, hidden_size, bias, device)
        self.nonlinearity = nonlinearity

    @classmethod
    def with_config(cls, input_size, hidden_size, bias, nonlinearity):
        return cls(input_size, hidden_size, bias, nonlinearity)

    def step(self, xi, h):
        pre = F.binary(xi, F.linear(h, self.weight_hh, self.bias_hh), "add")
        return F.unary(pre, self.nonlinearity.value)

    def forward(self, input, hidden):
        wrapped = isinstance(input, Tensor)
        x, h = _unwrap(input), _unwrap(hidden)
        self._check(x)
        return _wrap_out(self.step(self.input_projection(x), h), wrapped)


class LSTMCell(_CellBase):
    gates = 4  # input, forget, cell, output

    def step(self, xi, h, c):
        # hidden projection (GEMM) + one fused gate kernel
        return F.lstm_gates(xi, F.linear(h, self.weight_hh, self.bias_hh), c)

    def forward(self, input, hx):
        wrapped = isinstance(input, Tensor)
        x, h, c = _unwrap(input), _unwrap(hx[0]), _unwrap(hx[1])
        self._check(x)
        return _wrap_out(self.step(self.input_projection(x), h, c), wrapped)


class GRUCell(_CellBase):
    gates = 3  # reset, update, new

    def step(self, xi, h):
        # h' = (1 - z) * n + z * h, n = tanh(xn + r * hn): hidden projection (GEMM) + one fused gate kernel
        return F.gru_gates(xi, F.linear(h, self.weight_hh, self.bias_hh), h)

    def forward(self, input, hidden):
        wrapped = isinstance(input, Tensor)
        x, h = _unwrap(input), _unwrap(hidden)
        self._check(x)
        return _wrap_out(self.step(self.input_projection(x), h), wrapped)


class _SeqBase(Module):
    cell_cls = RNNCell

    def __init__(self, input_size, hidden_size, num_layers=1, bias=True, device=None, **cell_kw):
        super().__init__()
        self.input_size, self._hidden, self.num_layers = int(input_size), int(hidden_size), int(num_layers)
        self.cells = torch.nn.ModuleList(
            [self.cell_cls(input_size if l == 0 else hidden_size, hidden_size, bias, device=device, **cell_kw)
             for l in range(num_layers)])

    @classmethod
    def new(cls, input_size, hidden_size, num_layers):
        return cls(input_size, hidden_size, num_layers)

    def hidden_size(self) -> int:
        return self._hidden

    def _zeros(self, x):
        return torch.zeros(self.num_layers, x.shape[1], self._hidden, device=x.device, dtype=x.dtype)

    def _check(self, x):
        if x.dim() != 3 or x.shape[2] != self.input_size:
            raise ShapeMismatch(type(self).__name__, f"[T, B, {self.input_size}]", list(x.shape))


class RNN(_SeqBase):
    cell_cls = RNNCell

    @classmethod
    def with_config(cls, input_size, hidden_size, num_layers, bias=True, nonlinearity=Nonlinearity.Tanh):
        return cls(input_size, hidden_size, num_layers, bias, nonlinearity=nonlinearity)

    def forward_seq(self, input, h_0=None):
        """``[T, B, F]`` -> (``[T, B, H]`` outputs of the last layer, ``[layers, B, H]`` final hidden states)."""
        wrapped = isinstance(input, Tensor)
        x = _unwrap(input)
        self._check(x)
        h0 = _unwrap(h_0) if h_0 is not None else self._zeros(x)
        finals, layer_in = [], x
        for l, cell in enumerate(self.cells):
            proj = cell.input_projection(layer_in)  # one GEMM for the whole sequence
            h, outs = h0[l], []
            for t in range(x.shape[0]):
                h = cell.step(proj[t], h)
                outs.append(h)
            layer_in = torch.stack(outs, 0)
            finals.append(h)
        return _wrap_out((layer_in, torch.stack(finals, 0)), wrapped)

    def forward(self, input):
        out = self.forward_seq(input)
        return out[0]


class GRU(RNN):
    cell_cls = GRUCell

    @classmethod
    def with_config(cls, input_size, hidden_size, num_layers, bias=True):
        return cls(input_size, hidden_size, num_layers, bias)


class LSTM(_SeqBase):
    cell_cls = LSTMCell

    @classmethod
    def with_config(cls, input_size, hidden_size, num_layers, bias=True):
        return cls(input_size, hidden_size, num_layers, bias)

    def forward_seq(self, input, hx=None):
        wrapped = isinstance(input, Tensor)
        x = _unwrap(input)
        self._check(x)
        h0 = _unwrap(hx[0]) if hx is not None else self._zeros(x)
        c0 = _unwrap(hx[1]) if hx is not None else self._zeros(x)
        hs, cs, layer_in = [], [], x
        for l, cell in enumerate(self.cells):
            proj = cell.input_projection(layer_in)
            h, c, outs = h0[l], c0[l], []
            for t in range(x.shape[0]):
                h, c = cell.step(proj[t], h, c)
                outs.append(h)
            layer_in = torch.stack(outs, 0)
            hs.append(h)
            cs.append(c)
        return _wrap_out((layer_in, (torch.stack(hs, 0), torch.stack(cs, 0))), wrapped)

    def forward(self, input):
        return self.forward_seq(input)[0]
