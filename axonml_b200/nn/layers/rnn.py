"""Recurrent layers (crates/axonml-nn/src/layers/rnn.rs): RNNCell / LSTMCell / GRUCell with
``weight_ih[G*H, in]``, ``weight_hh[G*H, H]`` (xavier-uniform), zero ``bias_ih``/``bias_hh``;
LSTM gate order i,f,g,o; GRU gate order r,z,n with ``n = tanh(ih_n + r * hh_n)``.  RNN / LSTM /
GRU stack cells, default ``batch_first=True``, zero initial state, and return the top layer's
hidden state for every time step.  The gate GEMMs go through ``ops.linear`` (tcgen05 on B200)."""
from __future__ import annotations

import torch

from ...ops.linear import linear as _linear
from .. import init
from ..module import Module, ModuleList, Parameter


class _Cell(Module):
    GATES = 1

    def __init__(self, input_size: int, hidden_size: int):
        super().__init__()
        self.input_size, self.hidden_size = input_size, hidden_size
        G = self.GATES
        self.weight_ih = Parameter(init.xavier_uniform(input_size, G * hidden_size))
        self.weight_hh = Parameter(init.xavier_uniform(hidden_size, G * hidden_size))
        self.bias_ih = Parameter(torch.zeros(G * hidden_size))
        self.bias_hh = Parameter(torch.zeros(G * hidden_size))

    @classmethod
    def new(cls, input_size, hidden_size): return cls(input_size, hidden_size)

    def _gates(self, x, h):
        return _linear(x, self.weight_ih, self.bias_ih), _linear(h, self.weight_hh, self.bias_hh)

    def forward_step(self, input, hidden):
        """One time step with an explicit previous state (rnn.rs ``forward_step``): a tensor for
        RNN / GRU cells, an ``(h, c)`` pair for the LSTM cell.  The feature size is checked."""
        if input.shape[-1] != self.input_size:
            raise ValueError(f"{type(self).__name__}: expected input size {self.input_size}, got {input.shape[-1]}")
        return self.forward(input, hidden)


class RNNCell(_Cell):
    GATES = 1

    def forward(self, x, h=None):
        if h is None:
            h = x.new_zeros(x.shape[0], self.hidden_size)
        gi, gh = self._gates(x, h)
        return torch.tanh(gi + gh)


class LSTMCell(_Cell):
    GATES = 4

    def forward(self, x, state=None):
        if state is None:
            z = x.new_zeros(x.shape[0], self.hidden_size)
            state = (z, z)
        h, c = state
        gi, gh = self._gates(x, h)
        i, f, g, o = (gi + gh).chunk(4, dim=-1)
        c2 = torch.sigmoid(f) * c + torch.sigmoid(i) * torch.tanh(g)
        h2 = torch.sigmoid(o) * torch.tanh(c2)
        return h2, c2


class GRUCell(_Cell):
    GATES = 3

    def forward(self, x, h=None):
        if h is None:
            h = x.new_zeros(x.shape[0], self.hidden_size)
        gi, gh = self._gates(x, h)
        ir, iz, inn = gi.chunk(3, dim=-1)
        hr, hz, hn = gh.chunk(3, dim=-1)
        r = torch.sigmoid(ir + hr)
        z = torch.sigmoid(iz + hz)
        n = torch.tanh(inn + r * hn)
        return (1 - z) * n + z * h


class _Recurrent(Module):
    CELL = RNNCell

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1,
                 batch_first: bool = True):
        super().__init__()
        self.input_size, self.hidden_size = input_size, hidden_size
        self.num_layers, self.batch_first = num_layers, batch_first
        self.cells = ModuleList([self.CELL(input_size if i == 0 else hidden_size, hidden_size)
                                 for i in range(num_layers)])

    @classmethod
    def new(cls, input_size, hidden_size, num_layers=1): return cls(input_size, hidden_size, num_layers)

    @classmethod
    def with_options(cls, input_size, hidden_size, num_layers, batch_first):
        return cls(input_size, hidden_size, num_layers, batch_first)

    def _step(self, cell, x, state):
        h = cell(x, state)
        return h, h

    SEQ_KIND = 0          # 4 = LSTM, 3 = GRU: cell types the whole-sequence kernel implements

    def _fused_sequence(self, x, state):
        """Inference on a B200 with H <= 128: one GEMM for all input projections of a layer, then
        one kernel for the whole sequence (csrc/kernels/rnn_seq.cu).  Returns None when the
        step-by-step path has to run (training, other devices, larger H, fp32 modules)."""
        from ... import _native as N
        if (self.SEQ_KIND == 0 or torch.is_grad_enabled() or not x.is_cuda or x.dtype != torch.bfloat16
                or self.hidden_size > 128 or not N.is_blackwell() or x.shape[1] == 0):
            return None
        if any(c.weight_hh.dtype != torch.bfloat16 for c in self.cells):
            return None
        B, T, _ = x.shape
        H, G = self.hidden_size, self.SEQ_KIND
        inp = x.contiguous()
        states = []
        for li, cell in enumerate(self.cells):
            xproj = _linear(inp.reshape(B * T, -1), cell.weight_ih, cell.bias_ih).float().contiguous()
            st = state[li] if state is not None else None
            h0 = c0 = None
            if st is not None:
                h0, c0 = (st if G == 4 else (st, None))
                h0 = h0.float().contiguous()
                c0 = c0.float().contiguous() if c0 is not None else None
            out = torch.empty((B, T, H), dtype=torch.bfloat16, device=x.device)
            h_last = torch.empty((B, H), dtype=torch.float32, device=x.device)
            c_last = torch.empty((B, H), dtype=torch.float32, device=x.device) if G == 4 else None
            rc = N.cuda().ax_rnn_seq_fwd(G, N.ptr(xproj), N.ptr(cell.weight_hh.detach().contiguous()),
                                         N.ptr(cell.bias_hh.detach().float().contiguous()), N.ptr(h0), N.ptr(c0), N.ptr(out), 1,
                                         N.ptr(h_last), N.ptr(c_last), B, T, H, N.stream_ptr())
            N.check(rc, "ax_rnn_seq_fwd")
            hl = h_last.to(x.dtype)
            states.append((hl, c_last.to(x.dtype)) if G == 4 else hl)
            inp = out
        self.last_state = states
        return inp

    def forward(self, x, state=None):
        if not self.batch_first:
            x = x.transpose(0, 1)
        fused = self._fused_sequence(x, state)
        if fused is not None:
            return fused if self.batch_first else fused.transpose(0, 1)
        B, T, _ = x.shape
        states = list(state) if state is not None else [None] * self.num_layers
        outs = []
        for t in range(T):
            inp = x[:, t]
            for li, cell in enumerate(self.cells):
                inp, states[li] = self._step(cell, inp, states[li])
            outs.append(inp)
        out = torch.stack(outs, dim=1)
        self.last_state = states
        return out if self.batch_first else out.transpose(0, 1)

    def forward_last(self, x):
        out = self.forward(x)
        return out[:, -1] if self.batch_first else out[-1]

    def forward_mean(self, x):
        out = self.forward(x)
        return out.mean(1 if self.batch_first else 0)


class RNN(_Recurrent):
    CELL = RNNCell


class GRU(_Recurrent):
    CELL = GRUCell
    SEQ_KIND = 3


class LSTM(_Recurrent):
    CELL = LSTMCell
    SEQ_KIND = 4

    def _step(self, cell, x, state):
        h, c = cell(x, state)
        return h, (h, c)
