"""Recurrent layers and packed sequences (ferrotorch-nn/src/rnn.rs:60-1700, rnn_utils.rs).

The input projections of a whole sequence are one GEMM per layer and direction; each step then adds the hidden projection and applies
the gate math. CUDA f32 steps of LSTM and GRU use this package's fused cell kernels (forward and backward in one launch each)."""
from __future__ import annotations

import math
from typing import List, NamedTuple, Optional, Sequence, Tuple, Union

import torch

from .. import ops
from ..errors import InvalidArgument, ShapeMismatch
from .module import Module, Parameter


# -- packed sequences -------------------------------------------------------------------------------------------------------------------
class PackedSequence(NamedTuple):
    """Time-major concatenation of the valid steps of a batch of sequences sorted by decreasing length. ``batch_sizes[t]`` sequences are
    still running at step ``t``; ``sorted_indices`` maps sorted position -> original batch index, ``unsorted_indices`` the inverse."""
    data: torch.Tensor
    batch_sizes: torch.Tensor
    sorted_indices: Optional[torch.Tensor] = None
    unsorted_indices: Optional[torch.Tensor] = None

    def to(self, *a, **k) -> "PackedSequence":
        return self._replace(data=self.data.to(*a, **k))


def _invert(perm: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(perm.numel(), device=perm.device)
    return inv


def pack_padded_sequence(x: torch.Tensor, lengths, batch_first: bool = False, enforce_sorted: bool = True) -> PackedSequence:
    lengths = torch.as_tensor(lengths, dtype=torch.long).cpu()
    if batch_first:
        x = x.transpose(0, 1)
    T, B = x.shape[:2]
    if lengths.numel() != B:
        raise ShapeMismatch(f"pack_padded_sequence: {lengths.numel()} lengths for a batch of {B}")
    if int(lengths.min()) <= 0 or int(lengths.max()) > T:
        raise InvalidArgument("pack_padded_sequence: every length must lie in [1, T]")
    if enforce_sorted:
        if bool((lengths[1:] > lengths[:-1]).any()):
            raise InvalidArgument("pack_padded_sequence: lengths must be sorted in decreasing order when enforce_sorted is set")
        order, sorted_idx, unsorted_idx = None, None, None
        ls = lengths
    else:
        ls, order = torch.sort(lengths, descending=True, stable=True)
        sorted_idx = order.to(x.device)
        unsorted_idx = _invert(sorted_idx)
        x = x.index_select(1, sorted_idx)
    steps = int(ls[0])
    batch_sizes = torch.tensor([int((ls > t).sum()) for t in range(steps)], dtype=torch.long)
    data = torch.cat([x[t, : int(batch_sizes[t])] for t in range(steps)], 0)
    return PackedSequence(data, batch_sizes, sorted_idx, unsorted_idx)


def pad_packed_sequence(seq, batch_first: bool = False, padding_value: float = 0.0, total_length: Optional[int] = None):
    data, bs = seq.data, seq.batch_sizes
    T, B = bs.numel(), int(bs[0])
    if total_length is not None:
        if total_length < T:
            raise InvalidArgument(f"total_length {total_length} is shorter than the longest sequence {T}")
        T_out = total_length
    else:
        T_out = T
    out = data.new_full((T_out, B, *data.shape[1:]), padding_value)
    off = 0
    rows = []
    for t in range(T):
        n = int(bs[t])
        rows.append((t, n, off))
        off += n
    # one scatter instead of T slice writes keeps the autograd graph small
    t_idx = torch.cat([torch.full((n,), t, dtype=torch.long) for t, n, _ in rows]).to(data.device)
    b_idx = torch.cat([torch.arange(n) for _, n, _ in rows]).to(data.device)
    out = out.index_put((t_idx, b_idx), data)
    lengths = torch.tensor([int((bs > b).sum()) for b in range(B)], dtype=torch.long)
    if seq.unsorted_indices is not None:
        out = out.index_select(1, seq.unsorted_indices)
        lengths = lengths[seq.unsorted_indices.cpu()]
    return (out.transpose(0, 1) if batch_first else out), lengths


def pad_sequence(sequences: Sequence[torch.Tensor], batch_first: bool = False, padding_value: float = 0.0) -> torch.Tensor:
    if not sequences:
        raise InvalidArgument("pad_sequence: empty list")
    T = max(s.shape[0] for s in sequences)
    tail = sequences[0].shape[1:]
    cols = []
    for s in sequences:
        if s.shape[1:] != tail:
            raise ShapeMismatch("pad_sequence: trailing dimensions differ")
        cols.append(s if s.shape[0] == T else torch.cat([s, s.new_full((T - s.shape[0], *tail), padding_value)], 0))
    out = torch.stack(cols, 1)
    return out.transpose(0, 1) if batch_first else out


def pack_sequence(sequences: Sequence[torch.Tensor], enforce_sorted: bool = True) -> PackedSequence:
    return pack_padded_sequence(pad_sequence(sequences), [s.shape[0] for s in sequences], enforce_sorted=enforce_sorted)


def _is_packed(x) -> bool:
    return isinstance(x, (PackedSequence, torch.nn.utils.rnn.PackedSequence))


# -- gate math ---------------------------------------------------------------------------------------------------------------------------
def _sig(x):
    return 1.0 / (1.0 + torch.exp(-x))


def lstm_pointwise(gates: torch.Tensor, c_prev: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``gates`` ``[B, 4H]`` in (input, forget, cell, output) order."""
    if gates.is_cuda and gates.dtype == torch.float32 and gates.dim() == 2:
        return ops.nn_ops.lstm_cell(gates.contiguous(), c_prev.contiguous())
    i, f, g, o = gates.chunk(4, -1)
    c = _sig(f) * c_prev + _sig(i) * torch.tanh(g)
    return _sig(o) * torch.tanh(c), c


def gru_pointwise(gi: torch.Tensor, gh: torch.Tensor, h_prev: torch.Tensor) -> torch.Tensor:
    """``gi``/``gh`` ``[B, 3H]`` in (reset, update, new) order; the reset gate multiplies the hidden half of the candidate."""
    if gi.is_cuda and gi.dtype == torch.float32 and gi.dim() == 2:
        return ops.nn_ops.gru_cell(gi.contiguous(), gh.contiguous(), h_prev.contiguous())
    ir, iz, in_ = gi.chunk(3, -1)
    hr, hz, hn = gh.chunk(3, -1)
    r, z = _sig(ir + hr), _sig(iz + hz)
    n = torch.tanh(in_ + r * hn)
    return (1 - z) * n + z * h_prev


def _lin(x, w, b):
    y = x @ w.t()
    return y if b is None else y + b


# -- cells ---------------------------------------------------------------------------------------------------------------------------------
class _CellBase(Module):
    _gates = 1

    def __init__(self, input_size: int, hidden_size: int, bias: bool = True, device=None, dtype=None):
        super().__init__()
        if input_size <= 0 or hidden_size <= 0:
            raise InvalidArgument("input_size and hidden_size must be positive")
        self.input_size, self.hidden_size, self.bias = input_size, hidden_size, bias
        g = self._gates * hidden_size
        self.weight_ih = Parameter(torch.empty(g, input_size, device=device, dtype=dtype))
        self.weight_hh = Parameter(torch.empty(g, hidden_size, device=device, dtype=dtype))
        if bias:
            self.bias_ih = Parameter(torch.empty(g, device=device, dtype=dtype))
            self.bias_hh = Parameter(torch.empty(g, device=device, dtype=dtype))
        else:
            self.register_parameter("bias_ih", None)
            self.register_parameter("bias_hh", None)
        self.reset_parameters()

    def reset_parameters(self) -> None:
        k = 1.0 / math.sqrt(self.hidden_size)
        with torch.no_grad():
            for p in self.parameters():
                p.uniform_(-k, k)

    def _prep(self, x, h):
        unb = x.dim() == 1
        if x.dim() not in (1, 2) or x.shape[-1] != self.input_size:
            raise ShapeMismatch(f"{type(self).__name__}: expected [B, {self.input_size}] or [{self.input_size}], got {list(x.shape)}")
        if unb:
            x = x.unsqueeze(0)
        return x, unb


class RNNCell(_CellBase):
    _gates = 1

    def __init__(self, input_size: int, hidden_size: int, bias: bool = True, nonlinearity: str = "tanh", device=None, dtype=None):
        nonlinearity = getattr(nonlinearity, "value", nonlinearity)
        if nonlinearity not in ("tanh", "relu"):
            raise InvalidArgument(f"unknown nonlinearity {nonlinearity!r}")
        self.nonlinearity = nonlinearity
        super().__init__(input_size, hidden_size, bias, device, dtype)

    def forward(self, x, h=None):
        x, unb = self._prep(x, h)
        h = x.new_zeros(x.shape[0], self.hidden_size) if h is None else (h.unsqueeze(0) if unb else h)
        pre = _lin(x, self.weight_ih, self.bias_ih) + _lin(h, self.weight_hh, self.bias_hh)
        out = torch.tanh(pre) if self.nonlinearity == "tanh" else torch.clamp_min(pre, 0)
        return out.squeeze(0) if unb else out


class LSTMCell(_CellBase):
    _gates = 4

    def forward(self, x, state=None):
        x, unb = self._prep(x, state)
        if state is None:
            h = c = x.new_zeros(x.shape[0], self.hidden_size)
        else:
            h, c = (s.unsqueeze(0) if unb else s for s in state)
        h, c = lstm_pointwise(_lin(x, self.weight_ih, self.bias_ih) + _lin(h, self.weight_hh, self.bias_hh), c)
        return (h.squeeze(0), c.squeeze(0)) if unb else (h, c)


class GRUCell(_CellBase):
    _gates = 3

    def forward(self, x, h=None):
        x, unb = self._prep(x, h)
        h = x.new_zeros(x.shape[0], self.hidden_size) if h is None else (h.unsqueeze(0) if unb else h)
        out = gru_pointwise(_lin(x, self.weight_ih, self.bias_ih), _lin(h, self.weight_hh, self.bias_hh), h)
        return out.squeeze(0) if unb else out


# -- multi-layer sequence modules ----------------------------------------------------------------------------------------------------------
class _RNNBase(Module):
    _gates = 1
    _mode = "rnn"

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, bias: bool = True, batch_first: bool = False, dropout: float = 0.0,
                 bidirectional: bool = False, proj_size: int = 0, device=None, dtype=None):
        super().__init__()
        if input_size <= 0 or hidden_size <= 0 or num_layers <= 0:
            raise InvalidArgument("input_size, hidden_size and num_layers must be positive")
        if not 0.0 <= dropout <= 1.0:
            raise InvalidArgument("dropout must lie in [0, 1]")
        if proj_size:
            raise InvalidArgument("projected LSTM states (proj_size > 0) are not provided")
        self.input_size, self.hidden_size, self.num_layers, self.bias = input_size, hidden_size, num_layers, bias
        self.batch_first, self.dropout, self.bidirectional, self.proj_size = batch_first, float(dropout), bidirectional, 0
        D = 2 if bidirectional else 1
        g = self._gates * hidden_size
        for layer in range(num_layers):
            for d in range(D):
                sfx = f"_l{layer}" + ("_reverse" if d else "")
                in_sz = input_size if layer == 0 else hidden_size * D
                setattr(self, "weight_ih" + sfx, Parameter(torch.empty(g, in_sz, device=device, dtype=dtype)))
                setattr(self, "weight_hh" + sfx, Parameter(torch.empty(g, hidden_size, device=device, dtype=dtype)))
                if bias:
                    setattr(self, "bias_ih" + sfx, Parameter(torch.empty(g, device=device, dtype=dtype)))
                    setattr(self, "bias_hh" + sfx, Parameter(torch.empty(g, device=device, dtype=dtype)))
        self.reset_parameters()

    def reset_parameters(self) -> None:
        k = 1.0 / math.sqrt(self.hidden_size)
        with torch.no_grad():
            for p in self.parameters():
                p.uniform_(-k, k)

    def flatten_parameters(self) -> None:
        """Kept for source compatibility: the weights are used where they are."""

    def _w(self, layer: int, d: int):
        sfx = f"_l{layer}" + ("_reverse" if d else "")
        return (getattr(self, "weight_ih" + sfx), getattr(self, "weight_hh" + sfx),
                getattr(self, "bias_ih" + sfx) if self.bias else None, getattr(self, "bias_hh" + sfx) if self.bias else None)

    # one step of this module's cell given the precomputed input projection
    def _step(self, gi, h, c, w_hh, b_hh):
        raise NotImplementedError

    def _run_direction(self, x, h0, c0, layer, d, mask):
        """``x`` ``[T, B, in]`` -> ``[T, B, H]``; ``mask`` ``[T, B, 1]`` (or None) freezes the state of sequences that have ended."""
        w_ih, w_hh, b_ih, b_hh = self._w(layer, d)
        T, B = x.shape[:2]
        gi_all = _lin(x.reshape(T * B, -1), w_ih, b_ih).view(T, B, -1)
        h, c = h0, c0
        outs: List[Optional[torch.Tensor]] = [None] * T
        for t in (range(T - 1, -1, -1) if d else range(T)):
            hn, cn = self._step(gi_all[t], h, c, w_hh, b_hh)
            if mask is not None:
                m = mask[t]
                hn = torch.where(m, hn, h)
                cn = torch.where(m, cn, c) if cn is not None else None
                outs[t] = torch.where(m, hn, torch.zeros_like(hn))
            else:
                outs[t] = hn
            h, c = hn, cn
        return torch.stack(outs, 0), h, c

    def _forward_impl(self, x, hx):
        packed = _is_packed(x)
        lengths = None
        if packed:
            seq = x
            x, lengths = pad_packed_sequence(PackedSequence(seq.data, seq.batch_sizes, seq.sorted_indices, seq.unsorted_indices))
        elif self.batch_first and x.dim() == 3:
            x = x.transpose(0, 1)
        unb = x.dim() == 2
        if unb:
            x = x.unsqueeze(1)
        if x.dim() != 3 or x.shape[-1] != self.input_size:
            raise ShapeMismatch(f"{type(self).__name__}: expected input [..., {self.input_size}] with 2 or 3 dimensions, got {list(x.shape)}")
        T, B = x.shape[:2]
        D = 2 if self.bidirectional else 1
        want = (self.num_layers * D, B, self.hidden_size)
        is_lstm = self._mode == "lstm"
        if hx is None:
            h0 = x.new_zeros(want)
            c0 = x.new_zeros(want) if is_lstm else None
        else:
            h0, c0 = (hx if is_lstm else (hx, None))
            if unb:
                h0 = h0.unsqueeze(1)
                c0 = c0.unsqueeze(1) if c0 is not None else None
            if tuple(h0.shape) != want or (c0 is not None and tuple(c0.shape) != want):
                raise ShapeMismatch(f"{type(self).__name__}: initial state must have shape {list(want)}, got {list(h0.shape)}")
        mask = None
        if lengths is not None and int(lengths.min()) < T:
            mask = (torch.arange(T).unsqueeze(1) < lengths.unsqueeze(0)).unsqueeze(-1).to(x.device)
        hs, cs = [], []
        inp = x
        for layer in range(self.num_layers):
            outs = []
            for d in range(D):
                k = layer * D + d
                o, h, c = self._run_direction(inp, h0[k], c0[k] if c0 is not None else None, layer, d, mask)
                outs.append(o)
                hs.append(h)
                cs.append(c)
            inp = outs[0] if D == 1 else torch.cat(outs, -1)
            if self.dropout > 0 and self.training and layer + 1 < self.num_layers:
                keep = 1.0 - self.dropout
                inp = inp * (torch.rand_like(inp) < keep).to(inp.dtype) / keep
        h_n = torch.stack(hs, 0)
        c_n = torch.stack(cs, 0) if is_lstm else None
        out = inp
        if packed:
            out = pack_padded_sequence(out, lengths, enforce_sorted=False)
            if isinstance(seq, torch.nn.utils.rnn.PackedSequence):
                out = torch.nn.utils.rnn.PackedSequence(out.data, out.batch_sizes, out.sorted_indices, out.unsorted_indices)
        elif unb:
            out, h_n = out.squeeze(1), h_n.squeeze(1)
            c_n = c_n.squeeze(1) if c_n is not None else None
        elif self.batch_first:
            out = out.transpose(0, 1)
        return out, ((h_n, c_n) if is_lstm else h_n)

    def forward(self, x, hx=None):
        return self._forward_impl(x, hx)

    def extra_repr(self):
        return (f"{self.input_size}, {self.hidden_size}, num_layers={self.num_layers}, bias={self.bias}, batch_first={self.batch_first}, "
                f"dropout={self.dropout}, bidirectional={self.bidirectional}")


class RNN(_RNNBase):
    _gates, _mode = 1, "rnn"

    def __init__(self, input_size: int, hidden_size: int, num_layers: int = 1, nonlinearity: str = "tanh", bias: bool = True, batch_first: bool = False,
                 dropout: float = 0.0, bidirectional: bool = False, device=None, dtype=None):
        nonlinearity = getattr(nonlinearity, "value", nonlinearity)
        if nonlinearity not in ("tanh", "relu"):
            raise InvalidArgument(f"unknown nonlinearity {nonlinearity!r}")
        self.nonlinearity = nonlinearity
        super().__init__(input_size, hidden_size, num_layers, bias, batch_first, dropout, bidirectional, 0, device, dtype)

    def _step(self, gi, h, c, w_hh, b_hh):
        pre = gi + _lin(h, w_hh, b_hh)
        return (torch.tanh(pre) if self.nonlinearity == "tanh" else torch.clamp_min(pre, 0)), None


class LSTM(_RNNBase):
    _gates, _mode = 4, "lstm"

    def _step(self, gi, h, c, w_hh, b_hh):
        return lstm_pointwise(gi + _lin(h, w_hh, b_hh), c)


class GRU(_RNNBase):
    _gates, _mode = 3, "gru"

    def _step(self, gi, h, c, w_hh, b_hh):
        return gru_pointwise(gi, _lin(h, w_hh, b_hh), h), None


__all__ = ["PackedSequence", "pack_padded_sequence", "pad_packed_sequence", "pad_sequence", "pack_sequence", "RNNCell", "LSTMCell", "GRUCell",
           "RNN", "LSTM", "GRU", "lstm_pointwise", "gru_pointwise"]
_ = Union
