"""Encoder / decoder transformer stacks (ferrotorch-nn/src/transformer.rs:49-846) built from this package's attention, LayerNorm and Linear.

Mask convention of this file: a boolean mask marks the positions that may NOT be attended (True = blocked); a float mask is added to the
scores. ``*_key_padding_mask`` is ``[B, S]`` with True at padding."""
from __future__ import annotations

import copy
from typing import Callable, Optional, Union

import torch

from ..errors import InvalidArgument
from . import activation as A
from .module import Module, ModuleList


def _additive(mask: Optional[torch.Tensor], dtype=torch.float32) -> Optional[torch.Tensor]:
    if mask is None:
        return None
    if mask.dtype == torch.bool:
        return torch.zeros(mask.shape, dtype=dtype, device=mask.device).masked_fill(mask, float("-inf"))
    return mask.to(dtype)


def _merge(attn_mask, key_padding_mask, causal: bool, Sq: int, Sk: int, device) -> Optional[torch.Tensor]:
    """Everything that restricts attention, as one additive ``[B|1, 1, Sq, Sk]`` tensor (None when unrestricted)."""
    m = None
    if attn_mask is not None:
        a = _additive(attn_mask)
        m = a.view(1, 1, Sq, Sk) if a.dim() == 2 else a.view(a.shape[0], -1, Sq, Sk) if a.dim() == 3 else a
    elif causal:
        m = torch.zeros(Sq, Sk, device=device).masked_fill(torch.ones(Sq, Sk, dtype=torch.bool, device=device).triu(Sk - Sq + 1),
                                                           float("-inf")).view(1, 1, Sq, Sk)
    if key_padding_mask is not None:
        k = _additive(key_padding_mask).view(key_padding_mask.shape[0], 1, 1, Sk)
        m = k if m is None else m + k
    return m


def _act(activation: Union[str, Callable]) -> Callable:
    if callable(activation):
        return activation
    try:
        return {"relu": A.relu, "gelu": _gelu}[activation]
    except KeyError:
        raise InvalidArgument(f"activation must be 'relu', 'gelu' or a callable, got {activation!r}") from None


def _gelu(x):
    from .extras import gelu
    return gelu(x)


def _dropout(x, p: float, training: bool):
    if p <= 0 or not training:
        return x
    return x * (torch.rand_like(x) >= p).to(x.dtype) / (1.0 - p)


class TransformerEncoderLayer(Module):
    """Self-attention block then feed-forward block, each with a residual connection and LayerNorm (before the block when ``norm_first``)."""

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1, activation: Union[str, Callable] = "relu",
                 layer_norm_eps: float = 1e-5, batch_first: bool = False, norm_first: bool = False, bias: bool = True, device=None, dtype=None):
        super().__init__()
        from .layers import LayerNorm, Linear, MultiheadAttention
        self.self_attn = MultiheadAttention(d_model, nhead, bias=bias, device=device, dtype=dtype)
        self.linear1 = Linear(d_model, dim_feedforward, bias, device, dtype)
        self.linear2 = Linear(dim_feedforward, d_model, bias, device, dtype)
        self.norm1 = LayerNorm(d_model, layer_norm_eps, bias=bias, device=device, dtype=dtype)
        self.norm2 = LayerNorm(d_model, layer_norm_eps, bias=bias, device=device, dtype=dtype)
        self.dropout_p, self.batch_first, self.norm_first = float(dropout), batch_first, norm_first
        self.activation = _act(activation)

    def _sa(self, x, mask, causal):
        return _dropout(self.self_attn.forward_qkv(x, x, x, causal and mask is None, mask), self.dropout_p, self.training)

    def _ff(self, x):
        h = _dropout(self.activation(self.linear1(x)), self.dropout_p, self.training)
        return _dropout(self.linear2(h), self.dropout_p, self.training)

    def forward(self, src, src_mask=None, src_key_padding_mask=None, is_causal: bool = False):
        x = src if self.batch_first else src.transpose(0, 1)
        S = x.shape[1]
        mask = _merge(src_mask, src_key_padding_mask, False, S, S, x.device)
        causal = is_causal and src_mask is None
        if causal and mask is not None:
            mask = _merge(None, None, True, S, S, x.device) + mask
        if self.norm_first:
            x = x + self._sa(self.norm1(x), mask, causal)
            x = x + self._ff(self.norm2(x))
        else:
            x = self.norm1(x + self._sa(x, mask, causal))
            x = self.norm2(x + self._ff(x))
        return x if self.batch_first else x.transpose(0, 1)


class TransformerDecoderLayer(Module):
    """Masked self-attention, attention over the encoder memory, feed-forward; residual + LayerNorm around each."""

    def __init__(self, d_model: int, nhead: int, dim_feedforward: int = 2048, dropout: float = 0.1, activation: Union[str, Callable] = "relu",
                 layer_norm_eps: float = 1e-5, batch_first: bool = False, norm_first: bool = False, bias: bool = True, device=None, dtype=None):
        super().__init__()
        from .layers import LayerNorm, Linear, MultiheadAttention
        self.self_attn = MultiheadAttention(d_model, nhead, bias=bias, device=device, dtype=dtype)
        self.multihead_attn = MultiheadAttention(d_model, nhead, bias=bias, device=device, dtype=dtype)
        self.linear1 = Linear(d_model, dim_feedforward, bias, device, dtype)
        self.linear2 = Linear(dim_feedforward, d_model, bias, device, dtype)
        self.norm1, self.norm2, self.norm3 = (LayerNorm(d_model, layer_norm_eps, bias=bias, device=device, dtype=dtype) for _ in range(3))
        self.dropout_p, self.batch_first, self.norm_first = float(dropout), batch_first, norm_first
        self.activation = _act(activation)

    def _ff(self, x):
        h = _dropout(self.activation(self.linear1(x)), self.dropout_p, self.training)
        return _dropout(self.linear2(h), self.dropout_p, self.training)

    def forward(self, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None, memory_key_padding_mask=None,
                tgt_is_causal: bool = False, memory_is_causal: bool = False):
        x = tgt if self.batch_first else tgt.transpose(0, 1)
        mem = memory if self.batch_first else memory.transpose(0, 1)
        T, S = x.shape[1], mem.shape[1]
        causal = tgt_is_causal and tgt_mask is None
        m_self = _merge(tgt_mask, tgt_key_padding_mask, False, T, T, x.device)
        if causal and m_self is not None:
            m_self, causal = _merge(None, None, True, T, T, x.device) + m_self, False
        m_cross = _merge(memory_mask, memory_key_padding_mask, memory_is_causal and memory_mask is None, T, S, x.device)

        def sa(v):
            return _dropout(self.self_attn.forward_qkv(v, v, v, causal, m_self), self.dropout_p, self.training)

        def ca(v):
            return _dropout(self.multihead_attn.forward_qkv(v, mem, mem, False, m_cross), self.dropout_p, self.training)

        if self.norm_first:
            x = x + sa(self.norm1(x))
            x = x + ca(self.norm2(x))
            x = x + self._ff(self.norm3(x))
        else:
            x = self.norm1(x + sa(x))
            x = self.norm2(x + ca(x))
            x = self.norm3(x + self._ff(x))
        return x if self.batch_first else x.transpose(0, 1)


def _clones(layer: Module, n: int) -> ModuleList:
    return ModuleList([copy.deepcopy(layer) for _ in range(n)])


class TransformerEncoder(Module):
    def __init__(self, encoder_layer: Module, num_layers: int, norm: Optional[Module] = None, enable_nested_tensor: bool = False, mask_check: bool = True):
        super().__init__()
        if num_layers <= 0:
            raise InvalidArgument("num_layers must be positive")
        self.layers, self.num_layers, self.norm = _clones(encoder_layer, num_layers), num_layers, norm

    def forward(self, src, mask=None, src_key_padding_mask=None, is_causal: bool = False):
        x = src
        for layer in self.layers:
            x = layer(x, src_mask=mask, src_key_padding_mask=src_key_padding_mask, is_causal=is_causal)
        return self.norm(x) if self.norm is not None else x


class TransformerDecoder(Module):
    def __init__(self, decoder_layer: Module, num_layers: int, norm: Optional[Module] = None):
        super().__init__()
        if num_layers <= 0:
            raise InvalidArgument("num_layers must be positive")
        self.layers, self.num_layers, self.norm = _clones(decoder_layer, num_layers), num_layers, norm

    def forward(self, tgt, memory, tgt_mask=None, memory_mask=None, tgt_key_padding_mask=None, memory_key_padding_mask=None,
                tgt_is_causal: bool = False, memory_is_causal: bool = False):
        x = tgt
        for layer in self.layers:
            x = layer(x, memory, tgt_mask=tgt_mask, memory_mask=memory_mask, tgt_key_padding_mask=tgt_key_padding_mask,
                      memory_key_padding_mask=memory_key_padding_mask, tgt_is_causal=tgt_is_causal, memory_is_causal=memory_is_causal)
        return self.norm(x) if self.norm is not None else x


class Transformer(Module):
    """Encoder-decoder model of "Attention Is All You Need": ``num_encoder_layers`` + ``num_decoder_layers`` blocks, a final LayerNorm on each stack."""

    def __init__(self, d_model: int = 512, nhead: int = 8, num_encoder_layers: int = 6, num_decoder_layers: int = 6, dim_feedforward: int = 2048,
                 dropout: float = 0.1, activation: Union[str, Callable] = "relu", custom_encoder: Optional[Module] = None,
                 custom_decoder: Optional[Module] = None, layer_norm_eps: float = 1e-5, batch_first: bool = False, norm_first: bool = False,
                 bias: bool = True, device=None, dtype=None):
        super().__init__()
        from .layers import LayerNorm
        kw = dict(dim_feedforward=dim_feedforward, dropout=dropout, activation=activation, layer_norm_eps=layer_norm_eps, batch_first=batch_first,
                  norm_first=norm_first, bias=bias, device=device, dtype=dtype)
        self.encoder = custom_encoder or TransformerEncoder(TransformerEncoderLayer(d_model, nhead, **kw), num_encoder_layers,
                                                            LayerNorm(d_model, layer_norm_eps, bias=bias, device=device, dtype=dtype))
        self.decoder = custom_decoder or TransformerDecoder(TransformerDecoderLayer(d_model, nhead, **kw), num_decoder_layers,
                                                            LayerNorm(d_model, layer_norm_eps, bias=bias, device=device, dtype=dtype))
        self.d_model, self.nhead, self.batch_first = d_model, nhead, batch_first
        # every block starts from its own draw: the stacks were cloned from one layer each
        for p in self.parameters():
            if p.dim() > 1:
                torch.nn.init.xavier_uniform_(p)

    @staticmethod
    def generate_square_subsequent_mask(sz: int, device=None, dtype=torch.float32) -> torch.Tensor:
        return torch.zeros(sz, sz, device=device, dtype=dtype).masked_fill(torch.ones(sz, sz, dtype=torch.bool, device=device).triu(1), float("-inf"))

    def forward(self, src, tgt, src_mask=None, tgt_mask=None, memory_mask=None, src_key_padding_mask=None, tgt_key_padding_mask=None,
                memory_key_padding_mask=None, src_is_causal: bool = False, tgt_is_causal: bool = False, memory_is_causal: bool = False):
        bdim = 0 if self.batch_first else 1
        if src.dim() == 3 and src.shape[bdim] != tgt.shape[bdim]:
            raise InvalidArgument("src and tgt must have the same batch size")
        if src.shape[-1] != self.d_model or tgt.shape[-1] != self.d_model:
            raise InvalidArgument(f"the feature dimension of src and tgt must equal d_model = {self.d_model}")
        memory = self.encoder(src, mask=src_mask, src_key_padding_mask=src_key_padding_mask, is_causal=src_is_causal)
        return self.decoder(tgt, memory, tgt_mask=tgt_mask, memory_mask=memory_mask, tgt_key_padding_mask=tgt_key_padding_mask,
                            memory_key_padding_mask=memory_key_padding_mask, tgt_is_causal=tgt_is_causal, memory_is_causal=memory_is_causal)


__all__ = ["TransformerEncoderLayer", "TransformerDecoderLayer", "TransformerEncoder", "TransformerDecoder", "Transformer"]
