"""BERT encoder and SentenceTransformer pooling head with HF-compatible parameter names.

Reference parity: ferrotorch-bert/src/{config.rs:19, embeddings.rs:25, attention.rs:27, layer.rs:241, encoder.rs:20, model.rs:144,
sentence_transformer.rs:373, loader.rs:107}.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .. import nn
from ..errors import InvalidArgument


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 768
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    intermediate_size: int = 3072
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    layer_norm_eps: float = 1e-12
    hidden_act: str = "gelu"
    pad_token_id: int = 0

    @classmethod
    def from_hf(cls, d: Dict) -> "BertConfig":
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})

    @classmethod
    def mini_lm_l6(cls) -> "BertConfig":
        return cls(hidden_size=384, num_hidden_layers=6, num_attention_heads=12, intermediate_size=1536)

    def validate(self) -> None:
        if self.hidden_size % self.num_attention_heads:
            raise InvalidArgument("hidden_size must be divisible by num_attention_heads")


class BertEmbeddings(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.word_embeddings = nn.Embedding(c.vocab_size, c.hidden_size)
        self.position_embeddings = nn.Embedding(c.max_position_embeddings, c.hidden_size)
        self.token_type_embeddings = nn.Embedding(c.type_vocab_size, c.hidden_size)
        self.LayerNorm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)

    def forward(self, ids, token_type_ids=None):
        S = ids.shape[1]
        pos = torch.arange(S, device=ids.device)[None]
        tt = token_type_ids if token_type_ids is not None else torch.zeros_like(ids)
        return self.LayerNorm(self.word_embeddings(ids) + self.position_embeddings(pos) + self.token_type_embeddings(tt))


class BertSelfAttention(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.h = c.num_attention_heads
        self.query, self.key, self.value = (nn.Linear(c.hidden_size, c.hidden_size) for _ in range(3))

    def forward(self, x, mask=None):
        B, S, E = x.shape
        sp = lambda t: t.view(B, S, self.h, E // self.h).transpose(1, 2)
        am = None
        if mask is not None:                                       # [B, S] 1 = keep
            am = (~mask.bool())[:, None, None, :].expand(B, 1, S, S)
            am = torch.zeros(B, 1, S, S, device=x.device, dtype=x.dtype).masked_fill(am, float("-inf"))
        o = F.scaled_dot_product_attention(sp(self.query(x)), sp(self.key(x)), sp(self.value(x)), attn_mask=am)
        return o.transpose(1, 2).reshape(B, S, E)


class _SelfOutput(nn.Module):
    def __init__(self, c, in_f):
        super().__init__()
        self.dense = nn.Linear(in_f, c.hidden_size)
        self.LayerNorm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)

    def forward(self, h, res):
        return self.LayerNorm(self.dense(h) + res)


class _Attention(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.self = BertSelfAttention(c)
        self.output = _SelfOutput(c, c.hidden_size)

    def forward(self, x, mask=None):
        return self.output(self.self(x, mask), x)


class _Intermediate(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.dense = nn.Linear(c.hidden_size, c.intermediate_size)
        self.act = {"gelu": F.gelu, "relu": F.relu, "gelu_new": lambda t: F.gelu(t, approximate="tanh")}[c.hidden_act]

    def forward(self, x):
        return self.act(self.dense(x))


class BertLayer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.attention = _Attention(c)
        self.intermediate = _Intermediate(c)
        self.output = _SelfOutput(c, c.intermediate_size)

    def forward(self, x, mask=None):
        a = self.attention(x, mask)
        return self.output(self.intermediate(a), a)


class BertEncoder(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.layer = nn.ModuleList([BertLayer(c) for _ in range(c.num_hidden_layers)])

    def forward(self, x, mask=None):
        for l in self.layer:
            x = l(x, mask)
        return x


class BertPooler(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.dense = nn.Linear(c.hidden_size, c.hidden_size)

    def forward(self, x):
        return torch.tanh(self.dense(x[:, 0]))


class BertModel(nn.Module):
    def __init__(self, c: BertConfig, add_pooling_layer: bool = True):
        super().__init__()
        c.validate()
        self.config = c
        self.embeddings = BertEmbeddings(c)
        self.encoder = BertEncoder(c)
        self.pooler = BertPooler(c) if add_pooling_layer else None

    def forward(self, input_ids, attention_mask=None, token_type_ids=None):
        h = self.encoder(self.embeddings(input_ids, token_type_ids), attention_mask)
        return h, (self.pooler(h) if self.pooler is not None else None)


class SentenceTransformer(nn.Module):
    """Mean / CLS / max pooling over the masked token states, optional L2 normalisation (all-MiniLM style)."""

    def __init__(self, bert: BertModel, pooling: str = "mean", normalize: bool = True):
        super().__init__()
        self.bert, self.pooling, self.normalize = bert, pooling, normalize

    def forward(self, input_ids, attention_mask=None):
        h, _ = self.bert(input_ids, attention_mask)
        m = (attention_mask if attention_mask is not None else torch.ones_like(input_ids)).to(h.dtype)[..., None]
        if self.pooling == "mean":
            e = (h * m).sum(1) / m.sum(1).clamp_min(1e-9)
        elif self.pooling == "cls":
            e = h[:, 0]
        elif self.pooling == "max":
            e = h.masked_fill(m == 0, float("-inf")).max(1).values
        else:
            raise InvalidArgument(f"unknown pooling {self.pooling}")
        return F.normalize(e, dim=-1) if self.normalize else e

    encode = forward


def load_bert_model(path: str, device="cpu", dtype=torch.float32) -> BertModel:
    """Loads ``config.json`` + ``model.safetensors`` from a directory (an optional ``bert.`` prefix is stripped)."""
    from ..serialize import load_safetensors
    cfg = BertConfig.from_hf(json.load(open(os.path.join(path, "config.json"))))
    sd = load_safetensors(os.path.join(path, "model.safetensors"))
    sd = {k[5:] if k.startswith("bert.") else k: v for k, v in sd.items()}
    m = BertModel(cfg, add_pooling_layer=any(k.startswith("pooler.") for k in sd))
    own = m.state_dict()
    m.load_state_dict({k: v for k, v in sd.items() if k in own}, strict=False)
    return m.to(device=device, dtype=dtype)
