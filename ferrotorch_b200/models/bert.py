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
from ..nn.functional import scaled_dot_product_attention as sdpa
from ..errors import InvalidArgument, ShapeMismatch


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
    def from_hf(cls, d) -> "BertConfig":
        """From a parsed ``config.json`` dict or an :class:`HfBertConfig` (validated first; ferrotorch-bert/src/config.rs:64)."""
        if isinstance(d, HfBertConfig):
            d.validate()
            d = d.__dict__
        return cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})

    @classmethod
    def mini_lm_l6(cls) -> "BertConfig":
        return cls(hidden_size=384, num_hidden_layers=6, num_attention_heads=12, intermediate_size=1536)

    all_minilm_l6_v2 = mini_lm_l6                       # the reference's name for the same preset (config.rs:43)

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def validate(self) -> None:
        if self.hidden_size % self.num_attention_heads:
            raise InvalidArgument("hidden_size must be divisible by num_attention_heads")


@dataclass
class HfBertConfig:
    """The fields of a Hugging Face BERT ``config.json`` with the hub's defaults (ferrotorch-bert/src/config.rs:124-216). Unknown keys are ignored;
    a missing required key is an :class:`InvalidArgument`."""
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    intermediate_size: int
    vocab_size: int
    max_position_embeddings: int
    layer_norm_eps: float = 1e-12
    type_vocab_size: int = 2
    hidden_act: str = "gelu"
    pad_token_id: int = 0
    architectures: tuple = ()
    model_type: Optional[str] = None
    position_embedding_type: str = "absolute"

    @classmethod
    def from_json_str(cls, s: str) -> "HfBertConfig":
        try:
            d = json.loads(s)
            return cls(**{k: (tuple(d[k]) if k == "architectures" else d[k]) for k in cls.__dataclass_fields__ if k in d})
        except (ValueError, TypeError) as e:
            raise InvalidArgument(f"failed to parse BERT config JSON: {e}") from None

    @classmethod
    def from_file(cls, path) -> "HfBertConfig":
        try:
            text = open(path, "rb").read().decode("utf-8")
        except (OSError, UnicodeDecodeError) as e:
            raise InvalidArgument(f"failed to read config file {path}: {e}") from None
        return cls.from_json_str(text)

    def validate(self) -> None:
        counts = (self.hidden_size, self.num_attention_heads, self.num_hidden_layers, self.intermediate_size, self.vocab_size, self.type_vocab_size,
                  self.max_position_embeddings)
        if any(int(v) <= 0 for v in counts):
            raise InvalidArgument("HfBertConfig: hidden_size / num_attention_heads / num_hidden_layers / intermediate_size / vocab_size / "
                                  "type_vocab_size / max_position_embeddings must all be positive")
        if self.hidden_size % self.num_attention_heads:
            raise InvalidArgument(f"HfBertConfig: hidden_size ({self.hidden_size}) must be divisible by num_attention_heads ({self.num_attention_heads})")
        if self.hidden_act not in ("gelu", "relu", "gelu_new"):
            raise InvalidArgument(f"HfBertConfig: unsupported hidden_act {self.hidden_act!r}")
        if self.position_embedding_type != "absolute":
            raise InvalidArgument(f"HfBertConfig: unsupported position_embedding_type {self.position_embedding_type!r}")


@dataclass
class DropReport:
    """Which checkpoint keys a loader left out on purpose (ferrotorch-bert/src/model.rs:353): the regenerated ``embeddings.position_ids`` buffer
    and the ``pooler.*`` tensors a sentence encoder never uses."""
    dropped_position_ids: bool = False
    dropped_pooler: tuple = ()
    dropped: tuple = ()            # Whisper encoder loader: keys outside ``encoder.*`` (ferrotorch-whisper/src/encoder.rs:445)
    unmapped: tuple = ()           # policy loader: keys that match no parameter (ferrotorch-rl/src/safetensors_loader.rs:46)


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
        o = sdpa(sp(self.query(x)), sp(self.key(x)), sp(self.value(x)), attn_mask=am)
        return o.transpose(1, 2).reshape(B, S, E)


class BertSelfOutput(nn.Module):
    """Projection + residual + LayerNorm after self-attention (ferrotorch-bert/src/attention.rs:191); with ``in_f`` = intermediate size it is the
    FFN's output block (:class:`BertOutput`, layer.rs:115)."""

    def __init__(self, c, in_f=None):
        super().__init__()
        self.dense = nn.Linear(in_f or c.hidden_size, c.hidden_size)
        self.LayerNorm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)

    def forward(self, h, res):
        return self.LayerNorm(self.dense(h) + res)

    forward_residual = forward


class BertOutput(BertSelfOutput):
    """FFN down-projection + residual + LayerNorm (ferrotorch-bert/src/layer.rs:115)."""

    def __init__(self, c):
        super().__init__(c, c.intermediate_size)


class BertAttention(nn.Module):
    """Self-attention followed by its output block (ferrotorch-bert/src/attention.rs:318)."""

    def __init__(self, c):
        super().__init__()
        self.self = BertSelfAttention(c)
        self.output = BertSelfOutput(c)

    def forward(self, x, mask=None):
        return self.output(self.self(x, mask), x)


class BertIntermediate(nn.Module):
    """FFN up-projection + activation (ferrotorch-bert/src/layer.rs:20)."""

    def __init__(self, c):
        super().__init__()
        self.dense = nn.Linear(c.hidden_size, c.intermediate_size)
        self.act = {"gelu": F.gelu, "relu": F.relu, "gelu_new": lambda t: F.gelu(t, approximate="tanh")}[c.hidden_act]

    def forward(self, x):
        return self.act(self.dense(x))


class BertLayer(nn.Module):
    def __init__(self, c: BertConfig):
        super().__init__()
        self.attention = BertAttention(c)
        self.intermediate = BertIntermediate(c)
        self.output = BertOutput(c)

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

    forward_from_ids = forward

    def load_hf_state_dict(self, hf_state: Dict[str, torch.Tensor], strict: bool = True) -> DropReport:
        """Loads a Hugging Face ``BertModel`` state dict (an optional ``bert.`` prefix is stripped). ``embeddings.position_ids`` is always dropped;
        ``pooler.*`` keys are loaded when this model has a pooler, otherwise dropped (``strict=False``) or refused (``strict=True``), and the
        report says which (ferrotorch-bert/src/model.rs:224-262)."""
        own = self.state_dict()
        keep, dropped_pos, dropped_pool = {}, False, []
        for k, v in hf_state.items():
            k = k[5:] if k.startswith("bert.") else k
            if k == "embeddings.position_ids":
                dropped_pos = True
            elif k.startswith("pooler.") and self.pooler is None:
                if strict:
                    raise InvalidArgument(f"BertModel.load_hf_state_dict: pooler key {k!r} present but this model has no pooler; "
                                          "load with strict=False to drop it")
                dropped_pool.append(k)
            elif k in own:
                if tuple(v.shape) != tuple(own[k].shape):
                    raise ShapeMismatch(f"{k}: checkpoint {tuple(v.shape)} vs model {tuple(own[k].shape)}")
                keep[k] = v
            elif strict:
                raise InvalidArgument(f'unexpected key in BertModel state_dict: "{k}"')
        missing = [k for k in own if k not in keep]
        if strict and missing:
            raise InvalidArgument(f"BertModel.load_hf_state_dict: missing keys {missing[:4]}{'...' if len(missing) > 4 else ''}")
        self.load_state_dict(keep, strict=False)
        return DropReport(dropped_pos, tuple(sorted(dropped_pool)))


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

    @torch.no_grad()
    def encode_texts(self, tokenizer, texts, max_length: int = 512, pad_id: int = 0) -> torch.Tensor:
        """Embeddings ``[len(texts), hidden]`` of strings: tokenised with the file's own special tokens (``[CLS] ... [SEP]``), truncated to
        ``max_length`` keeping the last special token, padded to the longest of the batch with a mask."""
        rows = []
        for t in texts:
            ids = tokenizer.encode(t, add_special_tokens=True)
            rows.append(ids[: max_length - 1] + ids[-1:] if len(ids) > max_length else ids)
        n = max(len(r) for r in rows)
        dev = next(self.parameters()).device
        ids = torch.tensor([r + [pad_id] * (n - len(r)) for r in rows], dtype=torch.long, device=dev)
        mask = torch.tensor([[1] * len(r) + [0] * (n - len(r)) for r in rows], dtype=torch.long, device=dev)
        return self(ids, mask)


def load_bert_model(path: str, cfg: Optional[BertConfig] = None, strict: bool = False, device="cpu", dtype=torch.float32):
    """Two forms. ``load_bert_model(directory)`` reads ``config.json`` + ``model.safetensors`` and returns the model (with a pooler when the file
    has one). ``load_bert_model(weights_file, cfg, strict)`` is the reference's form (ferrotorch-bert/src/safetensors_loader.rs:107): a model
    without pooler plus the :class:`DropReport` of the keys that were left out."""
    from ..serialize import load_safetensors
    if cfg is None:
        cfg = BertConfig.from_hf(json.load(open(os.path.join(path, "config.json"))))
        sd = load_safetensors(os.path.join(path, "model.safetensors"))
        m = BertModel(cfg, add_pooling_layer=any(k.startswith(("pooler.", "bert.pooler.")) for k in sd))
        m.load_hf_state_dict(sd, strict=False)
        return m.to(device=device, dtype=dtype)
    try:
        sd = load_safetensors(str(path))
    except Exception as e:
        raise InvalidArgument(f"load_bert_model: failed to read safetensors {path}: {e}") from None
    m = BertModel(cfg, add_pooling_layer=False)
    report = m.load_hf_state_dict(sd, strict=strict)
    return m.to(device=device, dtype=dtype), report


def load_sentence_transformer(path: str, cfg: BertConfig, normalize: bool = True, strict: bool = False, device="cpu", dtype=torch.float32):
    """A mean-pooling :class:`SentenceTransformer` over :func:`load_bert_model` (weights file + config), with the same drop report
    (ferrotorch-bert/src/safetensors_loader.rs:176)."""
    bert, report = load_bert_model(path, cfg, strict, device, dtype)
    return SentenceTransformer(bert, "mean", normalize), report
