"""Llama building blocks as stand-alone modules with Hugging Face parameter names, the gated-MLP activation variants, and the single-GPU
inferencer with activation-magnitude taps.

The training model (``models/llama.py``) runs a decoder layer as one fused autograd node over flat parameter units; the classes here are the
composable form of the same arithmetic: :class:`LlamaMLP` and :class:`LlamaAttention` (with a KV cache) for custom stacks and for the sparse
activation variants (ReLU / FATReLU) that the fused SwiGLU kernel does not cover, and :class:`LlamaGpuInferencer`, which keeps bf16 weights on
the device and can record per-head / per-MLP-block magnitudes during a forward.

Reference parity: ferrotorch-llama/src/{config.rs:12-19 (LlamaActivation), mlp.rs:24, attention.rs:32-121, gpu.rs:62-80 (ProfiledForwardResult),
gpu.rs:83 (LlamaGpuLayer), gpu.rs:153-440 (LlamaGpuInferencer)}.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import nn, ops
from ..errors import InvalidArgument, ShapeMismatch
from .llama import LlamaConfig


class LlamaActivation:
    """Gate activation of the MLP: ``Silu`` (SwiGLU, the published Llama models), ``Relu`` (ReluLLaMA) or ``FatRelu(threshold)``
    (ProSparse: ``x if x >= threshold else 0``)."""

    def __init__(self, kind: str, threshold: float = 0.0):
        if kind not in ("silu", "relu", "fatrelu"):
            raise InvalidArgument(f"LlamaConfig: unsupported hidden_act {kind!r}")
        self.kind, self.threshold = kind, float(threshold)

    @classmethod
    def FatRelu(cls, threshold: float = 0.01) -> "LlamaActivation":  # noqa: N802 (variant names follow the reference)
        return cls("fatrelu", threshold)

    @classmethod
    def parse(cls, name: str, param: Optional[float] = None) -> "LlamaActivation":
        """``hidden_act`` / ``hidden_act_param`` of a ``config.json`` (config.rs:122-141): silu | swish | relu | fatrelu (default threshold 0.01)."""
        if name in ("silu", "swish"):
            return cls.Silu
        if name == "relu":
            return cls.Relu
        if name == "fatrelu":
            return cls.FatRelu(0.01 if param is None else param)
        raise InvalidArgument(f"LlamaConfig: unsupported hidden_act {name!r}")

    def __call__(self, x: torch.Tensor) -> torch.Tensor:
        if self.kind == "silu":
            return F.silu(x)
        if self.kind == "relu":
            return F.relu(x)
        return torch.where(x >= self.threshold, x, torch.zeros_like(x))

    def __eq__(self, other):
        return isinstance(other, LlamaActivation) and (self.kind, self.threshold) == (other.kind, other.threshold)

    def __hash__(self):
        return hash((self.kind, self.threshold))

    def __repr__(self):
        return {"silu": "LlamaActivation.Silu", "relu": "LlamaActivation.Relu"}.get(self.kind, f"LlamaActivation.FatRelu({self.threshold})")


LlamaActivation.Silu = LlamaActivation("silu")
LlamaActivation.Relu = LlamaActivation("relu")


def config_activation(cfg: LlamaConfig) -> LlamaActivation:
    return LlamaActivation.parse(cfg.hidden_act, getattr(cfg, "hidden_act_param", None))


class LlamaMLP(nn.Module):
    """``down_proj(act(gate_proj(x)) * up_proj(x))``, bias-free (mlp.rs:24)."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        cfg.validate()
        self.act = config_activation(cfg)
        self.gate_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.up_proj = nn.Linear(cfg.hidden_size, cfg.intermediate_size, bias=False)
        self.down_proj = nn.Linear(cfg.intermediate_size, cfg.hidden_size, bias=False)

    def gated(self, x):
        return self.act(self.gate_proj(x)) * self.up_proj(x)

    def forward(self, x):
        return self.down_proj(self.gated(x))


class LlamaAttention(nn.Module):
    """Grouped-query causal self-attention with rotary embeddings (half-split convention) and an optional KV cache (attention.rs:32)."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        cfg.validate()
        self.cfg = cfg
        d, kv = cfg.hidden_size, cfg.num_key_value_heads * cfg.head_dim
        self.q_proj, self.k_proj, self.v_proj = nn.Linear(d, d, bias=False), nn.Linear(d, kv, bias=False), nn.Linear(d, kv, bias=False)
        self.o_proj = nn.Linear(d, d, bias=False)
        self._tables: Optional[Tuple[torch.Tensor, torch.Tensor]] = None

    def num_heads(self) -> int:
        return self.cfg.num_attention_heads

    def num_kv_heads(self) -> int:
        return self.cfg.num_key_value_heads

    def head_dim(self) -> int:
        return self.cfg.head_dim

    def _rope(self, t: torch.Tensor, pos0: int) -> torch.Tensor:
        c = self.cfg
        if self._tables is None or self._tables[0].device != t.device:
            self._tables = ops.rope_tables(c.max_position_embeddings, c.head_dim, c.rope_theta, t.device, c.rope_scaling)
        S, D = t.shape[1], c.head_dim
        if pos0 + S > c.max_position_embeddings:
            raise InvalidArgument(f"LlamaAttention: position {pos0 + S} exceeds max_position_embeddings {c.max_position_embeddings}")
        cos, sin = (x[pos0: pos0 + S].view(1, S, 1, -1) for x in self._tables)
        a, b = t[..., : D // 2].float(), t[..., D // 2:].float()
        return torch.cat([a * cos - b * sin, b * cos + a * sin], -1).to(t.dtype)

    def forward_with_cache(self, x: torch.Tensor, cache=None, head_tap: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
        """``x`` is ``[B, S, hidden]``; ``cache`` is one layer's cache (``append(k, v) -> (K, V)``, ``len()``) or ``None``. The new keys / values are
        appended and the queries attend to everything cached so far (attention.rs:121)."""
        if x.dim() != 3 or x.shape[-1] != self.cfg.hidden_size:
            raise ShapeMismatch(f"LlamaAttention: expected [B, S, {self.cfg.hidden_size}], got {list(x.shape)}")
        B, S, _ = x.shape
        c = self.cfg
        D, Hq, Hkv = c.head_dim, c.num_attention_heads, c.num_key_value_heads
        pos0 = cache.len() if cache is not None else 0
        q = self._rope(self.q_proj(x).view(B, S, Hq, D), pos0).transpose(1, 2)
        k = self._rope(self.k_proj(x).view(B, S, Hkv, D), pos0).transpose(1, 2)
        v = self.v_proj(x).view(B, S, Hkv, D).transpose(1, 2)
        if cache is not None:
            k, v = cache.append(k, v)
        T, rep = k.shape[2], Hq // Hkv
        sc = torch.matmul(q.float(), k.repeat_interleave(rep, 1).float().transpose(-1, -2)) / math.sqrt(D)
        sc = sc.masked_fill(torch.ones(S, T, dtype=torch.bool, device=x.device).triu(T - S + 1), float("-inf"))
        a = torch.matmul(torch.softmax(sc, -1), v.repeat_interleave(rep, 1).float()).to(x.dtype)          # [B, Hq, S, D]
        if head_tap is not None:
            head_tap.append(a.abs().amax(-1).transpose(1, 2).float())                                       # [B, S, Hq]
        return self.o_proj(a.transpose(1, 2).reshape(B, S, Hq * D))

    def forward(self, x):
        return self.forward_with_cache(x, None)


@dataclass
class ProfiledForwardResult:
    """Magnitudes seen during one forward (gpu.rs:62): ``attn_magnitudes [layers, seq, heads]`` is the largest absolute value of each head's
    output before ``o_proj``; ``mlp_magnitudes [layers, seq, blocks]`` the largest absolute value of the gated activation (or, with
    ``plainact_local``, of ``gated * (y @ down_proj)``) per block of ``mlp_block_size`` neurons; ``bootstrap_hidden`` the hidden state entering
    layer ``bootstrap_k`` when one was asked for."""
    seq_len: int
    attn_magnitudes: torch.Tensor
    mlp_magnitudes: torch.Tensor
    bootstrap_hidden: Optional[torch.Tensor]
    bootstrap_k: Optional[int]
    hidden_size: int


class LlamaGpuLayer(nn.Module):
    """One decoder layer's weights on the device (gpu.rs:83): two RMSNorm weights, attention and MLP projections."""

    def __init__(self, cfg: LlamaConfig):
        super().__init__()
        self.cfg = cfg
        self.input_layernorm = nn.Parameter(torch.ones(cfg.hidden_size))
        self.post_attention_layernorm = nn.Parameter(torch.ones(cfg.hidden_size))
        self.self_attn, self.mlp = LlamaAttention(cfg), LlamaMLP(cfg)

    def load(self, W: Dict[str, torch.Tensor], prefix: str) -> "LlamaGpuLayer":
        own = dict(self.named_parameters())
        names = {"input_layernorm": "input_layernorm.weight", "post_attention_layernorm": "post_attention_layernorm.weight"}
        with torch.no_grad():
            for n, p in own.items():
                key = prefix + names.get(n, n)
                if key not in W:
                    raise InvalidArgument(f"LlamaGpuLayer: missing weight {key}")
                if tuple(W[key].shape) != tuple(p.shape):
                    raise ShapeMismatch(f"{key}: {tuple(W[key].shape)} vs {tuple(p.shape)}")
                p.copy_(W[key])
        return self


def _rms(v: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    vf = v.float()
    return (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + eps) * w.float()).to(v.dtype)


class LlamaGpuInferencer:
    """Whole-prompt forward of a Llama checkpoint held on one device in bf16 (gpu.rs:153). ``weights`` uses Hugging Face names
    (``model.embed_tokens.weight``, ``model.layers.N.*``, ``model.norm.weight``, ``lm_head.weight``)."""

    def __init__(self, cfg: LlamaConfig, weights: Dict[str, torch.Tensor], device="cuda", dtype=torch.bfloat16):
        cfg.validate()
        self.config, self.device, self.dtype = cfg, torch.device(device), dtype
        for k in ("model.embed_tokens.weight", "model.norm.weight"):
            if k not in weights:
                raise InvalidArgument(f"LlamaGpuInferencer: missing weight {k}")
        self.embed = weights["model.embed_tokens.weight"].to(self.device, dtype)
        self.final_norm = weights["model.norm.weight"].to(self.device, dtype)
        self.lm_head = self.embed if cfg.tie_word_embeddings or "lm_head.weight" not in weights else weights["lm_head.weight"].to(self.device, dtype)
        self.layers: List[LlamaGpuLayer] = []
        for i in range(cfg.num_hidden_layers):
            self.layers.append(LlamaGpuLayer(cfg).load(weights, f"model.layers.{i}.").to(self.device, dtype))

    def _ids(self, ids: Sequence[int]) -> torch.Tensor:
        if len(ids) == 0:
            raise InvalidArgument("LlamaGpuInferencer: ids must not be empty")
        if max(ids) >= self.config.vocab_size:
            raise InvalidArgument(f"LlamaGpuInferencer: token id {max(ids)} outside the vocabulary ({self.config.vocab_size})")
        return torch.as_tensor(list(ids), dtype=torch.long, device=self.device)[None]

    @torch.no_grad()
    def _core(self, ids, taps: Optional[dict] = None) -> torch.Tensor:
        eps = self.config.rms_norm_eps
        x = self.embed[self._ids(ids)]
        for li, L in enumerate(self.layers):
            if taps is not None and taps["bootstrap_k"] == li:          # k layers have run: the input of (0-based) layer k
                taps["hidden"] = x[0].clone()
            x = x + L.self_attn.forward_with_cache(_rms(x, L.input_layernorm, eps), None, taps["attn"] if taps is not None else None)
            h = _rms(x, L.post_attention_layernorm, eps)
            gated = L.mlp.gated(h)
            x = x + L.mlp.down_proj(gated)
            if taps is not None:
                sig = gated * F.linear(x, L.mlp.down_proj.weight.t()) if taps["plainact_local"] else gated
                nb, bs = taps["n_mlp_blocks"], taps["mlp_block_size"]
                taps["mlp"].append(sig.abs().view(1, -1, nb, bs).amax(-1).float())
        if taps is not None and taps["bootstrap_k"] == len(self.layers):
            taps["hidden"] = x[0].clone()
        return _rms(x, self.final_norm, eps)

    def forward_logits_from_ids_all(self, ids: Sequence[int]) -> torch.Tensor:
        """Logits of every position, ``[seq, vocab]`` f32 (gpu.rs:336)."""
        return F.linear(self._core(ids)[0], self.lm_head).float()

    def forward_from_ids(self, ids: Sequence[int]) -> torch.Tensor:
        """Logits of the last position, ``[vocab]`` f32 (gpu.rs:300): only that row goes through the head."""
        return F.linear(self._core(ids)[0, -1:], self.lm_head)[0].float()

    def forward_from_ids_profiled(self, ids: Sequence[int], mlp_block_size: int, n_mlp_blocks: int) -> ProfiledForwardResult:
        return self.forward_from_ids_profiled_with_bootstrap(ids, mlp_block_size, n_mlp_blocks, None, False)

    def forward_from_ids_profiled_with_bootstrap(self, ids: Sequence[int], mlp_block_size: int, n_mlp_blocks: int, bootstrap_k: Optional[int] = None,
                                                 plainact_local: bool = False) -> ProfiledForwardResult:
        """gpu.rs:406-520. ``mlp_block_size * n_mlp_blocks`` must equal the intermediate size; ``bootstrap_k`` in ``1..=num_hidden_layers`` also
        returns the hidden state after layer ``k - 1``."""
        c = self.config
        if mlp_block_size <= 0 or n_mlp_blocks <= 0 or mlp_block_size * n_mlp_blocks != c.intermediate_size:
            raise InvalidArgument(f"mlp_block_size ({mlp_block_size}) x n_mlp_blocks ({n_mlp_blocks}) must equal intermediate_size ({c.intermediate_size})")
        if bootstrap_k is not None and not 1 <= bootstrap_k <= c.num_hidden_layers:
            raise InvalidArgument(f"bootstrap_k must be in 1..={c.num_hidden_layers}, got {bootstrap_k}")
        taps = {"attn": [], "mlp": [], "mlp_block_size": mlp_block_size, "n_mlp_blocks": n_mlp_blocks, "plainact_local": plainact_local,
                "bootstrap_k": bootstrap_k, "hidden": None}
        self._core(ids, taps)
        return ProfiledForwardResult(len(ids), torch.cat(taps["attn"], 0), torch.cat(taps["mlp"], 0), taps["hidden"], bootstrap_k, c.hidden_size)
