"""Llama-3 family: config, decoder stack, causal-LM head, fused training path.

Every decoder layer's weights live in one flat bf16 buffer
(:class:`~ferrotorch_b200.parallel.flat.FlatUnit`), with ``q/k/v`` fused into
one ``[ (Hq+2Hkv)*D, d ]`` matrix and ``gate/up`` into one ``[2F, d]`` matrix so
each is a single GEMM. A layer is one autograd node whose forward and backward
are hand-scheduled sequences of the sm_100a kernels (RMSNorm, tcgen05 GEMM,
in-place RoPE, FlashAttention, SwiGLU), saving only what the backward cannot
cheaply recompute. State dicts use the HF key names
(``model.layers.N.self_attn.q_proj.weight`` ...), splitting the fused matrices.

Reference parity: LlamaConfig + presets (ferrotorch-llama/src/config.rs:23-174), LlamaAttention
(attention.rs:32-185), LlamaMLP (mlp.rs:24), LlamaDecoderLayer (layer.rs:23-63), LlamaModel /
LlamaForCausalLM (model.rs:20-400), GPU inferencer op sequence (gpu.rs:518-700).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Callable, Dict, List, Optional

import torch

from .. import ops
from ..errors import InvalidArgument
from ..parallel.flat import FlatUnit


@dataclass
class LlamaConfig:
    vocab_size: int = 128256
    hidden_size: int = 4096
    intermediate_size: int = 14336
    num_hidden_layers: int = 32
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    rms_norm_eps: float = 1e-5
    rope_theta: float = 500000.0
    max_position_embeddings: int = 8192
    tie_word_embeddings: bool = False
    rope_scaling: Optional[dict] = None
    hidden_act: str = "silu"                      # silu | swish | relu | fatrelu (ferrotorch-llama/src/config.rs:12-19, 122-141)
    hidden_act_param: Optional[float] = None      # FATReLU threshold (0.01 when absent)

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def kv_group_size(self) -> int:
        return self.num_attention_heads // self.num_key_value_heads

    @property
    def activation(self):
        from .llama_blocks import LlamaActivation
        return LlamaActivation.parse(self.hidden_act, self.hidden_act_param)

    # -- presets (ferrotorch-llama/src/config.rs:50-113) ------------------------
    @staticmethod
    def llama3_8b() -> "LlamaConfig":
        return LlamaConfig()

    @staticmethod
    def llama3_70b() -> "LlamaConfig":
        return LlamaConfig(hidden_size=8192, intermediate_size=28672, num_hidden_layers=80, num_attention_heads=64,
                           num_key_value_heads=8)

    @staticmethod
    def llama3_3_70b_instruct() -> "LlamaConfig":
        c = LlamaConfig.llama3_70b()
        c.max_position_embeddings = 131072
        # the published checkpoint's config.json carries the frequency-dependent rope scaling of Llama 3.1 and later
        c.rope_scaling = {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
        return c

    @staticmethod
    def tiny(layers: int = 2, hidden: int = 256, heads: int = 2, kv_heads: int = 1, ffn: int = 512, vocab: int = 1024) -> "LlamaConfig":
        """A small configuration with head_dim 128 for tests and smoke runs."""
        return LlamaConfig(vocab_size=vocab, hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers,
                           num_attention_heads=heads, num_key_value_heads=kv_heads, max_position_embeddings=2048)

    @staticmethod
    def from_hf(src) -> "LlamaConfig":
        """Build from a HF ``config.json`` path or an already parsed dict."""
        d = json.loads(Path(src).read_text()) if not isinstance(src, dict) else src
        keys = {f for f in LlamaConfig.__dataclass_fields__}
        c = LlamaConfig(**{k: v for k, v in d.items() if k in keys})
        c.validate()
        return c

    def validate(self) -> None:
        if self.hidden_size % self.num_attention_heads:
            raise InvalidArgument("hidden_size must be divisible by num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads:
            raise InvalidArgument("num_attention_heads must be divisible by num_key_value_heads")
        if self.head_dim % 2:
            raise InvalidArgument("head_dim must be even for rotary embeddings")
        if min(self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers) <= 0:
            raise InvalidArgument("sizes must be positive")
        if self.hidden_act not in ("silu", "swish", "relu", "fatrelu"):
            raise InvalidArgument(f"LlamaConfig: unsupported hidden_act {self.hidden_act!r}")

    def num_parameters(self) -> int:
        d, F, V, L = self.hidden_size, self.intermediate_size, self.vocab_size, self.num_hidden_layers
        kv = self.num_key_value_heads * self.head_dim
        per = d * d * 2 + 2 * d * kv + 3 * d * F + 2 * d
        return L * per + V * d * (1 if self.tie_word_embeddings else 2) + d

    def to_dict(self) -> dict:
        return asdict(self)


def layer_shapes(cfg: LlamaConfig):
    d, F, D = cfg.hidden_size, cfg.intermediate_size, cfg.head_dim
    nqkv = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * D
    # in the order the forward pass reads them: a fully sharded engine gathers a unit front to back, so the consumers can start on the first
    # pieces while the rest is still in flight (the backward pass asks for the pieces in reverse order)
    return [("norm1", (d,)), ("norm2", (d,)), ("wqkv", (nqkv, d)), ("wo", (d, cfg.num_attention_heads * D)), ("wgu", (2 * F, d)),
            ("wd", (d, F))]


# ---------------------------------------------------------------------------
# hand-scheduled layer forward / backward on 2-D [tokens, features] buffers
# ---------------------------------------------------------------------------
def _layer_forward(x, P, cfg: LlamaConfig, B: int, S: int, rope):
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    cos, sin = rope
    gate = getattr(P, "gate", None)          # fully sharded engine: the weights may still be arriving (see parallel/gather.py)
    if gate is not None:
        gate.wait(P["norm1"])
        gate.wait(P["norm2"])
    h, rstd1, _ = ops.rmsnorm_fwd(x, P["norm1"], cfg.rms_norm_eps)
    qkv = ops.gemm(h, P["wqkv"], gate=gate)
    del h
    ops.rope_inplace(qkv, cos, sin, S, 0, Hq + Hkv, D)       # q heads and k heads are adjacent in the packed row
    attn, lse = ops.flash_fwd(qkv, B, S, Hq, Hkv, D, True)
    o = ops.gemm(attn, P["wo"], gate=gate)
    h2, rstd2, x1 = ops.rmsnorm_fwd(o, P["norm2"], cfg.rms_norm_eps, residual=x)   # x1 = x + o
    del o
    gu = ops.gemm(h2, P["wgu"], gate=gate)
    del h2
    a = ops.swiglu_fwd(gu)
    dn = ops.gemm(a, P["wd"], gate=gate)
    del a
    out = ops.add_(dn, x1)                                    # out = x1 + dn, written over dn
    return out, (x, rstd1, qkv, attn, lse, x1, rstd2, gu)


def _layer_backward(dout, saved, P, G, cfg: LlamaConfig, B: int, S: int, rope):
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    cos, sin = rope
    x, rstd1, qkv, attn, lse, x1, rstd2, gu = saved
    gate = getattr(P, "gate", None)
    if gate is not None:
        gate.wait(P["norm1"])
        gate.wait(P["norm2"])
    # ---- MLP ----
    a = ops.swiglu_fwd(gu)
    ops.gemm(dout, a, a_mn=True, b_mn=True, out=G["wd"])                 # dWd = dout^T a
    del a
    da = ops.gemm(dout, P["wd"], b_mn=True, gate=gate)                    # [T, F]
    dgu = ops.swiglu_bwd(gu, da, inplace=True)
    del da
    h2, _, _ = ops.rmsnorm_fwd(x1, P["norm2"], cfg.rms_norm_eps)
    ops.gemm(dgu, h2, a_mn=True, b_mn=True, out=G["wgu"])
    del h2
    dh2 = ops.gemm(dgu, P["wgu"], b_mn=True, gate=gate)
    del dgu
    dx1, _ = ops.rmsnorm_bwd(x1, P["norm2"], dh2, rstd2, dres=dout, dw_out=G["norm2"])
    del dh2
    # ---- attention ----
    ops.gemm(dx1, attn, a_mn=True, b_mn=True, out=G["wo"])
    dattn = ops.gemm(dx1, P["wo"], b_mn=True, gate=gate)
    dqkv = ops.flash_bwd(qkv, attn, lse, dattn, B, S, Hq, Hkv, D, True)
    del dattn
    ops.rope_inplace(dqkv, cos, sin, S, 0, Hq + Hkv, D, inverse=True)
    h, _, _ = ops.rmsnorm_fwd(x, P["norm1"], cfg.rms_norm_eps)
    ops.gemm(dqkv, h, a_mn=True, b_mn=True, out=G["wqkv"])
    del h
    dh = ops.gemm(dqkv, P["wqkv"], b_mn=True, gate=gate)
    del dqkv
    dx, _ = ops.rmsnorm_bwd(x, P["norm1"], dh, rstd1, dres=dx1, dw_out=G["norm1"])
    return dx


class _DecoderLayerFn(torch.autograd.Function):
    """One decoder layer as a single autograd node.

    ``owner`` supplies the weights and gradient buffers at the moment they are needed:
    ``owner.acquire_params()`` (all-gathers under FSDP), ``owner.acquire_grads()`` and
    ``owner.grads_ready()`` (reduce-scatter / optimizer step under the engine).
    """

    @staticmethod
    def forward(ctx, x, flat, owner, B, S):
        cfg, rope = owner.cfg, owner.rope
        x2 = x.reshape(B * S, cfg.hidden_size)
        P = owner.acquire_params()
        out, saved = _layer_forward(x2, P, cfg, B, S, rope)
        owner.release_params(after_forward=True)
        if owner.recompute:
            ctx.saved = (x2,)
        else:
            ctx.saved = saved
        ctx.owner, ctx.B, ctx.S = owner, B, S
        return out.view(B, S, cfg.hidden_size)

    @staticmethod
    def backward(ctx, dout):
        owner, B, S = ctx.owner, ctx.B, ctx.S
        cfg, rope = owner.cfg, owner.rope
        d2 = dout.reshape(B * S, cfg.hidden_size)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        P = owner.acquire_params(backward=True)
        saved = ctx.saved
        if owner.recompute:
            _, saved = _layer_forward(saved[0], P, cfg, B, S, rope)
        G = owner.acquire_grads()
        dx = _layer_backward(d2, saved, P, G, cfg, B, S, rope)
        ctx.saved = None
        owner.release_params(after_forward=False)
        owner.grads_ready()
        return dx.view(B, S, cfg.hidden_size), None, None, None, None


class _LMHeadLossFn(torch.autograd.Function):
    """Final norm output -> logits -> mean cross-entropy, with the gradients computed in the same pass.

    The logits of a row chunk are produced by the GEMM, turned into their own gradient in place by the fused
    cross-entropy kernel and consumed at once by the dgrad and wgrad GEMMs, so at most one chunk of
    ``[rows, vocab]`` is alive and nothing vocabulary-sized is saved for backward.
    """

    @staticmethod
    def forward(ctx, h, flat, owner, targets, ignore_index, chunk_rows):
        T, d = h.shape
        t = targets.reshape(-1)
        P = owner.acquire_params()
        w, gate = P["weight"], getattr(P, "gate", None)
        G = owner.acquire_grads()
        gw = G["weight"]
        n_valid = T if ignore_index is None else None
        if n_valid is None:
            n_valid = int((t != ignore_index).sum().item())
        scale = 1.0 / max(n_valid, 1)
        dh = torch.empty_like(h)
        total = torch.zeros((), device=h.device, dtype=torch.float32)
        first = True
        for r0 in range(0, T, chunk_rows):
            r1 = min(T, r0 + chunk_rows)
            logits = ops.gemm(h[r0:r1], w, gate=gate)
            loss_c, dl, cnt = ops.cross_entropy_fwd_bwd(logits, t[r0:r1], ignore_index=-100 if ignore_index is None else ignore_index,
                                                        grad_scale=scale, inplace_grad=True)
            total += loss_c * cnt
            ops.gemm(dl, w, b_mn=True, out=dh[r0:r1], gate=gate)
            if first:
                ops.gemm(dl, h[r0:r1], a_mn=True, b_mn=True, out=gw)
                first = False
            else:
                gw += ops.gemm(dl, h[r0:r1], a_mn=True, b_mn=True)
            del logits, dl
        owner.release_params(after_forward=False)
        ctx.save_for_backward(dh)
        ctx.owner = owner
        return total * scale

    @staticmethod
    def backward(ctx, g):
        (dh,) = ctx.saved_tensors
        # the engine calls backward with g == 1; a different upstream scale is folded into both gradients here
        if not (g.numel() == 1 and float(g) == 1.0):
            dh = dh * g.to(dh.dtype)
            ctx.owner.acquire_grads()["weight"].mul_(g.to(dh.dtype))
        ctx.owner.grads_ready()
        return dh, None, None, None, None, None


class _ParamOwner:
    """Default (single-device, no engine) owner of a unit: weights resident, gradients in a private buffer."""

    def __init__(self, unit: FlatUnit, cfg: LlamaConfig, rope=None):
        self.unit, self.cfg, self.rope = unit, cfg, rope
        self.recompute = False
        self.on_grads_ready: Optional[Callable] = None

    def acquire_params(self, backward: bool = False) -> Dict[str, torch.Tensor]:
        return self.unit.views()

    def release_params(self, after_forward: bool) -> None:
        pass

    def acquire_grads(self) -> Dict[str, torch.Tensor]:
        if self.unit.grad is None:
            self.unit.grad = torch.zeros_like(self.unit.full)
        return self.unit.views(self.unit.grad)

    def grads_ready(self) -> None:
        if self.on_grads_ready is not None:
            self.on_grads_ready(self.unit)


class LlamaDecoderLayer(torch.nn.Module):
    def __init__(self, cfg: LlamaConfig, idx: int, device, world: int = 1, rank: int = 0):
        super().__init__()
        self.cfg, self.idx = cfg, idx
        self.unit = FlatUnit(f"layers.{idx}", layer_shapes(cfg), device, torch.bfloat16, world, rank)
        self.flat = torch.nn.Parameter(self.unit.full, requires_grad=True)
        self.owner = _ParamOwner(self.unit, cfg)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, _ = x.shape
        if not x.is_cuda:
            return self._forward_reference(x)
        return _DecoderLayerFn.apply(x, self.flat, self.owner, B, S)

    def _forward_reference(self, x: torch.Tensor) -> torch.Tensor:
        """Plain PyTorch evaluation (CPU oracle / generic autograd path)."""
        cfg = self.cfg
        B, S, d = x.shape
        Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        P = {n: self.unit.view(n, self.flat) for n in self.unit.specs}
        cos, sin = self.owner.rope

        def rms(v, w):
            vf = v.float()
            return (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w.float()).to(v.dtype)

        def rot(t):  # [B,S,H,D]
            c, s = cos[:S].view(1, S, 1, D // 2), sin[:S].view(1, S, 1, D // 2)
            a, b = t[..., : D // 2].float(), t[..., D // 2:].float()
            return torch.cat([a * c - b * s, b * c + a * s], -1).to(t.dtype)

        h = rms(x, P["norm1"])
        qkv = torch.nn.functional.linear(h, P["wqkv"])
        q = rot(qkv[..., : Hq * D].reshape(B, S, Hq, D)).transpose(1, 2)
        k = rot(qkv[..., Hq * D: (Hq + Hkv) * D].reshape(B, S, Hkv, D)).transpose(1, 2)
        v = qkv[..., (Hq + Hkv) * D:].reshape(B, S, Hkv, D).transpose(1, 2)
        rep = Hq // Hkv
        k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        att = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True).to(x.dtype)
        o = torch.nn.functional.linear(att.transpose(1, 2).reshape(B, S, Hq * D), P["wo"])
        x1 = x + o
        gu = torch.nn.functional.linear(rms(x1, P["norm2"]), P["wgu"])
        F = cfg.intermediate_size
        a = (torch.nn.functional.silu(gu[..., :F].float()) * gu[..., F:].float()).to(x.dtype)
        return x1 + torch.nn.functional.linear(a, P["wd"])


class LlamaModel(torch.nn.Module):
    """Embedding + decoder stack + final RMSNorm."""

    def __init__(self, cfg: LlamaConfig, device="cuda", world: int = 1, rank: int = 0):
        super().__init__()
        cfg.validate()
        if cfg.hidden_act not in ("silu", "swish"):
            raise InvalidArgument(f"the fused training layer implements SwiGLU only; build {cfg.hidden_act!r} models from models.llama_blocks")
        self.cfg = cfg
        d, V = cfg.hidden_size, cfg.vocab_size
        self.embed_unit = FlatUnit("embed_tokens", [("weight", (V, d))], device, torch.bfloat16, world, rank)
        self.embed_flat = torch.nn.Parameter(self.embed_unit.full)
        self.layers = torch.nn.ModuleList([LlamaDecoderLayer(cfg, i, device, world, rank) for i in range(cfg.num_hidden_layers)])
        self.norm_unit = FlatUnit("norm", [("weight", (d,))], device, torch.bfloat16, world, rank)
        self.norm_flat = torch.nn.Parameter(self.norm_unit.full)
        self.embed_owner = _ParamOwner(self.embed_unit, cfg)
        self.norm_owner = _ParamOwner(self.norm_unit, cfg)
        self._rope_len = 0
        self.ensure_rope(min(cfg.max_position_embeddings, 8192))

    def ensure_rope(self, seq_len: int) -> None:
        if seq_len <= self._rope_len:
            return
        dev = self.embed_flat.device
        rope = ops.rope_tables(seq_len, self.cfg.head_dim, self.cfg.rope_theta, dev, self.cfg.rope_scaling)
        self._rope_len = seq_len
        self.rope = rope
        for l in self.layers:
            l.owner.rope = rope

    def units(self) -> List[FlatUnit]:
        return [self.embed_unit] + [l.unit for l in self.layers] + [self.norm_unit]

    def owners(self) -> List[_ParamOwner]:
        return [self.embed_owner] + [l.owner for l in self.layers] + [self.norm_owner]

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        B, S = ids.shape
        self.ensure_rope(S)
        if ids.is_cuda:
            x = _EmbedFn.apply(ids, self.embed_flat, self.embed_owner)
        else:
            x = self.embed_unit.view("weight", self.embed_flat)[ids]
        for l in self.layers:
            x = l(x)
        if x.is_cuda:
            return _FinalNormFn.apply(x, self.norm_flat, self.norm_owner)
        xf = x.float()
        w = self.norm_unit.view("weight", self.norm_flat)
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps) * w.float()).to(x.dtype)


class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, flat, owner):
        P = owner.acquire_params()
        if getattr(P, "gate", None) is not None:
            P.gate.wait(P["weight"])
        out = ops.embedding_fwd(ids, P["weight"])
        owner.release_params(after_forward=True)
        ctx.save_for_backward(ids)
        ctx.owner = owner
        return out

    @staticmethod
    def backward(ctx, dout):
        (ids,) = ctx.saved_tensors
        owner = ctx.owner
        G = owner.acquire_grads()
        gw = G["weight"]
        if not getattr(owner, "grad_preaccumulated", False):
            gw.zero_()
        ops.embedding_bwd(ids, dout.reshape(-1, gw.shape[1]).contiguous(), gw)
        owner.grads_ready()
        return None, None, None


class _FinalNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, flat, owner):
        shp = x.shape
        x2 = x.reshape(-1, shp[-1])
        P = owner.acquire_params()
        if getattr(P, "gate", None) is not None:
            P.gate.wait(P["weight"])
        y, rstd, _ = ops.rmsnorm_fwd(x2, P["weight"], owner.cfg.rms_norm_eps)
        owner.release_params(after_forward=True)
        ctx.save_for_backward(x2, rstd)
        ctx.owner, ctx.shp = owner, shp
        return y.view(shp)

    @staticmethod
    def backward(ctx, dy):
        x2, rstd = ctx.saved_tensors
        owner = ctx.owner
        P, G = owner.acquire_params(backward=True), owner.acquire_grads()
        if getattr(P, "gate", None) is not None:
            P.gate.wait(P["weight"])
        dx, _ = ops.rmsnorm_bwd(x2, P["weight"], dy.reshape(x2.shape).contiguous(), rstd, dw_out=G["weight"])
        owner.release_params(after_forward=False)
        owner.grads_ready()
        return dx.view(ctx.shp), None, None


class LlamaForCausalLM(torch.nn.Module):
    """Decoder stack + (untied unless ``tie_word_embeddings``) LM head.

    ``forward(ids)`` returns logits; ``forward(ids, labels=...)`` returns the mean next-token loss
    through the fused head+loss path (labels are already shifted: ``labels[b, s]`` is the target of position ``s``).
    """

    def __init__(self, cfg: LlamaConfig, device="cuda", world: int = 1, rank: int = 0, init_std: float = 0.02, seed: int = 0):
        super().__init__()
        self.cfg = cfg
        self.model = LlamaModel(cfg, device, world, rank)
        if cfg.tie_word_embeddings:
            self.head_unit, self.head_flat, self.head_owner = self.model.embed_unit, self.model.embed_flat, self.model.embed_owner
            self.head_owner.grad_preaccumulated = True
        else:
            self.head_unit = FlatUnit("lm_head", [("weight", (cfg.vocab_size, cfg.hidden_size))], device, torch.bfloat16, world, rank)
            self.head_flat = torch.nn.Parameter(self.head_unit.full)
            self.head_owner = _ParamOwner(self.head_unit, cfg)
        self.loss_chunk_rows = 8192
        self.reset_parameters(init_std, seed)

    def reset_parameters(self, std: float = 0.02, seed: int = 0) -> None:
        gen = torch.Generator(device=self.head_flat.device)
        gen.manual_seed(seed)
        with torch.no_grad():
            for u in self.units():
                for name, spec in u.specs.items():
                    v = u.view(name)
                    if len(spec.shape) == 1:
                        v.fill_(1.0)
                    else:
                        v.normal_(0.0, std, generator=gen)

    def units(self) -> List[FlatUnit]:
        us = self.model.units()
        if not self.cfg.tie_word_embeddings:
            us.append(self.head_unit)
        return us

    def owners(self):
        os_ = self.model.owners()
        if not self.cfg.tie_word_embeddings:
            os_.append(self.head_owner)
        return os_

    def set_recompute(self, flag: bool) -> None:
        for l in self.model.layers:
            l.owner.recompute = flag

    def forward(self, ids: torch.Tensor, labels: Optional[torch.Tensor] = None, ignore_index: Optional[int] = None):
        h = self.model(ids)
        B, S, d = h.shape
        if labels is not None and h.is_cuda:
            return _LMHeadLossFn.apply(h.reshape(B * S, d), self.head_flat, _HeadOwnerView(self.head_owner, self.cfg.tie_word_embeddings), labels,
                                       ignore_index, self.loss_chunk_rows)
        w = self.head_unit.view("weight", self.head_flat)
        if labels is None:
            return ops.linear(h, w)
        logits = torch.nn.functional.linear(h.float(), w.float())
        return torch.nn.functional.cross_entropy(logits.reshape(B * S, -1), labels.reshape(-1),
                                                 ignore_index=-100 if ignore_index is None else ignore_index)

    # -- HF-compatible state dict ------------------------------------------------------------
    def hf_state_dict(self) -> Dict[str, torch.Tensor]:
        cfg = self.cfg
        D, Hq, Hkv, F = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
        sd = {"model.embed_tokens.weight": self.model.embed_unit.view("weight")}
        for i, l in enumerate(self.model.layers):
            u, p = l.unit, f"model.layers.{i}."
            wqkv, wgu = u.view("wqkv"), u.view("wgu")
            sd[p + "self_attn.q_proj.weight"] = wqkv[: Hq * D]
            sd[p + "self_attn.k_proj.weight"] = wqkv[Hq * D: (Hq + Hkv) * D]
            sd[p + "self_attn.v_proj.weight"] = wqkv[(Hq + Hkv) * D:]
            sd[p + "self_attn.o_proj.weight"] = u.view("wo")
            sd[p + "mlp.gate_proj.weight"] = wgu[:F]
            sd[p + "mlp.up_proj.weight"] = wgu[F:]
            sd[p + "mlp.down_proj.weight"] = u.view("wd")
            sd[p + "input_layernorm.weight"] = u.view("norm1")
            sd[p + "post_attention_layernorm.weight"] = u.view("norm2")
        sd["model.norm.weight"] = self.model.norm_unit.view("weight")
        if not cfg.tie_word_embeddings:
            sd["lm_head.weight"] = self.head_unit.view("weight")
        return sd

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor], strict: bool = True) -> List[str]:
        mine = self.hf_state_dict()
        missing = [k for k in mine if k not in sd]
        unexpected = [k for k in sd if k not in mine and not (self.cfg.tie_word_embeddings and k == "lm_head.weight")]
        if strict and (missing or unexpected):
            raise InvalidArgument(f"state dict mismatch: missing {missing[:4]}, unexpected {unexpected[:4]}")
        with torch.no_grad():
            for k, dst in mine.items():
                if k in sd:
                    if tuple(sd[k].shape) != tuple(dst.shape):
                        raise InvalidArgument(f"shape mismatch for {k}: {tuple(sd[k].shape)} vs {tuple(dst.shape)}")
                    dst.copy_(sd[k])
        return missing


class _HeadOwnerView:
    """Adapts a unit owner to the head+loss function (which writes the head gradient during forward)."""

    def __init__(self, owner, tied: bool = False):
        self._o, self._tied = owner, tied

    def acquire_params(self, backward: bool = False):
        return self._o.acquire_params()

    def release_params(self, after_forward: bool):
        self._o.release_params(after_forward)

    def acquire_grads(self):
        return self._o.acquire_grads()

    def grads_ready(self):
        # with tied embeddings the shared unit is finished by the embedding's backward, which runs last
        if not self._tied:
            self._o.grads_ready()
