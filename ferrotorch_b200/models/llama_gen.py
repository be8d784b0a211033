"""Generation utilities for causal LMs: KV-cached incremental forward (any device), sampling strategies (greedy, temperature,
top-k, top-p, repetition penalty), streaming, beam search, speculative decoding, 4-bit checkpoint loaders (GPTQ / AWQ / HQQ)
and the GGUF -> HF tensor-name remap.

Reference parity: ferrotorch-llama/src/{kv_cache.rs:37-207, generation.rs:20-404, spec_decode.rs:42-264, quant_loaders.rs:34-406,
gguf_remap.rs:23-66, model.rs:284 (forward_one_with_cache)}.
"""
from __future__ import annotations

import math
import re
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..errors import InvalidArgument
from .llama import LlamaConfig


# ----------------------------------------------------------------------------------------------------------------------
# KV cache + incremental forward over an HF-named weight dict
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class LayerKvCache:
    k: Optional[torch.Tensor] = None      # [B, Hkv, T, D]
    v: Optional[torch.Tensor] = None

    def append(self, k_new: torch.Tensor, v_new: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        self.k = k_new if self.k is None else torch.cat([self.k, k_new], 2)
        self.v = v_new if self.v is None else torch.cat([self.v, v_new], 2)
        return self.k, self.v

    def len(self) -> int:  # noqa: A003
        return 0 if self.k is None else self.k.shape[2]

    def truncate(self, n: int) -> None:
        if self.k is not None:
            self.k, self.v = self.k[:, :, :n], self.v[:, :, :n]


class KvCache:
    def __init__(self, num_layers: int):
        self.layers = [LayerKvCache() for _ in range(num_layers)]

    def len(self) -> int:  # noqa: A003
        return self.layers[0].len()

    def truncate(self, n: int) -> None:
        for l in self.layers:
            l.truncate(n)

    def clone(self) -> "KvCache":
        c = KvCache(len(self.layers))
        for a, b in zip(c.layers, self.layers):
            a.k, a.v = (None if b.k is None else b.k.clone()), (None if b.v is None else b.v.clone())
        return c


class CachedLlama:
    """Incremental decoder over HF-named weights: ``logits = model(ids_new, cache)`` appends to the cache and returns the logits of
    the new positions. Works on any device in the weights' dtype (f32 math for norms / softmax)."""

    def __init__(self, cfg: LlamaConfig, weights: Dict[str, torch.Tensor]):
        self.cfg, self.W = cfg, weights
        dev = weights["model.embed_tokens.weight"].device
        self.cos, self.sin = ops.rope_tables(cfg.max_position_embeddings, cfg.head_dim, cfg.rope_theta, dev, cfg.rope_scaling)

    def new_cache(self) -> KvCache:
        return KvCache(self.cfg.num_hidden_layers)

    def _rms(self, v, w):
        vf = v.float()
        return (vf * torch.rsqrt(vf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps) * w.float()).to(v.dtype)

    def _rot(self, t, pos0):
        S, D = t.shape[1], self.cfg.head_dim
        c, s = self.cos[pos0: pos0 + S].view(1, S, 1, -1), self.sin[pos0: pos0 + S].view(1, S, 1, -1)
        a, b = t[..., : D // 2].float(), t[..., D // 2:].float()
        return torch.cat([a * c - b * s, b * c + a * s], -1).to(t.dtype)

    @torch.no_grad()
    def __call__(self, ids: torch.Tensor, cache: KvCache) -> torch.Tensor:
        cfg, W = self.cfg, self.W
        B, S = ids.shape
        D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        pos0 = cache.len()
        x = W["model.embed_tokens.weight"][ids]
        for i in range(cfg.num_hidden_layers):
            p = f"model.layers.{i}."
            h = self._rms(x, W[p + "input_layernorm.weight"])
            q = self._rot(F.linear(h, W[p + "self_attn.q_proj.weight"]).view(B, S, Hq, D), pos0).transpose(1, 2)
            k = self._rot(F.linear(h, W[p + "self_attn.k_proj.weight"]).view(B, S, Hkv, D), pos0).transpose(1, 2)
            v = F.linear(h, W[p + "self_attn.v_proj.weight"]).view(B, S, Hkv, D).transpose(1, 2)
            kk, vv = cache.layers[i].append(k, v)
            rep = Hq // Hkv
            sc = torch.matmul(q.float(), kk.repeat_interleave(rep, 1).float().transpose(-1, -2)) / math.sqrt(D)
            T = kk.shape[2]
            mask = torch.ones(S, T, dtype=torch.bool, device=ids.device).triu(T - S + 1)
            sc = sc.masked_fill(mask, float("-inf"))
            a = torch.matmul(torch.softmax(sc, -1), vv.repeat_interleave(rep, 1).float()).to(x.dtype)
            x = x + F.linear(a.transpose(1, 2).reshape(B, S, Hq * D), W[p + "self_attn.o_proj.weight"])
            h2 = self._rms(x, W[p + "post_attention_layernorm.weight"])
            x = x + F.linear(F.silu(F.linear(h2, W[p + "mlp.gate_proj.weight"])) * F.linear(h2, W[p + "mlp.up_proj.weight"]), W[p + "mlp.down_proj.weight"])
        head = W["model.embed_tokens.weight"] if cfg.tie_word_embeddings else W["lm_head.weight"]
        return F.linear(self._rms(x, W["model.norm.weight"]), head).float()


# ----------------------------------------------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class GenerationConfig:
    max_new_tokens: int = 64
    do_sample: bool = False
    temperature: float = 1.0
    top_k: int = 0
    top_p: float = 1.0
    repetition_penalty: float = 1.0
    eos_token_id: Optional[int] = None
    seed: Optional[int] = None
    num_beams: int = 1
    length_penalty: float = 1.0

    def with_temperature(self, t): self.temperature, self.do_sample = t, True; return self
    def with_top_k(self, k): self.top_k, self.do_sample = k, True; return self
    def with_top_p(self, p): self.top_p, self.do_sample = p, True; return self
    def with_max_new_tokens(self, n): self.max_new_tokens = n; return self


def apply_repetition_penalty(logits: torch.Tensor, seq: torch.Tensor, penalty: float) -> torch.Tensor:
    if penalty == 1.0:
        return logits
    g = logits.gather(1, seq)
    return logits.scatter(1, seq, torch.where(g > 0, g / penalty, g * penalty))


def top_k_filter(logits: torch.Tensor, k: int) -> torch.Tensor:
    if k <= 0 or k >= logits.shape[-1]:
        return logits
    kth = logits.topk(k, -1).values[..., -1:]
    return logits.masked_fill(logits < kth, float("-inf"))


def top_p_filter(logits: torch.Tensor, p: float) -> torch.Tensor:
    if p >= 1.0:
        return logits
    sl, si = logits.sort(-1, descending=True)
    cp = sl.softmax(-1).cumsum(-1)
    drop = cp - sl.softmax(-1) > p          # keep the smallest prefix whose mass reaches p (always at least one token)
    sl = sl.masked_fill(drop, float("-inf"))
    return torch.full_like(logits, float("-inf")).scatter(-1, si, sl)


def sample_next(logits: torch.Tensor, seq: torch.Tensor, cfg: GenerationConfig, gen: Optional[torch.Generator] = None) -> torch.Tensor:
    logits = apply_repetition_penalty(logits, seq, cfg.repetition_penalty)
    if not cfg.do_sample:
        return logits.argmax(-1)
    logits = top_p_filter(top_k_filter(logits / max(cfg.temperature, 1e-6), cfg.top_k), cfg.top_p)
    return torch.multinomial(logits.softmax(-1), 1, generator=gen).squeeze(-1)


@torch.no_grad()
def generate(model: Callable[[torch.Tensor, KvCache], torch.Tensor], new_cache: Callable[[], KvCache], ids: torch.Tensor,
             cfg: Optional[GenerationConfig] = None, streamer: Optional[Callable[[torch.Tensor], None]] = None,
             logits_processor: Optional[Callable[[torch.Tensor, torch.Tensor], torch.Tensor]] = None) -> torch.Tensor:
    """Autoregressive generation with a KV cache; returns ``[B, S + new]``. ``streamer(tokens)`` is called with each new token batch;
    ``logits_processor(logits, seq)`` can constrain decoding (e.g. :class:`ferrotorch_b200.grammar.JsonSchemaProcessor`)."""
    cfg = cfg or GenerationConfig()
    if cfg.num_beams > 1:
        return beam_search(model, new_cache, ids, cfg)
    gen = None
    if cfg.seed is not None:
        gen = torch.Generator(device=ids.device).manual_seed(cfg.seed)
    cache = new_cache()
    seq = ids
    logits = model(ids, cache)[:, -1]
    done = torch.zeros(ids.shape[0], dtype=torch.bool, device=ids.device)
    for _ in range(cfg.max_new_tokens):
        if logits_processor is not None:
            logits = logits_processor(logits, seq)
        nxt = sample_next(logits, seq, cfg, gen)
        if cfg.eos_token_id is not None:
            nxt = torch.where(done, torch.full_like(nxt, cfg.eos_token_id), nxt)
            done |= nxt == cfg.eos_token_id
        seq = torch.cat([seq, nxt[:, None]], 1)
        if streamer is not None:
            streamer(nxt)
        if cfg.eos_token_id is not None and bool(done.all()):
            break
        logits = model(nxt[:, None], cache)[:, -1]
    return seq


@torch.no_grad()
def beam_search(model, new_cache, ids: torch.Tensor, cfg: GenerationConfig) -> torch.Tensor:
    """Beam search for batch size 1 (the beams are the batch dimension of the cached forward); returns the best sequence ``[1, S+new]``."""
    if ids.shape[0] != 1:
        raise InvalidArgument("beam search takes a single prompt")
    nb = cfg.num_beams
    cache = new_cache()
    logp = model(ids, cache)[:, -1].log_softmax(-1)
    top = logp.topk(nb, -1)
    seqs = torch.cat([ids.repeat(nb, 1), top.indices.view(nb, 1)], 1)
    scores = top.values.view(nb)
    for l in cache.layers:
        l.k, l.v = l.k.repeat(nb, 1, 1, 1), l.v.repeat(nb, 1, 1, 1)
    finished: List[Tuple[float, torch.Tensor]] = []
    for step in range(1, cfg.max_new_tokens):
        logp = model(seqs[:, -1:], cache)[:, -1].log_softmax(-1)
        cand = (scores[:, None] + logp).view(-1)
        top = cand.topk(nb)
        beam, tok = top.indices // logp.shape[-1], top.indices % logp.shape[-1]
        seqs = torch.cat([seqs[beam], tok[:, None]], 1)
        scores = top.values
        for l in cache.layers:
            l.k, l.v = l.k[beam], l.v[beam]
        if cfg.eos_token_id is not None:
            ended = tok == cfg.eos_token_id
            for b in torch.where(ended)[0].tolist():
                finished.append((float(scores[b]) / (seqs.shape[1] - ids.shape[1]) ** cfg.length_penalty, seqs[b].clone()))
                scores[b] = float("-inf")
            if len(finished) >= nb:
                break
    for b in range(nb):
        if scores[b] > float("-inf"):
            finished.append((float(scores[b]) / (seqs.shape[1] - ids.shape[1]) ** cfg.length_penalty, seqs[b]))
    return max(finished, key=lambda t: t[0])[1][None]


# ----------------------------------------------------------------------------------------------------------------------
# speculative decoding
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class SpecDecodeConfig:
    num_draft_tokens: int = 4
    max_new_tokens: int = 64
    eos_token_id: Optional[int] = None


@dataclass
class SpecDecodeStats:
    proposed: int = 0
    accepted: int = 0

    def acceptance_rate(self) -> float:
        return self.accepted / max(self.proposed, 1)


@torch.no_grad()
def speculative_generate(target, target_cache_fn, draft, draft_cache_fn, ids: torch.Tensor, cfg: Optional[SpecDecodeConfig] = None):
    """Greedy speculative decoding (batch 1): the draft proposes ``k`` tokens, the target scores them in one forward, the longest
    agreeing prefix is accepted plus the target's own next token. The output equals plain greedy decoding with the target."""
    cfg = cfg or SpecDecodeConfig()
    if ids.shape[0] != 1:
        raise InvalidArgument("speculative decoding takes a single prompt")
    tc, dc = target_cache_fn(), draft_cache_fn()
    stats = SpecDecodeStats()
    seq = ids
    t_logits = target(ids, tc)[:, -1]
    draft(ids, dc)
    produced = 0
    while produced < cfg.max_new_tokens:
        nxt = t_logits.argmax(-1)                                   # the target's token at the current position
        seq = torch.cat([seq, nxt[:, None]], 1)
        produced += 1
        if cfg.eos_token_id is not None and int(nxt) == cfg.eos_token_id or produced >= cfg.max_new_tokens:
            break
        # draft proposes k tokens after `nxt`
        base = seq.shape[1]
        d_in, prop = nxt[:, None], []
        for _ in range(cfg.num_draft_tokens):
            d_tok = draft(d_in, dc)[:, -1].argmax(-1)
            prop.append(d_tok)
            d_in = d_tok[:, None]
        prop_t = torch.stack(prop, 1)                                # [1, k]
        stats.proposed += prop_t.shape[1]
        ver = target(torch.cat([nxt[:, None], prop_t], 1), tc)      # logits after nxt, p1, ..., pk
        tgt = ver.argmax(-1)                                         # target's choice following each of them
        n_ok = 0
        while n_ok < prop_t.shape[1] and int(tgt[0, n_ok]) == int(prop_t[0, n_ok]):
            n_ok += 1
        stats.accepted += n_ok
        take = min(n_ok, cfg.max_new_tokens - produced)
        if take:
            seq = torch.cat([seq, prop_t[:, :take]], 1)
            produced += take
        t_logits = ver[:, take]                                      # logits following the last accepted token
        tc.truncate(base + take)                                     # drop cache entries of rejected proposals
        dc.truncate(base + take - 1 if take == prop_t.shape[1] else base + take)
        if dc.len() < base + take:                                   # the draft has not seen the last accepted token yet
            draft(seq[:, dc.len():], dc)
        if cfg.eos_token_id is not None and take and (seq[0, -take:] == cfg.eos_token_id).any():
            break
    return seq, stats


# ----------------------------------------------------------------------------------------------------------------------
# 4-bit checkpoint loaders
# ----------------------------------------------------------------------------------------------------------------------
def _unpack_int4(packed: torch.Tensor, dim: int) -> torch.Tensor:
    """int32 words holding eight 4-bit values (LSB first) along ``dim`` -> uint8 tensor eight times longer on ``dim``."""
    shifts = torch.arange(0, 32, 4, device=packed.device, dtype=torch.int32)
    p = packed.to(torch.int32).unsqueeze(dim + 1)
    shape = [1] * p.dim()
    shape[dim + 1] = 8
    vals = (p >> shifts.view(shape)) & 0xF
    out_shape = list(packed.shape)
    out_shape[dim] *= 8
    return vals.reshape(out_shape).to(torch.uint8)


def dequantize_gptq_q4(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, g_idx: Optional[torch.Tensor] = None,
                       group_size: int = 128) -> torch.Tensor:
    """GPTQ 4-bit: ``qweight`` int32 ``[in/8, out]``, ``qzeros`` int32 ``[groups, out/8]``, ``scales`` ``[groups, out]`` -> weight ``[out, in]``.
    The stored zero is one less than the actual zero point (AutoGPTQ convention)."""
    w = _unpack_int4(qweight, 0).float()                             # [in, out]
    z = _unpack_int4(qzeros, 1).float() + 1.0                        # [groups, out]
    gi = g_idx.long() if g_idx is not None else torch.arange(w.shape[0], device=w.device) // group_size
    return ((w - z[gi]) * scales.float()[gi]).t().contiguous()


_AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]


def dequantize_awq_q4(qweight: torch.Tensor, qzeros: torch.Tensor, scales: torch.Tensor, group_size: int = 128) -> torch.Tensor:
    """AWQ 4-bit (GEMM layout): ``qweight`` int32 ``[in, out/8]``. Output channel ``c`` of a word sits in nibble ``[0, 4, 1, 5, 2, 6, 3, 7][c]``
    (AutoAWQ packs the channels of a word in the order 0, 2, 4, 6, 1, 3, 5, 7; ferrotorch-llama/src/quant_loaders.rs:244-331 reads them back the
    same way)."""
    order = torch.tensor(_AWQ_ORDER, device=qweight.device)
    w = _unpack_int4(qweight, 1).view(qweight.shape[0], -1, 8)[:, :, order].reshape(qweight.shape[0], -1).float()
    z = _unpack_int4(qzeros, 1).view(qzeros.shape[0], -1, 8)[:, :, order].reshape(qzeros.shape[0], -1).float()
    gi = torch.arange(w.shape[0], device=w.device) // group_size
    return ((w - z[gi]) * scales.float()[gi]).t().contiguous()


def dequantize_hqq(w_q: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor, shape: Sequence[int], nbits: int = 4, group_size: int = 64) -> torch.Tensor:
    """HQQ: ``w_q`` uint8 with two 4-bit values per byte (first half of the rows in the high nibble), per-group ``scale``/``zero``."""
    if nbits == 4:
        hi, lo = (w_q >> 4) & 0xF, w_q & 0xF
        q = torch.cat([hi, lo], 0).float()
    elif nbits == 8:
        q = w_q.float()
    else:
        raise InvalidArgument("HQQ loader supports 4 and 8 bits")
    return ((q - zero.float()) * scale.float()).reshape(tuple(shape))


def load_quantized_linear_weights(sd: Dict[str, torch.Tensor], prefix: str, method: str, group_size: int = 128) -> torch.Tensor:
    if method == "gptq":
        return dequantize_gptq_q4(sd[prefix + "qweight"], sd[prefix + "qzeros"], sd[prefix + "scales"], sd.get(prefix + "g_idx"), group_size)
    if method == "awq":
        return dequantize_awq_q4(sd[prefix + "qweight"], sd[prefix + "qzeros"], sd[prefix + "scales"], group_size)
    raise InvalidArgument(f"unknown quantisation method {method}")


# ----------------------------------------------------------------------------------------------------------------------
# GGUF -> HF names
# ----------------------------------------------------------------------------------------------------------------------
_GGUF_MAP = {"attn_q": "self_attn.q_proj", "attn_k": "self_attn.k_proj", "attn_v": "self_attn.v_proj", "attn_output": "self_attn.o_proj",
             "ffn_gate": "mlp.gate_proj", "ffn_up": "mlp.up_proj", "ffn_down": "mlp.down_proj", "attn_norm": "input_layernorm",
             "ffn_norm": "post_attention_layernorm"}


def gguf_to_hf_name(name: str) -> Optional[str]:
    if name == "token_embd.weight":
        return "model.embed_tokens.weight"
    if name == "output_norm.weight":
        return "model.norm.weight"
    if name == "output.weight":
        return "lm_head.weight"
    m = re.match(r"blk\.(\d+)\.(\w+)\.(weight|bias)$", name)
    if m and m.group(2) in _GGUF_MAP:
        return f"model.layers.{m.group(1)}.{_GGUF_MAP[m.group(2)]}.{m.group(3)}"
    return None


def gguf_unpermute_qk(w: torch.Tensor, n_heads: int) -> torch.Tensor:
    """llama.cpp stores q/k projections with the interleaved rotary layout; this restores the HF half-rotation row order."""
    out, d = w.shape
    return w.view(n_heads, out // n_heads // 2, 2, d).transpose(1, 2).reshape(out, d)


def remap_gguf_state_dict(tensors: Dict[str, torch.Tensor], cfg: LlamaConfig) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in tensors.items():
        hf = gguf_to_hf_name(k)
        if hf is None:
            continue
        if hf.endswith("q_proj.weight"):
            v = gguf_unpermute_qk(v, cfg.num_attention_heads)
        elif hf.endswith("k_proj.weight"):
            v = gguf_unpermute_qk(v, cfg.num_key_value_heads)
        out[hf] = v
    return out
