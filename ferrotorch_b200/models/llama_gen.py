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
from ..errors import InvalidArgument, ShapeMismatch
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
        self.act = cfg.activation
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
            x = x + F.linear(self.act(F.linear(h2, W[p + "mlp.gate_proj.weight"])) * F.linear(h2, W[p + "mlp.up_proj.weight"]), W[p + "mlp.down_proj.weight"])
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
    eos_token_ids: List[int] = field(default_factory=list)        # several stop tokens (Llama 3: 128001 and 128009)

    @classmethod
    def greedy(cls, max_new_tokens: int) -> "GenerationConfig":
        """ferrotorch-llama/src/generation.rs:67."""
        return cls(max_new_tokens=max_new_tokens, do_sample=False, temperature=0.0)

    @classmethod
    def sampling(cls, max_new_tokens: int, temperature: float) -> "GenerationConfig":
        return cls(max_new_tokens=max_new_tokens, do_sample=temperature > 0.0, temperature=temperature)

    @classmethod
    def nucleus(cls, max_new_tokens: int, top_p: float, temperature: float) -> "GenerationConfig":
        return cls(max_new_tokens=max_new_tokens, do_sample=temperature > 0.0, temperature=temperature, top_p=top_p)

    def stop_ids(self) -> List[int]:
        return list(self.eos_token_ids) + ([self.eos_token_id] if self.eos_token_id is not None else [])

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


def apply_temperature(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """``logits / temperature`` (ferrotorch-llama/src/generation.rs:238)."""
    return logits * (1.0 / temperature)


def argmax(logits) -> int:
    """Index of the largest logit of one row, the first one on ties (generation.rs:311)."""
    t = torch.as_tensor(logits).reshape(-1)
    return int((t == t.max()).nonzero()[0]) if t.numel() and not bool(torch.isnan(t.max())) else 0


class XorShift64:
    """The 13 / 7 / 17 xorshift generator that drives the reference's samplers (generation.rs:581, spec_decode.rs:497); a run with the same
    seed draws the same uniforms in the same order."""
    DEFAULT_SEED = 0xDEADBEEFCAFEBABE
    _M = (1 << 64) - 1

    def __init__(self, seed: Optional[int] = None):
        self.state = (self.DEFAULT_SEED if seed is None else int(seed)) & self._M
        if self.state == 0:
            raise InvalidArgument("XorShift64: the seed must be non-zero")

    def next_u64(self) -> int:
        x = self.state
        x ^= (x << 13) & self._M
        x ^= x >> 7
        x ^= (x << 17) & self._M
        self.state = x
        return x

    def uniform(self) -> float:
        return self.next_u64() / float(self._M)


def _softmax64(logits) -> torch.Tensor:
    t = torch.as_tensor(logits).reshape(-1).to(torch.float64)
    m = t.max()
    if not bool(torch.isfinite(m)):
        return torch.zeros_like(t)
    e = (t - m).exp()
    return e / e.sum()


def _sample_weights(w: torch.Tensor, rng: XorShift64, fallback) -> int:
    total = float(w.sum())
    if not (total > 0.0 and math.isfinite(total)):
        return fallback()
    u = rng.uniform() * total
    return min(int(torch.searchsorted(w.cumsum(0), torch.tensor(u, dtype=w.dtype))), w.numel() - 1)      # first i with u <= cum[i]


def sample_softmax(logits, rng: XorShift64) -> int:
    """One draw from ``softmax(logits)`` by inverse CDF in f64; when every logit is ``-inf`` the argmax is returned (generation.rs:324)."""
    return _sample_weights(_softmax64(logits), rng, lambda: argmax(logits))


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
    stops = cfg.stop_ids()
    stop_t = torch.tensor(stops, dtype=torch.long, device=ids.device)
    for _ in range(cfg.max_new_tokens):
        if logits_processor is not None:
            logits = logits_processor(logits, seq)
        nxt = sample_next(logits, seq, cfg, gen)
        if stops:
            nxt = torch.where(done, torch.full_like(nxt, stops[0]), nxt)
            done |= torch.isin(nxt, stop_t)
        seq = torch.cat([seq, nxt[:, None]], 1)
        if streamer is not None:
            streamer(nxt)
        if stops and bool(done.all()):
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


@torch.no_grad()
def generate_with_streamer(model, prompt_ids: Sequence[int], config: GenerationConfig, streamer: Callable[[int], bool],
                           new_cache: Optional[Callable[[], "KvCache"]] = None) -> List[int]:
    """Single-prompt generation in the reference's form (ferrotorch-llama/src/generation.rs:145-232): returns the new tokens only, the stop
    token included; ``streamer(token)`` sees every token as it is chosen and ends the run by returning ``False``. ``temperature == 0`` is greedy;
    otherwise repetition penalty, temperature, top-k, top-p, then an inverse-CDF draw in f64 from :class:`XorShift64` seeded by
    ``config.seed``, so a (prompt, config) pair always gives the same tokens. ``model(ids, cache)`` returns ``[1, S, vocab]`` logits and keeps
    its KV cache, so each step feeds one token instead of the whole prefix."""
    if len(prompt_ids) == 0:
        raise InvalidArgument("generate: prompt_ids must not be empty")
    if config.temperature < 0.0:
        raise InvalidArgument(f"generate: temperature must be >= 0, got {config.temperature}")
    if not 0.0 <= config.top_p <= 1.0:
        raise InvalidArgument(f"generate: top_p must be in [0, 1], got {config.top_p}")
    if config.repetition_penalty <= 0.0:
        raise InvalidArgument(f"generate: repetition_penalty must be > 0, got {config.repetition_penalty}")
    cache = (new_cache or model.new_cache)()
    dev = getattr(model, "W", {}).get("model.embed_tokens.weight").device if hasattr(model, "W") else "cpu"
    rng = XorShift64(config.seed)
    ids, produced, stops = list(int(t) for t in prompt_ids), [], set(config.stop_ids())
    feed = ids
    greedy = config.temperature == 0.0 or not config.do_sample
    for _ in range(config.max_new_tokens):
        out = model(torch.tensor([feed], dtype=torch.long, device=dev), cache)
        if out.dim() != 3:
            raise InvalidArgument(f"generate: expected logits shape [1, S, V], got {list(out.shape)}")
        logits = out[0, -1].to(torch.float64).cpu()
        if abs(config.repetition_penalty - 1.0) > 2.3e-16:
            seen = torch.tensor([t for t in set(ids) if t < logits.numel()], dtype=torch.long)
            g = logits[seen]
            logits[seen] = torch.where(g > 0, g / config.repetition_penalty, g * config.repetition_penalty)
        if greedy:
            nxt = argmax(logits)
        else:
            logits = apply_temperature(logits, config.temperature)
            logits = top_p_filter(top_k_filter(logits[None], config.top_k), config.top_p)[0]
            nxt = sample_softmax(logits, rng)
        produced.append(nxt)
        if not streamer(nxt) or nxt in stops:
            break
        ids.append(nxt)
        feed = [nxt]
    return produced


# ----------------------------------------------------------------------------------------------------------------------
# speculative decoding
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class SpecDecodeConfig:
    num_draft_tokens: int = 4
    max_new_tokens: int = 64
    eos_token_id: Optional[int] = None
    draft_k: Optional[int] = None                                  # the reference's name for ``num_draft_tokens`` (spec_decode.rs:167)
    seed: Optional[int] = None
    eos_token_ids: List[int] = field(default_factory=list)

    def __post_init__(self):
        if self.draft_k is None:
            self.draft_k = self.num_draft_tokens
        else:
            self.num_draft_tokens = self.draft_k

    def validate(self) -> None:
        if self.draft_k < 1:
            raise InvalidArgument("SpecDecodeConfig: draft_k must be >= 1")
        if self.max_new_tokens < 1:
            raise InvalidArgument("SpecDecodeConfig: max_new_tokens must be >= 1")

    def stop_ids(self) -> List[int]:
        return list(self.eos_token_ids) + ([self.eos_token_id] if self.eos_token_id is not None else [])


@dataclass
class SpecDecodeOutput:
    """New tokens (prompt excluded) and the draft-token bookkeeping of one run (spec_decode.rs:218)."""
    tokens: List[int]
    accepted_count: int
    proposed_count: int

    def acceptance_rate(self) -> float:
        return 1.0 if self.proposed_count == 0 else self.accepted_count / self.proposed_count


class ModelHandle:
    """What speculative decoding needs from a model (spec_decode.rs:42): last-position logits for a token list, per-position logits for the
    verify pass (the default loops over prefixes; real handles override it with one forward), and the vocabulary size."""

    def forward_ids(self, ids: Sequence[int]) -> torch.Tensor:
        raise NotImplementedError

    def forward_ids_all_positions(self, ids: Sequence[int]) -> torch.Tensor:
        return torch.stack([self.forward_ids(ids[:j]) for j in range(1, len(ids) + 1)])

    def vocab_size(self) -> int:
        raise NotImplementedError


class LlamaHandle(ModelHandle):
    """:class:`ModelHandle` over a cached decoder ``model(ids, cache) -> [1, S, vocab]`` (spec_decode.rs:101). ``forward_ids`` keeps one KV cache
    and re-feeds only the tokens after the longest prefix it has already seen, so drafting K tokens costs K single-token steps."""

    def __init__(self, model, new_cache: Optional[Callable[[], "KvCache"]] = None, vocab_size: Optional[int] = None):
        self.model, self._new_cache = model, new_cache or model.new_cache
        self._vocab = vocab_size if vocab_size is not None else model.cfg.vocab_size
        self._dev = model.W["model.embed_tokens.weight"].device if hasattr(model, "W") else "cpu"
        self._seen: List[int] = []
        self._cache = None

    def vocab_size(self) -> int:
        return self._vocab

    @torch.no_grad()
    def forward_ids(self, ids: Sequence[int]) -> torch.Tensor:
        ids = [int(t) for t in ids]
        n = 0
        if self._cache is not None:
            while n < min(len(ids) - 1, len(self._seen)) and ids[n] == self._seen[n]:
                n += 1
        if self._cache is None or n == 0:
            self._cache, n = self._new_cache(), 0
        else:
            self._cache.truncate(n)
        out = self.model(torch.tensor([ids[n:]], dtype=torch.long, device=self._dev), self._cache)
        self._seen = ids
        return out[0, -1].to(torch.float64).cpu()

    @torch.no_grad()
    def forward_ids_all_positions(self, ids: Sequence[int]) -> torch.Tensor:
        out = self.model(torch.tensor([[int(t) for t in ids]], dtype=torch.long, device=self._dev), self._new_cache())
        return out[0].to(torch.float64).cpu()


@torch.no_grad()
def speculative_decode(draft: ModelHandle, target: ModelHandle, prompt_ids: Sequence[int], config: Optional[SpecDecodeConfig] = None) -> SpecDecodeOutput:
    """Speculative sampling (Leviathan et al. 2023, Algorithm 1) as in ferrotorch-llama/src/spec_decode.rs:264-420: the draft samples ``K``
    tokens from its own distributions ``q``; one target forward over ``context + draft`` gives ``p`` at the ``K + 1`` positions; token ``j`` is
    kept with probability ``min(1, p_j / q_j)``; the first rejected position is redrawn from ``norm(max(0, p - q))``; if all are kept a bonus
    token is drawn from ``p_K``. The emitted tokens are distributed exactly as samples from the target alone. All draws come from one
    :class:`XorShift64` (``config.seed``), in the reference's order."""
    config = config or SpecDecodeConfig()
    if len(prompt_ids) == 0:
        raise InvalidArgument("speculative_decode: prompt_ids must not be empty")
    config.validate()
    vocab = draft.vocab_size()
    if target.vocab_size() != vocab:
        raise InvalidArgument(f"speculative_decode: draft vocab_size ({vocab}) != target vocab_size ({target.vocab_size()})")
    rng = XorShift64(config.seed)
    stops = set(config.stop_ids())
    context, produced = [int(t) for t in prompt_ids], []
    accepted = proposed = 0
    pick = lambda w: _sample_weights(w, rng, lambda: argmax(w))
    while len(produced) < config.max_new_tokens:
        k = min(config.draft_k, config.max_new_tokens - len(produced))
        d_tok, d_prob, ctx = [], [], list(context)
        for _ in range(k):
            q = _softmax64(draft.forward_ids(ctx))
            t = pick(q)
            d_tok.append(t)
            d_prob.append(q)
            ctx.append(t)
        rows = target.forward_ids_all_positions(context + d_tok)
        if rows.shape[0] != len(context) + k:
            raise InvalidArgument(f"speculative_decode: forward_ids_all_positions returned {rows.shape[0]} rows for input length {len(context) + k}")
        t_prob = [_softmax64(rows[len(context) - 1 + j]) for j in range(k + 1)]
        proposed += k
        n_ok, corrected = 0, None
        for j in range(k):
            q, p = float(d_prob[j][d_tok[j]]), float(t_prob[j][d_tok[j]])
            if rng.uniform() < (0.0 if q <= 0.0 else min(p / q, 1.0)):
                n_ok += 1
            else:
                resid = (t_prob[j] - d_prob[j]).clamp_min(0.0)
                corrected = _sample_weights(resid, rng, lambda: pick(t_prob[j]))
                break
        accepted += n_ok
        stop = False
        for t in d_tok[:n_ok]:
            produced.append(t)
            context.append(t)
            if t in stops or len(produced) >= config.max_new_tokens:
                stop = True
                break
        if stop:
            break
        extra = corrected if corrected is not None else pick(t_prob[k])
        produced.append(extra)
        context.append(extra)
        if extra in stops:
            break
    return SpecDecodeOutput(produced[: config.max_new_tokens], accepted, proposed)


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


@dataclass
class GptqQ4:
    """One GPTQ 4-bit linear weight as stored in a checkpoint (ferrotorch-llama/src/quant_loaders.rs:34): ``qweight`` int32 ``[K/8, N]``,
    ``qzeros`` int32 ``[K/G, N/8]``, ``scales`` ``[K/G, N]``, optional ``g_idx`` ``[K]`` (``act_order``)."""
    qweight: torch.Tensor
    qzeros: torch.Tensor
    scales: torch.Tensor
    g_idx: Optional[torch.Tensor]
    in_features: int
    out_features: int
    group_size: int


@dataclass
class AwqQ4:
    """One AWQ 4-bit linear weight (GEMM layout; quant_loaders.rs:203): ``qweight`` int32 ``[K, N/8]``, ``qzeros`` int32 ``[K/G, N/8]``,
    ``scales`` ``[K/G, N]``."""
    qweight: torch.Tensor
    qzeros: torch.Tensor
    scales: torch.Tensor
    in_features: int
    out_features: int
    group_size: int


@dataclass
class HqqWeights:
    """One HQQ weight (quant_loaders.rs:355): packed ``w_q`` bytes, per-group ``scale`` / ``zero``, and the dense shape."""
    bits: int
    w_q: torch.Tensor
    scale: torch.Tensor
    zero: torch.Tensor
    out_features: int
    in_features: int


def _check_q4(name: str, K: int, N: int, G: int, shapes) -> None:
    if K % 8 or N % 8:
        raise InvalidArgument(f"{name}: in_features ({K}) and out_features ({N}) must be multiples of 8")
    if G <= 0 or K % G:
        raise InvalidArgument(f"{name}: in_features ({K}) must be divisible by group_size ({G})")
    for what, t, want in shapes:
        if t.numel() != want:
            raise InvalidArgument(f"{name}: {what} has {t.numel()} elements, expected {want}")


def dequantize_gptq_q4(qweight, qzeros: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None, g_idx: Optional[torch.Tensor] = None,
                       group_size: int = 128) -> torch.Tensor:
    """Also takes one :class:`GptqQ4` (buffers may be flat; sizes are checked as in quant_loaders.rs:90-120).

    GPTQ 4-bit: ``qweight`` int32 ``[in/8, out]``, ``qzeros`` int32 ``[groups, out/8]``, ``scales`` ``[groups, out]`` -> weight ``[out, in]``.
    The stored zero is one less than the actual zero point (AutoGPTQ convention)."""
    if isinstance(qweight, GptqQ4):
        t = qweight
        K, N, G = t.in_features, t.out_features, t.group_size
        _check_q4("dequantize_gptq_q4", K, N, G, (("qweight", t.qweight, K // 8 * N), ("qzeros", t.qzeros, K // max(G, 1) * (N // 8)),
                                                    ("scales", t.scales, K // max(G, 1) * N)))
        if t.g_idx is not None and t.g_idx.numel() != K:
            raise InvalidArgument(f"dequantize_gptq_q4: g_idx has {t.g_idx.numel()} elements, expected {K}")
        return dequantize_gptq_q4(t.qweight.reshape(K // 8, N), t.qzeros.reshape(K // G, N // 8), t.scales.reshape(K // G, N), t.g_idx, G)
    w = _unpack_int4(qweight, 0).float()                             # [in, out]
    z = _unpack_int4(qzeros, 1).float() + 1.0                        # [groups, out]
    gi = g_idx.long() if g_idx is not None else torch.arange(w.shape[0], device=w.device) // group_size
    return ((w - z[gi]) * scales.float()[gi]).t().contiguous()


_AWQ_ORDER = [0, 4, 1, 5, 2, 6, 3, 7]


def dequantize_awq_q4(qweight, qzeros: Optional[torch.Tensor] = None, scales: Optional[torch.Tensor] = None, group_size: int = 128) -> torch.Tensor:
    """Also takes one :class:`AwqQ4`. AWQ 4-bit (GEMM layout): ``qweight`` int32 ``[in, out/8]``. Output channel ``c`` of a word sits in nibble ``[0, 4, 1, 5, 2, 6, 3, 7][c]``
    (AutoAWQ packs the channels of a word in the order 0, 2, 4, 6, 1, 3, 5, 7; ferrotorch-llama/src/quant_loaders.rs:244-331 reads them back the
    same way)."""
    if isinstance(qweight, AwqQ4):
        t = qweight
        K, N, G = t.in_features, t.out_features, t.group_size
        _check_q4("dequantize_awq_q4", K, N, G, (("qweight", t.qweight, K * (N // 8)), ("qzeros", t.qzeros, K // max(G, 1) * (N // 8)),
                                                   ("scales", t.scales, K // max(G, 1) * N)))
        return dequantize_awq_q4(t.qweight.reshape(K, N // 8), t.qzeros.reshape(K // G, N // 8), t.scales.reshape(K // G, N), G)
    order = torch.tensor(_AWQ_ORDER, device=qweight.device)
    w = _unpack_int4(qweight, 1).view(qweight.shape[0], -1, 8)[:, :, order].reshape(qweight.shape[0], -1).float()
    z = _unpack_int4(qzeros, 1).view(qzeros.shape[0], -1, 8)[:, :, order].reshape(qzeros.shape[0], -1).float()
    gi = torch.arange(w.shape[0], device=w.device) // group_size
    return ((w - z[gi]) * scales.float()[gi]).t().contiguous()


def dequantize_hqq(w_q, scale: Optional[torch.Tensor] = None, zero: Optional[torch.Tensor] = None, shape: Optional[Sequence[int]] = None, nbits: int = 4,
                   group_size: int = 64) -> torch.Tensor:
    """Tensor form: ``w_q`` uint8 with two 4-bit values per byte (first half of the rows in the high nibble), per-group ``scale``/``zero``. One :class:`HqqWeights` argument selects the
    reference's packed form instead (1, 2, 3, 4 or 8 bits)."""
    if isinstance(w_q, HqqWeights):
        # reference form (quant_loaders.rs:335-570): one little-endian bit stream, element i in bits [i*b, i*b + b); scale / zero per output row
        t = w_q
        if t.bits not in (1, 2, 3, 4, 8):
            raise InvalidArgument(f"HQQ: bits must be 1/2/3/4/8, got {t.bits}")
        if t.scale.numel() != t.out_features or t.zero.numel() != t.out_features:
            raise ShapeMismatch(f"HQQ: scale len {t.scale.numel()} / zero len {t.zero.numel()} != out_features {t.out_features}")
        total = t.out_features * t.in_features
        need = -(-total // 8) * 3 if t.bits == 3 else -(-total * t.bits // 8)
        raw = t.w_q.reshape(-1).to(torch.uint8)
        if raw.numel() < need:
            raise ShapeMismatch(f"HQQ {t.bits}-bit: packed buffer too short ({raw.numel()} bytes for {total} weights, need {need})")
        bits = (raw[:need, None] >> torch.arange(8, device=raw.device, dtype=torch.uint8)) & 1
        q = (bits.reshape(-1)[: total * t.bits].reshape(total, t.bits).float() * (2.0 ** torch.arange(t.bits, device=raw.device))).sum(1)
        return (q.view(t.out_features, t.in_features) - t.zero.float().view(-1, 1)) * t.scale.float().view(-1, 1)
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


gguf_key_to_hf = gguf_to_hf_name                                  # the reference's name (ferrotorch-llama/src/gguf_remap.rs:23)


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


gguf_to_hf_state_dict = remap_gguf_state_dict                     # ferrotorch-llama/src/gguf_remap.rs:66
LlamaKvCache = KvCache                                            # ferrotorch-llama/src/kv_cache.rs
