"""Paged KV cache bookkeeping, flex attention, initialisers, gradient utilities, QAT helpers.

Reference parity: ferrotorch-nn/src/paged_attention.rs:59-518, flex_attention.rs:42-755, init.rs:13-457, utils.rs:134-352,
qat.rs:21-170, rnn_utils.rs:20-187, upsample.rs:140-1139.
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass, field
from typing import Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import ops
from ..errors import InvalidArgument
from .module import Module

# ----------------------------------------------------------------------------------------------------------------------
# paged KV cache
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class KVPage:
    index: int
    ref_count: int = 0
    filled: int = 0


class PagePool:
    """Fixed pool of KV pages of ``page_size`` tokens; pages are reference counted so prefixes can be shared."""

    def __init__(self, num_pages: int, page_size: int = 16):
        self.page_size = page_size
        self.pages = [KVPage(i) for i in range(num_pages)]
        self.free: List[int] = list(range(num_pages - 1, -1, -1))

    def allocate(self) -> int:
        if not self.free:
            raise InvalidArgument("KV page pool exhausted")
        i = self.free.pop()
        self.pages[i].ref_count, self.pages[i].filled = 1, 0
        return i

    def retain(self, i: int) -> None:
        self.pages[i].ref_count += 1

    def release(self, i: int) -> None:
        p = self.pages[i]
        p.ref_count -= 1
        if p.ref_count == 0:
            self.free.append(i)

    def num_free(self) -> int:
        return len(self.free)


class PagedKVCache:
    """Device storage ``[num_pages, page_size, kv_heads, head_dim]`` for K and V of one layer plus per-sequence block tables."""

    def __init__(self, pool: PagePool, kv_heads: int, head_dim: int, device="cpu", dtype=torch.float32):
        self.pool = pool
        n, ps = len(pool.pages), pool.page_size
        self.k = torch.zeros(n, ps, kv_heads, head_dim, device=device, dtype=dtype)
        self.v = torch.zeros_like(self.k)
        self.tables: Dict[int, List[int]] = {}
        self.lengths: Dict[int, int] = {}

    def add_sequence(self, seq_id: int) -> None:
        self.tables[seq_id], self.lengths[seq_id] = [], 0

    def free_sequence(self, seq_id: int) -> None:
        for p in self.tables.pop(seq_id, []):
            self.pool.release(p)
        self.lengths.pop(seq_id, None)

    def fork(self, src: int, dst: int) -> None:
        """Share the pages of ``src`` with a new sequence ``dst`` (copy-on-write happens at the page being appended to)."""
        self.tables[dst] = list(self.tables[src])
        self.lengths[dst] = self.lengths[src]
        for p in self.tables[dst]:
            self.pool.retain(p)

    def append(self, seq_id: int, k_new: torch.Tensor, v_new: torch.Tensor) -> None:
        """``k_new`` / ``v_new``: ``[tokens, kv_heads, head_dim]``."""
        ps = self.pool.page_size
        for t in range(k_new.shape[0]):
            pos = self.lengths[seq_id]
            if pos % ps == 0:
                self.tables[seq_id].append(self.pool.allocate())
            page = self.tables[seq_id][-1]
            if self.pool.pages[page].ref_count > 1:      # copy on write
                fresh = self.pool.allocate()
                self.k[fresh].copy_(self.k[page]); self.v[fresh].copy_(self.v[page])
                self.pool.release(page)
                self.tables[seq_id][-1] = page = fresh
            self.k[page, pos % ps] = k_new[t]
            self.v[page, pos % ps] = v_new[t]
            self.pool.pages[page].filled = pos % ps + 1
            self.lengths[seq_id] = pos + 1

    def gather(self, seq_id: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Contiguous ``[len, kv_heads, head_dim]`` views of a sequence (the oracle for the paged decode kernel)."""
        n = self.lengths[seq_id]
        idx = torch.tensor(self.tables[seq_id], device=self.k.device, dtype=torch.long)
        k = self.k[idx].reshape(-1, *self.k.shape[2:])[:n]
        v = self.v[idx].reshape(-1, *self.v.shape[2:])[:n]
        return k, v

    def block_table(self, seq_ids: Sequence[int], max_blocks: Optional[int] = None) -> torch.Tensor:
        mb = max_blocks or max(len(self.tables[s]) for s in seq_ids)
        t = torch.full((len(seq_ids), mb), -1, dtype=torch.int32)
        for i, s in enumerate(seq_ids):
            t[i, : len(self.tables[s])] = torch.tensor(self.tables[s], dtype=torch.int32)
        return t.to(self.k.device)


class PagedAttentionManager:
    """One :class:`PagedKVCache` per layer sharing a page pool; tracks live sequences."""

    def __init__(self, num_layers: int, num_pages: int, page_size: int, kv_heads: int, head_dim: int, device="cpu", dtype=torch.float32):
        self.pools = [PagePool(num_pages, page_size) for _ in range(num_layers)]
        self.layers = [PagedKVCache(p, kv_heads, head_dim, device, dtype) for p in self.pools]

    def add_sequence(self, seq_id: int) -> None:
        for l in self.layers:
            l.add_sequence(seq_id)

    def free_sequence(self, seq_id: int) -> None:
        for l in self.layers:
            l.free_sequence(seq_id)

    def attend(self, layer: int, seq_id: int, q: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
        """Single-token decode attention for one sequence: ``q`` ``[heads, head_dim]`` against the cached keys/values."""
        k, v = self.layers[layer].gather(seq_id)
        H, D = q.shape
        rep = H // k.shape[1]
        k, v = k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)
        s = torch.einsum("hd,thd->ht", q.float(), k.float()) * (scale or 1.0 / math.sqrt(D))
        return torch.einsum("ht,thd->hd", torch.softmax(s, -1), v.float()).to(q.dtype)


# ----------------------------------------------------------------------------------------------------------------------
# flex attention
# ----------------------------------------------------------------------------------------------------------------------
class BlockMask:
    """Block-sparse mask: ``mask_fn(q_idx, kv_idx) -> bool`` evaluated per (block_q x block_kv) tile; all-masked tiles are skipped."""

    def __init__(self, q_len: int, kv_len: int, mask_fn: Callable[[torch.Tensor, torch.Tensor], torch.Tensor], block: int = 128):
        self.q_len, self.kv_len, self.block, self.mask_fn = q_len, kv_len, block, mask_fn
        qi = torch.arange(q_len).view(-1, 1)
        ki = torch.arange(kv_len).view(1, -1)
        self.dense = mask_fn(qi, ki)
        nq, nk = (q_len + block - 1) // block, (kv_len + block - 1) // block
        pad = F.pad(self.dense, (0, nk * block - kv_len, 0, nq * block - q_len))
        tiles = pad.view(nq, block, nk, block).permute(0, 2, 1, 3)
        self.any = tiles.any(-1).any(-1)
        self.full = tiles.all(-1).all(-1)

    def sparsity(self) -> float:
        return 1.0 - self.any.float().mean().item()

    @staticmethod
    def causal(q_len: int, kv_len: int, block: int = 128) -> "BlockMask":
        return BlockMask(q_len, kv_len, lambda q, k: k <= q + (kv_len - q_len), block)


def causal_score_mod(score, b, h, q_idx, kv_idx):
    return torch.where(kv_idx <= q_idx, score, torch.full_like(score, float("-inf")))


def alibi_score_mod(slopes: torch.Tensor):
    def mod(score, b, h, q_idx, kv_idx):
        return score - slopes.to(score.device).view(1, -1, 1, 1) * (q_idx - kv_idx).abs()
    return mod


def relative_position_score_mod(bias: torch.Tensor):
    """``bias``: ``[heads, 2*max_dist+1]`` learned relative-position bias."""
    max_dist = (bias.shape[1] - 1) // 2

    def mod(score, b, h, q_idx, kv_idx):
        rel = (kv_idx - q_idx).clamp(-max_dist, max_dist) + max_dist            # broadcast index grid [..., Sq, Sk]
        rel = rel.reshape(rel.shape[-2], rel.shape[-1])
        return score + bias.to(score.device)[:, rel].unsqueeze(0)               # [1, heads, Sq, Sk]
    return mod


def relative_position_bias_score_mod(bias_table: torch.Tensor, max_dist: int):
    """One shared 1-D table ``[2 * max_dist + 1]`` indexed by ``clamp(q_idx - kv_idx, -max_dist, max_dist) + max_dist``
    (ferrotorch-nn/src/flex_attention.rs:755); :func:`relative_position_score_mod` is the per-head form."""
    table = bias_table.reshape(-1)

    def mod(score, b, h, q_idx, kv_idx):
        rel = ((q_idx - kv_idx).clamp(-max_dist, max_dist) + max_dist).clamp_max(table.numel() - 1)
        return score + table.to(score.device)[rel]
    return mod


def flex_attention(q, k, v, score_mod: Optional[Callable] = None, block_mask: Optional[BlockMask] = None, scale: Optional[float] = None):
    """Attention on ``[B, H, S, D]`` with an arbitrary score modification and/or block mask."""
    B, H, Sq, D = q.shape
    Sk = k.shape[2]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    rep = H // k.shape[1]
    k, v = (k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1)) if rep > 1 else (k, v)
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) * scale
    if score_mod is not None:
        qi = torch.arange(Sq, device=q.device).view(1, 1, Sq, 1)
        ki = torch.arange(Sk, device=q.device).view(1, 1, 1, Sk)
        s = score_mod(s, torch.arange(B, device=q.device).view(B, 1, 1, 1), torch.arange(H, device=q.device).view(1, H, 1, 1), qi, ki)
    if block_mask is not None:
        s = s.masked_fill(~block_mask.dense.to(q.device), float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.nan_to_num(p, nan=0.0)
    return torch.matmul(p, v.float()).to(q.dtype)


# ----------------------------------------------------------------------------------------------------------------------
# init
# ----------------------------------------------------------------------------------------------------------------------
class NonLinearity(enum.Enum):
    Linear = "linear"
    ReLU = "relu"
    LeakyReLU = "leaky_relu"
    Tanh = "tanh"
    Sigmoid = "sigmoid"
    SELU = "selu"


class init:  # namespace
    NonLinearity = NonLinearity
    constant = staticmethod(lambda t, v: torch.nn.init.constant_(t, v))
    zeros = staticmethod(torch.nn.init.zeros_)
    ones = staticmethod(torch.nn.init.ones_)
    uniform = staticmethod(lambda t, a=0.0, b=1.0: torch.nn.init.uniform_(t, a, b))
    normal = staticmethod(lambda t, mean=0.0, std=1.0: torch.nn.init.normal_(t, mean, std))
    xavier_uniform = staticmethod(lambda t, gain=1.0: torch.nn.init.xavier_uniform_(t, gain))
    xavier_normal = staticmethod(lambda t, gain=1.0: torch.nn.init.xavier_normal_(t, gain))
    kaiming_uniform = staticmethod(lambda t, nonlinearity=NonLinearity.ReLU, a=0.0: torch.nn.init.kaiming_uniform_(
        t, a=a, nonlinearity=nonlinearity.value if isinstance(nonlinearity, NonLinearity) else nonlinearity))
    kaiming_normal = staticmethod(lambda t, nonlinearity=NonLinearity.ReLU, a=0.0: torch.nn.init.kaiming_normal_(
        t, a=a, nonlinearity=nonlinearity.value if isinstance(nonlinearity, NonLinearity) else nonlinearity))
    trunc_normal_ = staticmethod(lambda t, mean=0.0, std=1.0, a=-2.0, b=2.0: torch.nn.init.trunc_normal_(t, mean, std, a, b))
    orthogonal_ = staticmethod(lambda t, gain=1.0: torch.nn.init.orthogonal_(t, gain))
    sparse_ = staticmethod(lambda t, sparsity, std=0.01: torch.nn.init.sparse_(t, sparsity, std))
    dirac_ = staticmethod(lambda t, groups=1: torch.nn.init.dirac_(t, groups))
    eye_ = staticmethod(torch.nn.init.eye_)


# ----------------------------------------------------------------------------------------------------------------------
# gradient utilities
# ----------------------------------------------------------------------------------------------------------------------
def clip_grad_norm_(parameters: Iterable[torch.Tensor], max_norm: float, norm_type: float = 2.0, error_if_nonfinite: bool = False) -> torch.Tensor:
    """Scale gradients so their global norm is at most ``max_norm``; returns the norm before clipping.
    For the L2 norm of CUDA gradients one multi-buffer reduction kernel computes the norm and the clip coefficient on the
    device (no per-parameter host sync), then one scale kernel per gradient applies it."""
    ps = [p for p in parameters if p.grad is not None]
    if not ps:
        return torch.tensor(0.0)
    grads = [p.grad for p in ps]
    if norm_type == 2.0 and grads[0].is_cuda and all(g.dtype in (torch.float32, torch.bfloat16) and g.is_contiguous() for g in grads):
        norm, coef = ops.grad_norm_([g.reshape(-1) for g in grads], max_norm)
        if error_if_nonfinite and not torch.isfinite(norm):
            raise InvalidArgument("non-finite gradient norm")
        for g in grads:
            ops.scale_(g, 1.0, coef)
        return norm
    return torch.nn.utils.clip_grad_norm_(ps, max_norm, norm_type, error_if_nonfinite)


def clip_grad_value_(parameters: Iterable[torch.Tensor], clip_value: float) -> None:
    torch.nn.utils.clip_grad_value_([p for p in parameters if p.grad is not None], clip_value)


# ----------------------------------------------------------------------------------------------------------------------
# packed sequences / resampling
# ----------------------------------------------------------------------------------------------------------------------
from .rnn import PackedSequence, pack_padded_sequence, pad_packed_sequence, pad_sequence, pack_sequence  # noqa: E402,F401


class InterpolateMode(enum.Enum):
    """ferrotorch-nn/src/upsample.rs:32."""
    Nearest = "nearest"
    Bilinear = "bilinear"
    Bicubic = "bicubic"


class GridSampleMode(enum.Enum):
    """ferrotorch-nn/src/upsample.rs:54."""
    Bilinear = "bilinear"
    Nearest = "nearest"


class GridSamplePaddingMode(enum.Enum):
    """ferrotorch-nn/src/upsample.rs:43."""
    Zeros = "zeros"
    Border = "border"
    Reflection = "reflection"


class GeluApproximate(enum.Enum):
    """``None`` = exact erf form, ``Tanh`` = tanh polynomial, ``Sigmoid`` = ``x * sigmoid(1.702 x)`` (ferrotorch-core/src/grad_fns/activation.rs:254)."""
    None_ = "none"
    Tanh = "tanh"
    Sigmoid = "sigmoid"

    def __str__(self):
        return self.value


def _enum_value(v):
    return v.value if isinstance(v, enum.Enum) else v


def gelu(x: torch.Tensor, approximate="none") -> torch.Tensor:
    """GELU in the three forms of :class:`GeluApproximate` (a string or the enum)."""
    a = _enum_value(approximate)
    if a == "sigmoid":
        return x * torch.sigmoid(1.702 * x)
    if a not in ("none", "tanh"):
        raise InvalidArgument(f"gelu: unknown approximation {approximate!r}")
    return F.gelu(x, approximate=a)


gelu_with = gelu                                             # ferrotorch-core's name for the form that takes the mode


class GELU(Module):
    def __init__(self, approximate="none"):
        super().__init__()
        self.approximate = _enum_value(approximate)
        if self.approximate not in ("none", "tanh", "sigmoid"):
            raise InvalidArgument(f"GELU: unknown approximation {approximate!r}")

    def forward(self, x):
        return gelu(x, self.approximate)

    def extra_repr(self):
        return f"approximate={self.approximate!r}"


from .resample import affine_grid, grid_sample, interpolate  # noqa: E402,F401  (written out on gather arithmetic: nn/resample.py)

# functional pooling / reshaping forms the reference exports at the crate root (ferrotorch-nn/src/pooling.rs, upsample.rs)
from .pooling import (max_pool1d, max_pool2d, max_pool3d, avg_pool1d, avg_pool2d, avg_pool3d, adaptive_avg_pool1d, adaptive_avg_pool2d,  # noqa: E402,F401
                      adaptive_avg_pool3d, adaptive_max_pool1d, adaptive_max_pool2d, adaptive_max_pool3d, lp_pool1d, lp_pool2d, max_unpool2d,
                      pixel_shuffle, pixel_unshuffle, unfold, fold)

# hook signatures (ferrotorch-nn/src/hooks.rs:37-48)
ForwardHook = Callable[[torch.Tensor, torch.Tensor], None]               # (input, output)
ForwardPreHook = Callable[[torch.Tensor], torch.Tensor]                  # input -> replacement input
BackwardHook = Callable[[torch.Tensor, torch.Tensor], None]              # (grad_input, grad_output)


def functional_pad_1d(x, pad, mode="constant", value=0.0):
    """Flat ``(last_lo, last_hi, ...)`` padding amounts; modes constant / reflect / replicate / circular."""
    from .padding import pad as _pad
    return _pad(x, pad, _enum_value(mode), value)


functional_pad_2d = functional_pad_1d
functional_pad_3d = functional_pad_1d


# ----------------------------------------------------------------------------------------------------------------------
# quantisation-aware training
# ----------------------------------------------------------------------------------------------------------------------
class ObserverType(enum.Enum):
    MinMax = "minmax"
    MovingAverage = "moving_average"
    PerChannel = "per_channel"


@dataclass
class QatConfig:
    bits: int = 8
    symmetric: bool = True
    observer: ObserverType = ObserverType.MovingAverage
    momentum: float = 0.01


class _FakeQuant(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, scale, zero, qmin, qmax):
        q = torch.clamp(torch.round(x / scale) + zero, qmin, qmax)
        ctx.save_for_backward((x / scale + zero >= qmin) & (x / scale + zero <= qmax))
        return (q - zero) * scale

    @staticmethod
    def backward(ctx, g):
        (m,) = ctx.saved_tensors
        return g * m, None, None, None, None     # straight-through estimator inside the clamp range


class FakeQuantize(Module):
    def __init__(self, cfg: QatConfig):
        super().__init__()
        self.cfg = cfg
        self.register_buffer("lo", torch.tensor(0.0))
        self.register_buffer("hi", torch.tensor(0.0))
        self.register_buffer("seen", torch.tensor(0))

    def forward(self, x):
        if self.training:
            lo, hi = x.detach().min(), x.detach().max()
            if int(self.seen) == 0 or self.cfg.observer == ObserverType.MinMax:
                self.lo = torch.minimum(self.lo, lo) if int(self.seen) else lo
                self.hi = torch.maximum(self.hi, hi) if int(self.seen) else hi
            else:
                m = self.cfg.momentum
                self.lo, self.hi = self.lo * (1 - m) + lo * m, self.hi * (1 - m) + hi * m
            self.seen += 1
        qmax = 2 ** (self.cfg.bits - 1) - 1 if self.cfg.symmetric else 2 ** self.cfg.bits - 1
        qmin = -qmax - 1 if self.cfg.symmetric else 0
        if self.cfg.symmetric:
            scale = torch.clamp(torch.maximum(self.lo.abs(), self.hi.abs()) / qmax, min=1e-8)
            zero = torch.zeros_like(scale)
        else:
            scale = torch.clamp((self.hi - self.lo) / (qmax - qmin), min=1e-8)
            zero = torch.round(qmin - self.lo / scale)
        return _FakeQuant.apply(x, scale, zero, qmin, qmax)


class QuantizedModel(Module):
    """A model whose Linear / Conv inputs and weights go through fake-quantisation observers."""

    def __init__(self, model: torch.nn.Module, cfg: QatConfig):
        super().__init__()
        self.model, self.cfg = model, cfg
        self.observers = torch.nn.ModuleDict()
        for name, m in model.named_modules():
            if isinstance(m, (torch.nn.Linear, torch.nn.Conv2d)) or type(m).__name__ in ("Linear", "Conv2d"):
                key = name.replace(".", "_") or "root"
                self.observers[key + "_act"] = FakeQuantize(cfg)
                self.observers[key + "_w"] = FakeQuantize(cfg)
                m.register_forward_pre_hook(self._pre(key))

    def _pre(self, key):
        def hook(mod, args):
            x = self.observers[key + "_act"](args[0])
            mod._qat_orig_weight = mod.weight.data
            mod.weight.data = self.observers[key + "_w"](mod.weight).data
            mod.register_forward_hook(self._post, always_call=True) if not getattr(mod, "_qat_post", False) else None
            mod._qat_post = True
            return (x, *args[1:])
        return hook

    @staticmethod
    def _post(mod, args, out):
        if hasattr(mod, "_qat_orig_weight"):
            mod.weight.data = mod._qat_orig_weight
            del mod._qat_orig_weight
        return out

    def forward(self, *a, **k):
        return self.model(*a, **k)


QatModel = QuantizedModel                                    # ferrotorch-nn/src/qat.rs


def prepare_qat(model: torch.nn.Module, cfg: Optional[QatConfig] = None) -> QuantizedModel:
    return QuantizedModel(model, cfg or QatConfig())
