"""Context (sequence) parallel attention over a process group: Ulysses head/sequence exchange and ring attention.

* :class:`UlyssesAttention`: activations are sharded on the sequence; an all-to-all turns ``[S/W, H, D]`` into ``[S, H/W, D]`` (all tokens of a
  subset of heads), attention runs locally (FlashAttention kernel on CUDA), a second all-to-all restores the sequence sharding. On a CUDA group
  the exchange is the peer-memory all-to-all kernel (``SymmComm.all_to_all``); it is differentiable through the mirrored exchange.
* :func:`ring_attention`: K/V blocks circulate; at step ``s`` rank ``r`` attends its queries to the block of rank ``(r - s) mod W`` pulled from
  that peer's symmetric buffer, and partial results are merged with the running log-sum-exp. Causal masking skips blocks from later ranks.
  Forward only (inference / evaluation).

The reference has no cross-device sequence parallelism (its long-context support is single-device: ferrotorch-nn/src/flash_attention.rs:45,
ferrotorch-nn/src/transformer.rs:210-266); both modes are additions built on the same bounded-wait symmetric-memory fabric.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn.functional as F

from ..errors import InvalidArgument


def _group(group):
    g = group if group is not None else dist.group.WORLD
    return g, dist.get_world_size(g), dist.get_rank(g)


def _all_to_all_chunks(x: torch.Tensor, group, comm=None, buf=None) -> torch.Tensor:
    """``x``: ``[W, chunk...]`` (slice q goes to rank q) -> ``[W, chunk...]`` (slice q came from rank q)."""
    g, W, rank = _group(group)
    if comm is not None and x.is_cuda:
        chunk = x[0].numel()
        buf.tensor[: x.numel()].view_as(x).copy_(x)
        out = torch.empty_like(x)
        comm.all_to_all(buf, out, chunk)
        return out
    outs = [torch.empty_like(x[0]) for _ in range(W)]
    if x.is_cuda:
        dist.all_to_all(outs, [x[q].contiguous() for q in range(W)], group=g)
    else:                                            # gloo has no all_to_all: gather everything, keep the slices addressed to this rank
        full = [torch.empty_like(x) for _ in range(W)]
        dist.all_gather(full, x.contiguous(), group=g)
        outs = [full[q][rank] for q in range(W)]
    return torch.stack(outs, 0)


class _SeqToHeads(torch.autograd.Function):
    """[S/W, H, D] (sequence shard, all heads) -> [S, H/W, D] (all tokens, head shard); the backward is the inverse exchange."""

    @staticmethod
    def forward(ctx, x, group, comm, buf, inverse):
        ctx.args = (group, comm, buf, inverse)
        return _exchange(x, group, comm, buf, inverse)

    @staticmethod
    def backward(ctx, g):
        group, comm, buf, inverse = ctx.args
        return _exchange(g.contiguous(), group, comm, buf, not inverse), None, None, None, None


def _exchange(x, group, comm, buf, inverse):
    _, W, _ = _group(group)
    if not inverse:
        s, H, D = x.shape
        send = x.view(s, W, H // W, D).permute(1, 0, 2, 3).contiguous()          # [W(dst head group), s, H/W, D]
        recv = _all_to_all_chunks(send, group, comm, buf)                         # [W(src seq shard), s, H/W, D]
        return recv.reshape(W * s, H // W, D)
    S, h, D = x.shape
    send = x.view(W, S // W, h, D).contiguous()                                   # [W(dst seq shard), s, h, D]
    recv = _all_to_all_chunks(send, group, comm, buf)                             # [W(src head group), s, h, D]
    return recv.permute(1, 0, 2, 3).reshape(S // W, W * h, D)


def _local_attention(q, k, v, causal: bool, scale: float) -> torch.Tensor:
    """q ``[S, Hq, D]``, k/v ``[S, Hkv, D]`` -> ``[S, Hq, D]`` (FlashAttention kernel for bf16 CUDA with D = 128, SDPA otherwise)."""
    S, Hq, D = q.shape
    Hkv = k.shape[1]
    if q.is_cuda and q.dtype == torch.bfloat16 and D == 128:
        from ..ops import attention_packed
        qkv = torch.cat([q.reshape(S, Hq * D), k.reshape(S, Hkv * D), v.reshape(S, Hkv * D)], 1)
        return attention_packed(qkv, 1, S, Hq, Hkv, D, causal, scale).view(S, Hq, D)
    rep = Hq // Hkv
    o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.repeat_interleave(rep, 1).transpose(0, 1)[None], v.repeat_interleave(rep, 1).transpose(0, 1)[None],
                                       is_causal=causal, scale=scale)
    return o[0].transpose(0, 1)


class UlyssesAttention(torch.nn.Module):
    """Sequence-parallel attention by head exchange. ``forward(q, k, v)`` takes this rank's sequence shard ``[S/W, H, D]`` of each tensor."""

    def __init__(self, group=None, causal: bool = True, use_symmetric_memory: bool = True):
        super().__init__()
        self.group, self.world, self.rank = _group(group)
        self.causal, self.use_symm = causal, use_symmetric_memory
        self._comm = self._buf = None

    def _fabric(self, x):
        if not (self.use_symm and x.is_cuda and self.world > 1 and x.dtype in (torch.bfloat16, torch.float32)):
            return None, None
        need = x.numel()
        if self._comm is None or self._buf.tensor.numel() < need or self._buf.tensor.dtype != x.dtype:
            from .symm import SymmComm, SymmetricBuffer
            self._comm = self._comm or SymmComm(x.device, self.group)
            self._buf = SymmetricBuffer(need * 2, x.dtype, x.device, self.group)
        return self._comm, self._buf

    def forward(self, q, k, v, scale: Optional[float] = None):
        W = self.world
        if q.shape[1] % W or k.shape[1] % W:
            raise InvalidArgument("head counts must be divisible by the group size")
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        if W == 1:
            return _local_attention(q, k, v, self.causal, scale)
        comm, buf = self._fabric(q)
        qh, kh, vh = (_SeqToHeads.apply(t.contiguous(), self.group, comm, buf, False) for t in (q, k, v))
        o = _local_attention(qh, kh, vh, self.causal, scale)
        return _SeqToHeads.apply(o.contiguous(), self.group, comm, buf, True)


def _block_attention(q, k, v, causal: bool, scale: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """Attention of one (query block, key block) pair in f32 with its log-sum-exp: returns (out ``[S, Hq, D]`` f32, lse ``[S, Hq]``)."""
    S, Hq, D = q.shape
    rep = Hq // k.shape[1]
    if q.is_cuda and q.dtype == torch.bfloat16 and D == 128:
        from ..ops import flash_fwd
        Hkv = k.shape[1]
        qkv = torch.cat([q.reshape(S, Hq * D), k.reshape(S, Hkv * D), v.reshape(S, Hkv * D)], 1)
        out, lse = flash_fwd(qkv, 1, S, Hq, Hkv, D, causal, scale)
        if lse is not None:
            return out.view(S, Hq, D).float(), lse[0].transpose(0, 1)
    sc = torch.einsum("shd,thd->hst", q.float(), k.repeat_interleave(rep, 1).float()) * scale
    if causal:
        sc = sc.masked_fill(torch.ones(S, k.shape[0], dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    lse = torch.logsumexp(sc, -1)
    out = torch.einsum("hst,thd->shd", torch.exp(sc - lse[..., None]), v.repeat_interleave(rep, 1).float())
    return out, lse.transpose(0, 1)


@torch.no_grad()
def ring_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group=None, causal: bool = True, scale: Optional[float] = None, fabric=None) -> torch.Tensor:
    """q, k, v: this rank's contiguous sequence block ``[S/W, H, D]`` (rank r holds positions ``[r S/W, (r+1) S/W)``). Returns the attention
    output for the local queries. ``fabric = (SymmComm, SymmetricBuffer)`` pulls the K/V blocks over NVLink peer memory; without it (CPU
    groups) the blocks are exchanged with an all-gather."""
    g, W, rank = _group(group)
    scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
    if W == 1:
        return _block_attention(q, k, v, causal, scale)[0].to(q.dtype)
    kv = torch.cat([k.reshape(-1), v.reshape(-1)]).contiguous()
    if fabric is not None and q.is_cuda:
        comm, buf = fabric
        buf.tensor[: kv.numel()].copy_(kv)
        blocks = None
    else:
        blocks = [torch.empty_like(kv) for _ in range(W)]
        dist.all_gather(blocks, kv, group=g)
    acc = torch.zeros(q.shape, device=q.device, dtype=torch.float32)
    lse_run = torch.full(q.shape[:2], float("-inf"), device=q.device)
    n = k.numel()
    for step in range(W):
        src = (rank - step) % W
        if fabric is not None and q.is_cuda:
            blk = torch.empty_like(kv)
            comm.broadcast(buf, blk, kv.numel(), root=src)          # every rank pulls from its own source; the launch is still collective
        else:
            blk = blocks[src]
        if causal and src > rank:
            continue                                                 # keys from later positions: fully masked
        kb, vb = blk[:n].view_as(k), blk[n:].view_as(v)
        out, lse = _block_attention(q, kb, vb, causal and src == rank, scale)
        new = torch.logaddexp(lse_run, lse)
        acc = acc * torch.exp(lse_run - new)[..., None] + out * torch.exp(lse - new)[..., None]
        lse_run = new
    return acc.to(q.dtype)
