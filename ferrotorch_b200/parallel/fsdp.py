"""Fully-sharded data parallel training engine over flat parameter units.

Sharding: every :class:`FlatUnit` (one per decoder layer, plus embedding, final
norm and head) is split evenly across ranks. Each rank keeps the f32 master
weights and AdamW moments of its slice only (ZeRO-3 state sharding); the bf16
compute copy of a unit is produced by an all-gather and its bf16 gradient is
reduce-scattered (mean) to the owners as soon as the unit's backward finishes,
where the sharded AdamW update runs at once ("optimizer in backward"), followed
by the all-gather of the updated slice, which therefore overlaps the rest of
the backward pass and is complete long before the next forward needs it.

Transports:
  * ``comm="nccl"``   - torch.distributed collectives on a side stream (the library baseline).
  * ``comm="fused"``  - one hand-written kernel per unit over NVLink peer memory:
                        pull-reduce of the gradient slice from every peer in fixed rank order, AdamW on the
                        f32 master slice, bf16 result pushed straight into every peer's parameter buffer
                        (reduce-scatter + optimizer + all-gather in one launch; see ``parallel/symm.py``).
At world size 1 both reduce to the plain fused AdamW kernel on a side stream.

Reference parity: ferrotorch-distributed/src/fsdp.rs:44-61 (ShardingStrategy), :151-288 (construction),
:389-542 (forward gather), :627-789 (sync_gradients), :806-845 (broadcast_updated_params). The reference gathers
every parameter of the whole model up front on host vectors; here gathers are per unit, on device, overlapped.
"""
from __future__ import annotations

import enum
import os
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

from .. import ops
from ..errors import InvalidArgument
from .flat import FlatUnit


class ShardingStrategy(enum.Enum):
    FULL_SHARD = "full_shard"          # ZeRO-3: params, grads and optimizer state sharded
    SHARD_GRAD_OP = "shard_grad_op"    # ZeRO-2: grads and optimizer state sharded, params replicated
    NO_SHARD = "no_shard"              # DDP-like: all-reduce gradients, replicated state
    HYBRID_SHARD = "hybrid_shard"      # shard inside a node, replicate across nodes


@dataclass
class AdamWConfig:
    lr: float = 3e-4
    betas: tuple = (0.9, 0.95)
    eps: float = 1e-8
    weight_decay: float = 0.01
    maximize: bool = False


class _EngineOwner:
    """Unit owner installed by the engine (see ``_ParamOwner`` in models/llama.py for the protocol)."""

    def __init__(self, engine: "FSDP", unit: FlatUnit, base_owner):
        self.engine, self.unit = engine, unit
        self.cfg, self.rope = base_owner.cfg, base_owner.rope
        self.recompute = base_owner.recompute
        self.grad_preaccumulated = getattr(base_owner, "grad_preaccumulated", False)
        self._base = base_owner

    def acquire_params(self) -> Dict[str, torch.Tensor]:
        return self.engine._acquire_params(self.unit)

    def release_params(self, after_forward: bool) -> None:
        self.engine._release_params(self.unit, after_forward)

    def acquire_grads(self) -> Dict[str, torch.Tensor]:
        return self.engine._acquire_grads(self.unit)

    def grads_ready(self) -> None:
        self.engine._grads_ready(self.unit)


class FSDP:
    """Training engine: ``loss = engine.train_step(ids, labels)`` runs forward, backward, gradient
    reduce-scatter, sharded AdamW and parameter all-gather for one micro-batch per rank.

    What is sharded: the f32 master weights, both AdamW moments and the reduced gradients live only on the owner of each slice (every
    parameter is owned, updated and checkpointed in shards). The bf16 all-gathered copy that the GEMMs read is kept resident between steps
    as a cache (16 GB of an 8B model per GPU, out of 180 GB) and is refreshed by the all-gather that follows each unit's update, so a step
    moves every parameter across the fabric once (after the update) instead of twice (before forward and again before backward) and the
    gather is hidden behind the rest of the backward pass. ``FULL_SHARD`` and ``SHARD_GRAD_OP`` therefore run the same schedule here;
    ``NO_SHARD`` (use :class:`ferrotorch_b200.parallel.DDP`) and ``HYBRID_SHARD`` (one NVSwitch domain has no second level) are refused."""

    def __init__(self, model, optim: AdamWConfig | None = None, process_group=None, strategy: ShardingStrategy = ShardingStrategy.FULL_SHARD,
                 comm: str | None = None, grad_buffers: int = 2, overlap_optimizer: bool = True):
        import torch.distributed as dist
        self.model = model
        self.optim = optim or AdamWConfig()
        if strategy not in (ShardingStrategy.FULL_SHARD, ShardingStrategy.SHARD_GRAD_OP):
            raise InvalidArgument(f"{strategy} is not available in the device engine: use parallel.DDP for NO_SHARD; HYBRID_SHARD needs more than "
                                  "one NVSwitch domain (the host-side distributed.FSDP implements both)")
        self.strategy = strategy
        self.pg = process_group
        self.dist = dist if (dist.is_available() and dist.is_initialized()) else None
        self.world = self.dist.get_world_size(self.pg) if self.dist else 1
        self.rank = self.dist.get_rank(self.pg) if self.dist else 0
        self.units: List[FlatUnit] = model.units()
        for u in self.units:
            if u.world != self.world or u.rank != self.rank:
                raise InvalidArgument(f"unit {u.name} was built for world {u.world}/rank {u.rank}, engine has {self.world}/{self.rank}")
        self.device = self.units[0].device
        self.comm = comm or os.environ.get("FT_FSDP_COMM", "fused")
        self.step_count = 0
        cuda = self.device.type == "cuda"
        if os.environ.get("FT_NO_SIDE_STREAM") == "1":
            overlap_optimizer = False
        self._opt_ctas = int(os.environ.get("FT_OPT_CTAS", "296")) if (cuda and overlap_optimizer) else 0   # two CTAs per SM beside the GEMM
        self._debug_skip_opt = os.environ.get("FT_DEBUG_SKIP_OPT") == "1"      # diagnosis only: measures the step without any update
        self.side = torch.cuda.Stream(device=self.device, priority=-1) if (cuda and overlap_optimizer) else None
        # gradient buffers: a small rotating pool of full-size bf16 buffers, sized for the largest unit
        maxn = max(u.padded for u in self.units)
        self._grad_pool = [torch.empty(maxn, device=self.device, dtype=torch.bfloat16) for _ in range(max(grad_buffers, 1))]
        self._grad_free_ev = [None] * len(self._grad_pool)
        self._grad_next = 0
        self._unit_grad_slot: Dict[str, int] = {}
        self._param_ready_ev: Dict[str, object] = {}
        self._grad_shard = torch.empty(max(u.chunk for u in self.units), device=self.device, dtype=torch.bfloat16) if self.world > 1 else None
        for u in self.units:
            u.init_adam()
        # install engine owners
        for o in model.owners():
            eo = _EngineOwner(self, o.unit, o)
            self._swap_owner(model, o, eo)
        self._fused = None
        if self.world > 1 and self.comm == "fused":
            from .symm import FusedShardedAdamW
            try:
                self._fused = FusedShardedAdamW(self)
            except (RuntimeError, ImportError, AttributeError) as e:   # no symmetric memory on this fabric: library collectives
                import warnings
                warnings.warn(f"symmetric memory unavailable ({e}); FSDP falls back to NCCL collectives")
                self.comm = "nccl"
        if self.world == 1:
            self.comm = "none"

    # -- owner plumbing ---------------------------------------------------------------
    @staticmethod
    def _swap_owner(model, old, new) -> None:
        for mod in model.modules():
            for attr in ("owner", "embed_owner", "norm_owner", "head_owner"):
                if getattr(mod, attr, None) is old:
                    setattr(mod, attr, new)

    def _acquire_params(self, unit: FlatUnit) -> Dict[str, torch.Tensor]:
        ev = self._param_ready_ev.pop(unit.name, None)
        if ev is not None:
            torch.cuda.current_stream().wait_event(ev)
        return unit.views()

    def _release_params(self, unit: FlatUnit, after_forward: bool) -> None:
        pass  # the gathered bf16 copy stays resident as a cache (see the class docstring)

    def _acquire_grads(self, unit: FlatUnit) -> Dict[str, torch.Tensor]:
        slot = self._unit_grad_slot.get(unit.name)
        if slot is None:
            slot = self._grad_next
            self._grad_next = (self._grad_next + 1) % len(self._grad_pool)
            ev = self._grad_free_ev[slot]
            if ev is not None:
                torch.cuda.current_stream().wait_event(ev)   # the optimizer that last read this buffer has finished
                self._grad_free_ev[slot] = None
            self._unit_grad_slot[unit.name] = slot
            unit.grad = self._grad_pool[slot][: unit.padded]
        return unit.views(unit.grad)

    def _grads_ready(self, unit: FlatUnit) -> None:
        slot = self._unit_grad_slot.pop(unit.name)
        o = self.optim
        unit.step += 1
        cur = torch.cuda.current_stream() if self.device.type == "cuda" else None
        if self.side is not None:
            done = torch.cuda.Event()
            done.record(cur)
            self.side.wait_event(done)
            ctx = torch.cuda.stream(self.side)
        else:
            import contextlib
            ctx = contextlib.nullcontext()
        with ctx:
            if self._debug_skip_opt:
                pass
            elif self.world == 1:
                ops.adamw_flat_(unit.master, unit.full, unit.exp_avg, unit.exp_avg_sq, unit.grad, lr=o.lr, beta1=o.betas[0],
                                beta2=o.betas[1], eps=o.eps, weight_decay=o.weight_decay, step=unit.step, maximize=o.maximize,
                                max_ctas=self._opt_ctas)
            elif self._fused is not None:
                self._fused.step(unit, slot)
            else:
                gs = self._grad_shard[: unit.chunk]
                self.dist.reduce_scatter_tensor(gs, unit.grad, op=self.dist.ReduceOp.AVG, group=self.pg)
                mine = unit.shard_slice(unit.full)
                ops.adamw_flat_(unit.master, mine, unit.exp_avg, unit.exp_avg_sq, gs, lr=o.lr, beta1=o.betas[0], beta2=o.betas[1],
                                eps=o.eps, weight_decay=o.weight_decay, step=unit.step, maximize=o.maximize, max_ctas=self._opt_ctas)
                self.dist.all_gather_into_tensor(unit.full, mine, group=self.pg)
            if self.side is not None:
                ev = torch.cuda.Event()
                ev.record(self.side)
                self._grad_free_ev[slot] = ev
                self._param_ready_ev[unit.name] = ev
        unit.grad = None

    # -- public API -----------------------------------------------------------------------
    def train_step(self, ids: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """One optimizer step on this rank's micro-batch; returns the (local) mean loss as a 0-d device tensor."""
        self.step_count += 1
        loss = self.model(ids, labels=labels)
        loss.backward()
        return loss.detach()

    def synchronize(self) -> None:
        if self.side is not None:
            torch.cuda.current_stream().wait_stream(self.side)

    def state_bytes(self) -> int:
        return sum(u.nbytes_state() for u in self.units)
