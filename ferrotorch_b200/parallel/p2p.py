"""Device point-to-point channels over symmetric memory and a GPipe pipeline stage built on them.

A :class:`P2PChannel` is a directed chain: every rank receives from one upstream peer and sends to one downstream peer. A message is put
straight into a slot of the receiver's ring buffer by the sender's kernel (peer stores) followed by a release-store of the message number on
the receiver's flag; the receiver's kernel waits (bounded, 2 s) for the flag, copies the slot out and acknowledges on the sender so the slot
can be re-used. No host synchronisation, no library call: launches of both sides are ordinary stream work.

:class:`GpuPipelineStage` runs one stage of a GPipe schedule: activations go downstream through one channel, the gradient with respect to the
stage input (the real gradient, computed by autograd) goes upstream through a second one.

Reference parity: ferrotorch-distributed/src/pipeline.rs:35,66,136-222,250-331 (host byte transport, zero grad-input) and p2p.rs:19-150.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Sequence

import torch
import torch.distributed as dist

from .. import _lib
from ..errors import InvalidArgument
from .symm import SymmetricBuffer


class P2PChannel:
    def __init__(self, slot_bytes: int, slots: int = 4, device=None, group=None):
        if slot_bytes % 16 or slots < 1:
            raise InvalidArgument("slot size must be a multiple of 16 bytes")
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.slot_bytes, self.slots, self.device = slot_bytes, slots, torch.device(device or "cuda")
        self.ring = SymmetricBuffer(slots * slot_bytes, torch.uint8, self.device, self.group)
        self.flags = SymmetricBuffer(slots, torch.int32, self.device, self.group, zero=True)
        self.acks = SymmetricBuffer(slots, torch.int32, self.device, self.group, zero=True)
        self.counter = torch.zeros(2, device=self.device, dtype=torch.int32)
        self.sent = self.received = 0
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)

    def _check(self, t: torch.Tensor) -> int:
        nbytes = t.numel() * t.element_size()
        if not t.is_cuda or not t.is_contiguous() or nbytes % 16 or nbytes > self.slot_bytes:
            raise InvalidArgument(f"message must be a contiguous CUDA tensor of a multiple of 16 bytes, at most {self.slot_bytes}")
        return nbytes

    def send(self, t: torch.Tensor, dst: int) -> None:
        nbytes = self._check(t)
        self.sent += 1
        msg, slot = self.sent, (self.sent - 1) % self.slots
        prev = msg - self.slots if msg > self.slots else 0
        _lib.call("ft_comm_p2p_put", t, self.ring.ptrs[dst] + slot * self.slot_bytes, nbytes, self.flags.ptrs[dst] + 4 * slot, self.acks.ptrs[self.rank] + 4 * slot,
                  msg, prev, self.counter[0:1], _lib.S())

    def recv(self, out: torch.Tensor, src: int) -> torch.Tensor:
        nbytes = self._check(out)
        self.received += 1
        msg, slot = self.received, (self.received - 1) % self.slots
        _lib.call("ft_comm_p2p_get", out, self.ring.ptrs[self.rank] + slot * self.slot_bytes, nbytes, self.flags.ptrs[self.rank] + 4 * slot,
                  self.acks.ptrs[src] + 4 * slot, msg, self.counter[1:2], _lib.S())
        return out


class GpuPipelineStage:
    """One stage of a GPipe pipeline over device channels. ``module`` maps ``[mb, *in_shape] -> [mb, *out_shape]``; all ranks run
    :meth:`forward_backward` with the same number of micro-batches."""

    def __init__(self, module: torch.nn.Module, in_shape: Sequence[int], out_shape: Sequence[int], micro_batch: int, dtype=torch.float32, group=None, slots: int = 4):
        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.module, self.mb, self.dtype = module, micro_batch, dtype
        self.in_shape, self.out_shape = (micro_batch, *in_shape), (micro_batch, *out_shape)
        dev = next(module.parameters()).device
        item = torch.empty(0, dtype=dtype).element_size()

        def nbytes(shape):
            n = item
            for s in shape:
                n *= s
            return (n + 15) // 16 * 16
        # every rank allocates both channels with the largest message any stage sends (symmetric allocation), sized by all-reduce MAX
        need = torch.tensor([max(nbytes(self.in_shape), nbytes(self.out_shape))], device=dev)
        dist.all_reduce(need, op=dist.ReduceOp.MAX, group=self.group)
        self.fwd, self.bwd = P2PChannel(int(need), slots, dev, self.group), P2PChannel(int(need), slots, dev, self.group)
        self.dev = dev

    @property
    def first(self) -> bool:
        return self.rank == 0

    @property
    def last(self) -> bool:
        return self.rank == self.world - 1

    def forward_backward(self, inputs: Optional[Sequence[torch.Tensor]], n_micro: int, loss_fn: Optional[Callable[[torch.Tensor, int], torch.Tensor]] = None):
        """GPipe: all forwards, then all backwards in reverse order. The first stage passes ``inputs`` (one tensor per micro-batch); the last stage
        passes ``loss_fn(output, micro_index) -> scalar``. Returns the list of losses on the last stage, else ``None``. Gradients accumulate in the
        module's parameters."""
        xs: List[torch.Tensor] = []
        ys: List[torch.Tensor] = []
        losses = []
        for i in range(n_micro):
            if self.first:
                x = inputs[i].to(self.dev, self.dtype)
            else:
                x = self.fwd.recv(torch.empty(self.in_shape, device=self.dev, dtype=self.dtype), self.rank - 1).requires_grad_()
            y = self.module(x)
            xs.append(x)
            ys.append(y)
            if not self.last:
                self.fwd.send(y.detach().contiguous(), self.rank + 1)
        for i in reversed(range(n_micro)):
            if self.last:
                loss = loss_fn(ys[i], i)
                losses.append(loss.detach())
                loss.backward()
            else:
                g = self.bwd.recv(torch.empty(self.out_shape, device=self.dev, dtype=self.dtype), self.rank + 1)
                ys[i].backward(g)
            if not self.first:
                self.bwd.send(xs[i].grad.contiguous(), self.rank - 1)
        return list(reversed(losses)) if self.last else None
