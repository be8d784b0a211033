"""Training loop utilities: ``Learner`` (fit / evaluate / checkpoint-resume), callbacks, metrics, AMP context,
activation checkpointing for sequential stacks, and a TensorBoard event-file writer (TFRecord framing with masked CRC32C and
hand-encoded Event/Summary protobufs - no TensorFlow dependency).

Reference parity: ferrotorch-train/src/learner.rs:57-394, callback.rs:30-259, metric.rs:25-290, history.rs, amp.rs:75,
checkpoint.rs:102 (checkpoint_sequential), tensorboard.rs:302-450.
"""
from __future__ import annotations

import contextlib
import math
import os
import socket
import struct
import time
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
from torch.utils.checkpoint import checkpoint as _ckpt

from ..serialize import TrainingCheckpoint


# ----------------------------------------------------------------------------------------------------------------------
# metrics
# ----------------------------------------------------------------------------------------------------------------------
class Metric:
    name = "metric"

    def update(self, output: torch.Tensor, target: torch.Tensor, loss: Optional[float] = None) -> None:
        raise NotImplementedError

    def compute(self) -> float:
        raise NotImplementedError

    def reset(self) -> None:
        raise NotImplementedError


class LossMetric(Metric):
    name = "loss"

    def __init__(self):
        self.reset()

    def update(self, output, target, loss=None):
        if loss is not None:
            n = target.shape[0] if target.dim() else 1
            self.total += float(loss) * n
            self.count += n

    def compute(self):
        return self.total / max(self.count, 1)

    def reset(self):
        self.total, self.count = 0.0, 0


class AccuracyMetric(Metric):
    name = "accuracy"

    def __init__(self):
        self.reset()

    def update(self, output, target, loss=None):
        pred = output.argmax(-1)
        self.correct += int((pred == target.to(pred.dtype).view_as(pred)).sum())
        self.count += target.numel()

    def compute(self):
        return self.correct / max(self.count, 1)

    def reset(self):
        self.correct, self.count = 0, 0


class TopKAccuracy(Metric):
    def __init__(self, k: int = 5):
        self.k, self.name = k, f"top{k}_accuracy"
        self.reset()

    def update(self, output, target, loss=None):
        top = output.topk(min(self.k, output.shape[-1]), -1).indices
        self.correct += int((top == target.long().view(-1, 1)).any(-1).sum())
        self.count += target.numel()

    def compute(self):
        return self.correct / max(self.count, 1)

    def reset(self):
        self.correct, self.count = 0, 0


class RunningAverage:
    """Exponential running average ``v = alpha*v + (1-alpha)*x`` with bias correction."""

    def __init__(self, alpha: float = 0.98):
        self.alpha, self.v, self.n = alpha, 0.0, 0

    def update(self, x: float) -> float:
        self.n += 1
        self.v = self.alpha * self.v + (1 - self.alpha) * x
        return self.value()

    def value(self) -> float:
        return self.v / (1 - self.alpha ** self.n) if self.n else 0.0


# ----------------------------------------------------------------------------------------------------------------------
# history
# ----------------------------------------------------------------------------------------------------------------------
class EvalResult(tuple):
    """What :meth:`Learner.evaluate` returns: mean loss and metric values (ferrotorch-train/src/history.rs:97). It is also the plain
    ``(loss, metrics)`` pair, so ``loss, metrics = learner.evaluate(data)`` keeps working."""

    def __new__(cls, loss: float, metrics: Optional[Dict[str, float]] = None):
        return super().__new__(cls, (float(loss), dict(metrics or {})))

    @classmethod
    def new_with_defaults(cls, loss: float) -> "EvalResult":
        return cls(loss, {})

    loss = property(lambda self: self[0])
    metrics = property(lambda self: self[1])

    def __str__(self):
        return "".join([f"eval_loss={self.loss:.6f}"] + [f", {k}={v:.6f}" for k, v in self.metrics.items()])


LossFn = Callable[[torch.Tensor, torch.Tensor], torch.Tensor]      # (output, target) -> scalar loss (ferrotorch-train/src/learner.rs:45)


@dataclass
class EpochResult:
    epoch: int
    train_loss: float
    val_loss: Optional[float] = None
    metrics: Dict[str, float] = field(default_factory=dict)
    seconds: float = 0.0
    lr: Optional[float] = None


@dataclass
class TrainingHistory:
    epochs: List[EpochResult] = field(default_factory=list)

    def push(self, r: EpochResult) -> None:
        self.epochs.append(r)

    def best(self, key: str = "val_loss", mode: str = "min") -> Optional[EpochResult]:
        vals = [(getattr(e, key, None) if hasattr(e, key) else e.metrics.get(key), e) for e in self.epochs]
        vals = [(v, e) for v, e in vals if v is not None]
        if not vals:
            return None
        return (min if mode == "min" else max)(vals, key=lambda t: t[0])[1]

    def losses(self) -> List[float]:
        return [e.train_loss for e in self.epochs]


# ----------------------------------------------------------------------------------------------------------------------
# callbacks
# ----------------------------------------------------------------------------------------------------------------------
class Callback:
    def on_train_start(self, learner): ...
    def on_train_end(self, learner): ...
    def on_epoch_start(self, learner, epoch: int): ...
    def on_epoch_end(self, learner, epoch: int, result: EpochResult): ...
    def on_batch_start(self, learner, step: int): ...
    def on_batch_end(self, learner, step: int, loss: float): ...

    def should_stop(self) -> bool:
        return False


class EarlyStopping(Callback):
    def __init__(self, patience: int = 5, min_delta: float = 0.0, monitor: str = "val_loss", mode: str = "min"):
        self.patience, self.min_delta, self.monitor, self.mode = patience, min_delta, monitor, mode
        self.best, self.bad, self._stop = None, 0, False

    def on_epoch_end(self, learner, epoch, result):
        v = getattr(result, self.monitor, None)
        if v is None:
            v = result.metrics.get(self.monitor, result.train_loss)
        better = self.best is None or (v < self.best - self.min_delta if self.mode == "min" else v > self.best + self.min_delta)
        if better:
            self.best, self.bad = v, 0
        else:
            self.bad += 1
            self._stop = self.bad >= self.patience

    def should_stop(self):
        return self._stop


class ProgressLogger(Callback):
    def __init__(self, every: int = 50, printer: Callable[[str], None] = print):
        self.every, self.printer, self.avg = every, printer, RunningAverage()

    def on_batch_end(self, learner, step, loss):
        a = self.avg.update(loss)
        if self.every and step % self.every == 0:
            self.printer(f"step {step}: loss {loss:.4f} (avg {a:.4f})")

    def on_epoch_end(self, learner, epoch, result):
        extra = " ".join(f"{k}={v:.4f}" for k, v in result.metrics.items())
        self.printer(f"epoch {epoch}: train_loss {result.train_loss:.4f}" + (f" val_loss {result.val_loss:.4f}" if result.val_loss is not None else "") + (" " + extra if extra else "") + f" [{result.seconds:.1f}s]")


class EmaCallback(Callback):
    def __init__(self, decay: float = 0.999):
        self.decay, self.ema = decay, None

    def on_train_start(self, learner):
        from ..optim import ExponentialMovingAverage
        self.ema = ExponentialMovingAverage(learner.model.parameters(), self.decay)

    def on_batch_end(self, learner, step, loss):
        self.ema.update()


# ----------------------------------------------------------------------------------------------------------------------
# AMP
# ----------------------------------------------------------------------------------------------------------------------
class AmpContext:
    """Autocast + loss scaling bundle: ``with amp.autocast(): ...; amp.backward(loss); amp.step(opt)``."""

    def __init__(self, dtype: torch.dtype = torch.bfloat16, enabled: bool = True, device_type: str = "cuda", scaler=None):
        from ..optim import GradScaler, GradScalerConfig
        self.dtype, self.enabled, self.device_type = dtype, enabled, device_type
        self.scaler = scaler or GradScaler(GradScalerConfig(enabled=enabled and dtype == torch.float16))

    def autocast(self):
        if not self.enabled:
            return contextlib.nullcontext()
        return torch.autocast(self.device_type, dtype=self.dtype)

    def backward(self, loss: torch.Tensor) -> None:
        self.scaler.scale(loss).backward()

    def step(self, optimizer) -> None:
        self.scaler.step(optimizer)
        self.scaler.update()


def checkpoint_sequential(functions: Sequence[Callable], segments: int, x: torch.Tensor, use_reentrant: bool = False) -> torch.Tensor:
    """Run a stack in ``segments`` chunks, keeping only the chunk inputs and recomputing inside each chunk during backward."""
    fns = list(functions)
    per = math.ceil(len(fns) / max(1, segments))

    def run(lo, hi):
        def f(inp):
            for fn in fns[lo:hi]:
                inp = fn(inp)
            return inp
        return f
    for lo in range(0, len(fns), per):
        hi = min(len(fns), lo + per)
        x = _ckpt(run(lo, hi), x, use_reentrant=use_reentrant) if (x.requires_grad or torch.is_grad_enabled()) else run(lo, hi)(x)
    return x


# ----------------------------------------------------------------------------------------------------------------------
# TensorBoard event files
# ----------------------------------------------------------------------------------------------------------------------
def _crc32c_table():
    poly, tab = 0x82F63B78, []
    for i in range(256):
        c = i
        for _ in range(8):
            c = (c >> 1) ^ poly if c & 1 else c >> 1
        tab.append(c)
    return tab


_CRC = _crc32c_table()


def crc32c(data: bytes) -> int:
    c = 0xFFFFFFFF
    for b in data:
        c = _CRC[(c ^ b) & 0xFF] ^ (c >> 8)
    return c ^ 0xFFFFFFFF


def _masked_crc(data: bytes) -> int:
    c = crc32c(data)
    return (((c >> 15) | (c << 17)) + 0xA282EAD8) & 0xFFFFFFFF


def _varint(n: int) -> bytes:
    out = bytearray()
    while True:
        b = n & 0x7F
        n >>= 7
        out.append(b | (0x80 if n else 0))
        if not n:
            return bytes(out)


def _ld(num: int, data: bytes) -> bytes:
    return _varint((num << 3) | 2) + _varint(len(data)) + data


class TensorBoardWriter:
    """Writes ``events.out.tfevents.*`` files that TensorBoard reads: scalars, text, histograms."""

    def __init__(self, log_dir, filename_suffix: str = ""):
        self.dir = Path(log_dir)
        self.dir.mkdir(parents=True, exist_ok=True)
        self.path = self.dir / f"events.out.tfevents.{int(time.time())}.{socket.gethostname()}{filename_suffix}"
        self.f = open(self.path, "ab")
        self._event(_varint((3 << 3) | 2) + _varint(len(b"brain.Event:2")) + b"brain.Event:2", 0)

    def _record(self, data: bytes) -> None:
        hdr = struct.pack("<Q", len(data))
        self.f.write(hdr + struct.pack("<I", _masked_crc(hdr)) + data + struct.pack("<I", _masked_crc(data)))

    def _event(self, payload: bytes, step: int) -> None:
        ev = _varint((1 << 3) | 1) + struct.pack("<d", time.time()) + _varint((2 << 3) | 0) + _varint(step) + payload
        self._record(ev)

    def add_scalar(self, tag: str, value: float, step: int) -> None:
        val = _ld(1, tag.encode()) + _varint((2 << 3) | 5) + struct.pack("<f", float(value))
        self._event(_ld(5, _ld(1, val)), step)

    def add_scalars(self, prefix: str, values: Dict[str, float], step: int) -> None:
        for k, v in values.items():
            self.add_scalar(f"{prefix}/{k}", v, step)

    def add_histogram(self, tag: str, values: torch.Tensor, step: int, bins: int = 30) -> None:
        v = values.detach().float().flatten().cpu()
        lo, hi = float(v.min()), float(v.max())
        hi = hi if hi > lo else lo + 1e-6
        counts = torch.histc(v, bins=bins, min=lo, max=hi)
        edges = torch.linspace(lo, hi, bins + 1)[1:]
        h = (_varint((1 << 3) | 1) + struct.pack("<d", lo) + _varint((2 << 3) | 1) + struct.pack("<d", hi) + _varint((3 << 3) | 1) + struct.pack("<d", float(v.numel()))
             + _varint((4 << 3) | 1) + struct.pack("<d", float(v.sum())) + _varint((5 << 3) | 1) + struct.pack("<d", float((v * v).sum()))
             + _ld(6, b"".join(struct.pack("<d", float(e)) for e in edges)) + _ld(7, b"".join(struct.pack("<d", float(c)) for c in counts)))
        self._event(_ld(5, _ld(1, _ld(1, tag.encode()) + _ld(5, h))), step)

    def add_text(self, tag: str, text: str, step: int = 0) -> None:
        tensor = _varint((1 << 3) | 0) + _varint(7) + _ld(8, text.encode())
        meta = _ld(1, _ld(1, b"text"))
        self._event(_ld(5, _ld(1, _ld(1, tag.encode()) + _ld(9, meta) + _ld(8, tensor))), step)

    def flush(self) -> None:
        self.f.flush()

    def close(self) -> None:
        self.f.flush()
        self.f.close()


class TensorBoardCallback(Callback):
    def __init__(self, log_dir, every: int = 10):
        self.writer, self.every = TensorBoardWriter(log_dir), every

    def on_batch_end(self, learner, step, loss):
        if step % self.every == 0:
            self.writer.add_scalar("train/loss", loss, step)

    def on_epoch_end(self, learner, epoch, result):
        if result.val_loss is not None:
            self.writer.add_scalar("val/loss", result.val_loss, epoch)
        for k, v in result.metrics.items():
            self.writer.add_scalar(f"val/{k}", v, epoch)
        self.writer.flush()

    def on_train_end(self, learner):
        self.writer.close()


# ----------------------------------------------------------------------------------------------------------------------
# learner
# ----------------------------------------------------------------------------------------------------------------------
class Learner:
    """``Learner(model, optimizer, loss_fn).fit(train_data, epochs, val_data)``; data sources are callables or iterables yielding
    ``(input, target)`` batches. One ``loss.item()`` per step is the only host sync in the loop."""

    def __init__(self, model: torch.nn.Module, optimizer: torch.optim.Optimizer, loss_fn: Callable, scheduler=None,
                 metrics: Optional[List[Metric]] = None, callbacks: Optional[List[Callback]] = None, amp: Optional[AmpContext] = None,
                 grad_clip: Optional[float] = None, device=None):
        self.model, self.optimizer, self.loss_fn, self.scheduler = model, optimizer, loss_fn, scheduler
        self.metrics, self.callbacks = metrics or [], callbacks or []
        self.amp, self.grad_clip, self.device = amp, grad_clip, device
        self.history = TrainingHistory()
        self.epoch, self.step = 0, 0
        self.checkpoint_dir: Optional[Path] = None

    def with_checkpointing(self, directory) -> "Learner":
        self.checkpoint_dir = Path(directory)
        self.checkpoint_dir.mkdir(parents=True, exist_ok=True)
        return self

    def with_callback(self, cb: Callback) -> "Learner":
        self.callbacks.append(cb)
        return self

    def with_metric(self, m: Metric) -> "Learner":
        self.metrics.append(m)
        return self

    def _batches(self, data):
        it = data() if callable(data) else data
        for b in it:
            x, y = b[0], b[1]
            if self.device is not None:
                x, y = x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)
            yield x, y

    def load_checkpoint(self, path) -> None:
        ck = TrainingCheckpoint.load(path)
        self.model.load_state_dict(ck.model_state)
        if ck.optimizer_state:
            self.optimizer.load_state_dict(ck.optimizer_state)
        self.epoch, self.step = ck.epoch + 1, ck.step        # resume with the epoch after the one that was saved

    def _save(self, epoch: int) -> None:
        if self.checkpoint_dir is None:
            return
        try:
            TrainingCheckpoint(self.model.state_dict(), self.optimizer.state_dict(), epoch, self.step).save(
                self.checkpoint_dir / f"checkpoint_epoch_{epoch}.ftc")
        except OSError:
            pass        # a failed checkpoint write must not kill the run (the reference swallows it as well)

    def fit(self, train_data, epochs: int, val_data=None) -> TrainingHistory:
        for cb in self.callbacks:
            cb.on_train_start(self)
        start_epoch = self.epoch
        for epoch in range(start_epoch, start_epoch + epochs):
            t0 = time.time()
            for cb in self.callbacks:
                cb.on_epoch_start(self, epoch)
            self.model.train()
            tot, n = 0.0, 0
            for x, y in self._batches(train_data):
                for cb in self.callbacks:
                    cb.on_batch_start(self, self.step)
                self.optimizer.zero_grad(set_to_none=True)
                ctx = self.amp.autocast() if self.amp else contextlib.nullcontext()
                with ctx:
                    loss = self.loss_fn(self.model(x), y)
                if self.amp:
                    self.amp.backward(loss)
                    if self.grad_clip:
                        self.amp.scaler.unscale_(self.optimizer)
                else:
                    loss.backward()
                if self.grad_clip:
                    from ..nn import clip_grad_norm_
                    clip_grad_norm_(self.model.parameters(), self.grad_clip)
                if self.amp:
                    self.amp.step(self.optimizer)
                else:
                    self.optimizer.step()
                lv = float(loss.item())
                tot, n = tot + lv, n + 1
                self.step += 1
                for cb in self.callbacks:
                    cb.on_batch_end(self, self.step, lv)
            if self.scheduler is not None:
                self.scheduler.step()
            res = EpochResult(epoch, tot / max(n, 1), seconds=time.time() - t0, lr=self.optimizer.param_groups[0]["lr"])
            if val_data is not None:
                res.val_loss, res.metrics = self.evaluate(val_data)
            self.history.push(res)
            self.epoch = epoch + 1
            self._save(epoch)
            for cb in self.callbacks:
                cb.on_epoch_end(self, epoch, res)
            if any(cb.should_stop() for cb in self.callbacks):
                break
        for cb in self.callbacks:
            cb.on_train_end(self)
        return self.history

    @torch.no_grad()
    def evaluate(self, data) -> EvalResult:
        self.model.eval()
        for m in self.metrics:
            m.reset()
        tot, n = 0.0, 0
        for x, y in self._batches(data):
            out = self.model(x)
            lv = float(self.loss_fn(out, y).item())
            tot, n = tot + lv, n + 1
            for m in self.metrics:
                m.update(out, y, lv)
        return EvalResult(tot / max(n, 1), {m.name: m.compute() for m in self.metrics})


# the reference re-exports these at the crate root (ferrotorch-train/src/lib.rs)
from ..core import checkpoint  # noqa: E402
from ..nn.utils import clip_grad_norm_, clip_grad_value_  # noqa: E402
