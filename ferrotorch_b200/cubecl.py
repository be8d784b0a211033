"""Device-side GGUF block dequantisation and DFA token masking, with the runtime / storage handle types of the reference's portable-GPU crate.

The reference reaches these through CubeCL so that one kernel source serves CUDA, ROCm and wgpu. This framework targets CUDA (sm_100a) only:
:class:`CubeDevice` keeps the three variants for source compatibility, but only ``Cuda`` can be opened; the others raise
``DeviceUnavailable``. The operations upload the split host buffers once, unpack and scale on the device, and return a device tensor that is
never read back — the point of the path is that quantised weights go from file bytes to device floats without a host-side f32 copy. They
are written with stream-ordered tensor primitives (shifts, masks, gathers), so the same code also runs on a CPU tensor, which is how the CPU
test tier checks the arithmetic.

Reference parity: ferrotorch-cubecl/src/{runtime.rs:31 (CubeDevice, CubeRuntime, CubeClient), storage.rs:36-206, quant.rs:47-900 (block
splitters and ``dequantize_*_to_gpu``), grammar.rs:37-300 (DfaMaskInputs, kernel_compute_token_mask_dfa, compute_token_mask_dfa_to_gpu)}.
"""
from __future__ import annotations

import enum
from dataclasses import dataclass
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from .errors import DeviceUnavailable, InvalidArgument, ShapeMismatch


# -- runtime ---------------------------------------------------------------------------------------------------------------------
@dataclass(frozen=True)
class CubeDevice:
    kind: str
    ordinal: int = 0

    @classmethod
    def Cuda(cls, ordinal: int = 0): return cls("cuda", ordinal)      # noqa: E704,N802
    @classmethod
    def Wgpu(cls, ordinal: int = 0): return cls("wgpu", ordinal)      # noqa: E704,N802
    @classmethod
    def Rocm(cls, ordinal: int = 0): return cls("rocm", ordinal)      # noqa: E704,N802

    def is_available(self) -> bool:
        return self.kind == "cuda" and torch.cuda.is_available() and self.ordinal < torch.cuda.device_count()


class CubeClient:
    """Handle on one opened device: uploads host data and reads device tensors back."""

    def __init__(self, device: torch.device):
        self.device = device

    def create(self, data, dtype=None) -> torch.Tensor:
        return torch.as_tensor(np.asarray(data), dtype=dtype).to(self.device, non_blocking=True)

    def read_one(self, t: torch.Tensor) -> np.ndarray:
        return t.detach().cpu().numpy()


class CubeRuntime:
    """``CubeRuntime.new(CubeDevice.Cuda(0))`` opens the CUDA device; ``Wgpu`` / ``Rocm`` devices do not exist in this framework."""

    def __init__(self, device: CubeDevice, _torch_device: torch.device):
        self._device, self._td = device, _torch_device

    @classmethod
    def new(cls, device: CubeDevice, allow_host: bool = False) -> "CubeRuntime":
        if device.kind != "cuda":
            raise DeviceUnavailable(f"the {device.kind} runtime is not part of this framework (CUDA sm_100a only)")
        if not device.is_available():
            if allow_host:
                return cls(device, torch.device("cpu"))
            raise DeviceUnavailable(f"CUDA device {device.ordinal} is not available")
        return cls(device, torch.device("cuda", device.ordinal))

    def device(self) -> CubeDevice:
        return self._device

    def client(self) -> CubeClient:
        return CubeClient(self._td)


@dataclass
class CubeclStorageHandle:
    """A device allocation produced by one of the operations below, with the runtime that owns it (storage.rs:36)."""
    tensor: torch.Tensor
    runtime: CubeRuntime
    ordinal: int = 0

    def len(self) -> int:  # noqa: A003
        return self.tensor.numel()

    def read_to_host(self) -> np.ndarray:
        return self.runtime.client().read_one(self.tensor)


def upload_f32(data: Sequence[float], runtime: CubeRuntime, ordinal: int = 0) -> CubeclStorageHandle:
    return CubeclStorageHandle(runtime.client().create(np.asarray(data, dtype=np.float32)), runtime, ordinal)


def wrap_kernel_output(tensor: torch.Tensor, shape: Sequence[int], runtime: CubeRuntime, ordinal: int = 0) -> CubeclStorageHandle:
    n = int(np.prod(shape)) if len(shape) else 1
    if tensor.numel() != n:
        raise ShapeMismatch(f"wrap_kernel_output: {tensor.numel()} elements for shape {list(shape)}")
    return CubeclStorageHandle(tensor.reshape(tuple(shape)), runtime, ordinal)


def cubecl_handle_of(t) -> Optional[CubeclStorageHandle]:
    """The storage handle behind a value, when it has one."""
    return t if isinstance(t, CubeclStorageHandle) else None


# -- GGUF block layouts ---------------------------------------------------------------------------------------------------------------
class GgufBlockKind(enum.Enum):
    Q4_0 = "Q4_0"
    Q4_1 = "Q4_1"
    Q5_0 = "Q5_0"
    Q5_1 = "Q5_1"
    Q8_0 = "Q8_0"
    Q8_1 = "Q8_1"

    def block_size(self) -> int:
        return 32

    def block_bytes(self) -> int:
        """Bytes per block of 32 weights. ``Q8_1`` is the layout with f32 scale and f32 min (40 bytes), as the reference reads it."""
        return {"Q4_0": 18, "Q4_1": 20, "Q5_0": 22, "Q5_1": 24, "Q8_0": 34, "Q8_1": 40}[self.value]


def _blocks(raw, num_blocks: int, kind: GgufBlockKind) -> np.ndarray:
    b = np.frombuffer(bytes(raw), dtype=np.uint8)
    need = num_blocks * kind.block_bytes()
    if b.size < need:
        raise InvalidArgument(f"{kind.value}: {b.size} bytes for {num_blocks} blocks of {kind.block_bytes()} bytes")
    return b[:need].reshape(num_blocks, kind.block_bytes())


def _f16(col: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(col).view(np.float16).astype(np.float32).reshape(-1)


def _u32(cols: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(cols).view("<u4").reshape(-1)


def split_q4_0_blocks(raw, num_blocks: int) -> Tuple[np.ndarray, np.ndarray]:
    """``(scales f32 [B], packed nibbles u32 [4 B])`` of 18-byte blocks: f16 scale, 16 bytes holding 32 nibbles."""
    b = _blocks(raw, num_blocks, GgufBlockKind.Q4_0)
    return _f16(b[:, 0:2]), _u32(b[:, 2:18])


def split_q4_1_blocks(raw, num_blocks: int):
    b = _blocks(raw, num_blocks, GgufBlockKind.Q4_1)
    return _f16(b[:, 0:2]), _f16(b[:, 2:4]), _u32(b[:, 4:20])


def split_q5_0_blocks(raw, num_blocks: int):
    """``(scales, qh u32 [B], nibbles u32 [4 B])``: bit ``i`` of ``qh`` is the fifth bit of weight ``i``."""
    b = _blocks(raw, num_blocks, GgufBlockKind.Q5_0)
    return _f16(b[:, 0:2]), _u32(b[:, 2:6]), _u32(b[:, 6:22])


def split_q5_1_blocks(raw, num_blocks: int):
    b = _blocks(raw, num_blocks, GgufBlockKind.Q5_1)
    return _f16(b[:, 0:2]), _f16(b[:, 2:4]), _u32(b[:, 4:8]), _u32(b[:, 8:24])


def split_q8_0_blocks(raw, num_blocks: int):
    """``(scales, int8 values packed four to a u32 [8 B])``."""
    b = _blocks(raw, num_blocks, GgufBlockKind.Q8_0)
    return _f16(b[:, 0:2]), _u32(b[:, 2:34])


def split_q8_1_blocks(raw, num_blocks: int):
    b = _blocks(raw, num_blocks, GgufBlockKind.Q8_1)
    return (np.ascontiguousarray(b[:, 0:4]).view("<f4").reshape(-1).copy(), np.ascontiguousarray(b[:, 4:8]).view("<f4").reshape(-1).copy(), _u32(b[:, 8:40]))


def _up(client: CubeClient, a, dtype) -> torch.Tensor:
    t = torch.from_numpy(np.ascontiguousarray(a).astype(np.int64 if dtype == torch.int64 else np.float32, copy=False))
    return t.to(client.device, non_blocking=True)


def _check(num_elements: int, scales, words, words_per_block: int, what: str) -> int:
    nb = len(scales)
    if num_elements > nb * 32 or num_elements <= 0:
        raise InvalidArgument(f"{what}: {num_elements} elements do not fit {nb} blocks of 32")
    if len(words) != nb * words_per_block:
        raise ShapeMismatch(f"{what}: {len(words)} packed words for {nb} blocks, expected {nb * words_per_block}")
    return nb


def _nibbles(client: CubeClient, words, nb: int) -> torch.Tensor:
    """u32 words -> ``[B, 32]`` integers in GGUF order: weight ``i < 16`` is the low nibble of byte ``i``, weight ``16 + i`` its high nibble."""
    w = _up(client, words, torch.int64).view(nb, 4, 1)
    byts = ((w >> torch.arange(0, 32, 8, device=w.device).view(1, 1, 4)) & 0xFF).reshape(nb, 16)
    return torch.cat([byts & 0xF, byts >> 4], 1)


def _high_bits(client: CubeClient, qh, nb: int) -> torch.Tensor:
    return (_up(client, qh, torch.int64).view(nb, 1) >> torch.arange(32, device=client.device).view(1, 32)) & 1


def dequantize_q4_0_to_gpu(client: CubeClient, scales, nibbles, num_elements: int) -> torch.Tensor:
    """``(nibble - 8) * scale`` per weight, produced on the client's device; the result stays there."""
    nb = _check(num_elements, scales, nibbles, 4, "dequantize_q4_0_to_gpu")
    q = _nibbles(client, nibbles, nb)
    return ((q - 8).float() * _up(client, scales, torch.float32).view(nb, 1)).reshape(-1)[:num_elements]


def dequantize_q4_1_to_gpu(client: CubeClient, scales, mins, nibbles, num_elements: int) -> torch.Tensor:
    nb = _check(num_elements, scales, nibbles, 4, "dequantize_q4_1_to_gpu")
    q = _nibbles(client, nibbles, nb)
    return (q.float() * _up(client, scales, torch.float32).view(nb, 1) + _up(client, mins, torch.float32).view(nb, 1)).reshape(-1)[:num_elements]


def dequantize_q5_0_to_gpu(client: CubeClient, scales, qh, nibbles, num_elements: int) -> torch.Tensor:
    nb = _check(num_elements, scales, nibbles, 4, "dequantize_q5_0_to_gpu")
    q = _nibbles(client, nibbles, nb) | (_high_bits(client, qh, nb) << 4)
    return ((q - 16).float() * _up(client, scales, torch.float32).view(nb, 1)).reshape(-1)[:num_elements]


def dequantize_q5_1_to_gpu(client: CubeClient, scales, mins, qh, nibbles, num_elements: int) -> torch.Tensor:
    nb = _check(num_elements, scales, nibbles, 4, "dequantize_q5_1_to_gpu")
    q = _nibbles(client, nibbles, nb) | (_high_bits(client, qh, nb) << 4)
    return (q.float() * _up(client, scales, torch.float32).view(nb, 1) + _up(client, mins, torch.float32).view(nb, 1)).reshape(-1)[:num_elements]


def _int8s(client: CubeClient, words, nb: int) -> torch.Tensor:
    w = _up(client, words, torch.int64).view(nb, 8, 1)
    b = ((w >> torch.arange(0, 32, 8, device=w.device).view(1, 1, 4)) & 0xFF).reshape(nb, 32)
    return torch.where(b >= 128, b - 256, b)


def dequantize_q8_0_to_gpu(client: CubeClient, scales, packed, num_elements: int) -> torch.Tensor:
    nb = _check(num_elements, scales, packed, 8, "dequantize_q8_0_to_gpu")
    return (_int8s(client, packed, nb).float() * _up(client, scales, torch.float32).view(nb, 1)).reshape(-1)[:num_elements]


def dequantize_q8_1_to_gpu(client: CubeClient, scales, mins, packed, num_elements: int) -> torch.Tensor:
    nb = _check(num_elements, scales, packed, 8, "dequantize_q8_1_to_gpu")
    return (_int8s(client, packed, nb).float() * _up(client, scales, torch.float32).view(nb, 1) + _up(client, mins, torch.float32).view(nb, 1)).reshape(-1)[:num_elements]


def dequantize_blocks_to_gpu(client: CubeClient, kind: GgufBlockKind, raw, num_elements: int) -> torch.Tensor:
    """File bytes of one tensor -> device f32, choosing the splitter and the unpacker by ``kind``."""
    nb = -(-num_elements // 32)
    parts = {"Q4_0": split_q4_0_blocks, "Q4_1": split_q4_1_blocks, "Q5_0": split_q5_0_blocks, "Q5_1": split_q5_1_blocks, "Q8_0": split_q8_0_blocks,
             "Q8_1": split_q8_1_blocks}[kind.value](raw, nb)
    fn = {"Q4_0": dequantize_q4_0_to_gpu, "Q4_1": dequantize_q4_1_to_gpu, "Q5_0": dequantize_q5_0_to_gpu, "Q5_1": dequantize_q5_1_to_gpu,
          "Q8_0": dequantize_q8_0_to_gpu, "Q8_1": dequantize_q8_1_to_gpu}[kind.value]
    return fn(client, *parts, num_elements)


# -- DFA token mask (grammar.rs) -------------------------------------------------------------------------------------------------------
@dataclass
class DfaMaskInputs:
    """A compiled DFA over character classes plus the packed vocabulary (grammar.rs:137). ``transitions`` is ``[states, classes]`` flattened
    row-major; ``char_classes`` maps the 128 ASCII code points to classes (any other character rejects); token ``t`` is
    ``vocab_chars[vocab_offsets[t] : vocab_offsets[t + 1]]``."""
    transitions: Sequence[int]
    char_classes: Sequence[int]
    vocab_offsets: Sequence[int]
    vocab_chars: Sequence[int]
    num_classes: int
    start_state: int
    reject_state: int
    max_token_len: int

    @classmethod
    def new(cls, transitions, char_classes, vocab_offsets, vocab_chars, num_classes: int, start_state: int, reject_state: int, max_token_len: int) -> "DfaMaskInputs":
        if num_classes <= 0 or len(transitions) % num_classes:
            raise InvalidArgument(f"DfaMaskInputs: {len(transitions)} transitions do not form rows of {num_classes} classes")
        n_states = len(transitions) // num_classes
        if len(char_classes) != 128:
            raise InvalidArgument(f"DfaMaskInputs: char_classes must have 128 entries, got {len(char_classes)}")
        if len(vocab_offsets) < 1 or vocab_offsets[0] != 0 or vocab_offsets[-1] != len(vocab_chars):
            raise InvalidArgument("DfaMaskInputs: vocab_offsets needs vocab_size + 1 entries, from 0 to len(vocab_chars)")
        if any(b < a for a, b in zip(vocab_offsets, vocab_offsets[1:])):
            raise InvalidArgument("DfaMaskInputs: vocab_offsets must be non-decreasing")
        if not (0 <= start_state < n_states and 0 <= reject_state < n_states):
            raise InvalidArgument(f"DfaMaskInputs: start / reject state outside the {n_states} states")
        if any(not 0 <= c < num_classes for c in char_classes) or any(not 0 <= s < n_states for s in transitions):
            raise InvalidArgument("DfaMaskInputs: a class or a target state is out of range")
        longest = max((b - a for a, b in zip(vocab_offsets, vocab_offsets[1:])), default=0)
        if max_token_len < longest:
            raise InvalidArgument(f"DfaMaskInputs: max_token_len {max_token_len} is below the longest token ({longest})")
        return cls(list(transitions), list(char_classes), list(vocab_offsets), list(vocab_chars), num_classes, start_state, reject_state, max_token_len)

    def vocab_size(self) -> int:
        return len(self.vocab_offsets) - 1


def kernel_compute_token_mask_dfa(transitions: torch.Tensor, char_classes: torch.Tensor, vocab_offsets: torch.Tensor, vocab_chars: torch.Tensor,
                                  allow: torch.Tensor, num_classes: int, start_state, reject_state: int, max_token_len: int) -> None:
    """All tokens walk the DFA in lock step: step ``j`` advances every token that still has a ``j``-th character by one transition
    (a character outside ASCII sends it to the reject state, which is absorbing); ``allow[t] = 1`` iff token ``t`` never reached the reject
    state. ``start_state`` is an int or a one-element device tensor (so that a captured decode step follows the grammar's current state)."""
    V = vocab_offsets.numel() - 1
    dev = transitions.device
    start = vocab_offsets[:-1]
    length = vocab_offsets[1:] - start
    s0 = start_state.reshape(-1)[:1].to(dev) if torch.is_tensor(start_state) else torch.tensor([int(start_state)], device=dev)
    state = s0.expand(V).clone()
    n_chars = max(vocab_chars.numel(), 1)
    chars = vocab_chars if vocab_chars.numel() else torch.zeros(1, dtype=torch.long, device=dev)
    for j in range(int(max_token_len)):
        live = j < length
        ch = chars[(start + j).clamp_max(n_chars - 1)]
        ascii_ = ch < 128
        nxt = transitions[state * num_classes + char_classes[ch.clamp_max(127)]]
        nxt = torch.where(ascii_, nxt, torch.full_like(nxt, reject_state))
        nxt = torch.where(state == reject_state, state, nxt)
        state = torch.where(live, nxt, state)
    allow.copy_((state != reject_state).to(allow.dtype))


def compute_token_mask_dfa_to_gpu(client: CubeClient, inputs: DfaMaskInputs, start_state=None) -> Tuple[torch.Tensor, int]:
    """Uploads the tables, runs the walk on the client's device and returns ``(allow mask as int32 [vocab], vocab_size)``; the mask stays on
    the device, ready for the logits kernel."""
    up = lambda a: torch.as_tensor(np.asarray(a, dtype=np.int64)).to(client.device, non_blocking=True)   # noqa: E731
    allow = torch.empty(inputs.vocab_size(), dtype=torch.int32, device=client.device)
    kernel_compute_token_mask_dfa(up(inputs.transitions), up(inputs.char_classes), up(inputs.vocab_offsets), up(inputs.vocab_chars), allow,
                                  inputs.num_classes, inputs.start_state if start_state is None else start_state, inputs.reject_state, inputs.max_token_len)
    return allow, inputs.vocab_size()
