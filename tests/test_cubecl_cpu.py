"""Device-side GGUF block dequantisation and DFA token masking, checked on the host against the file-format reader and a per-token walk."""
import struct

import numpy as np
import pytest
import torch

from ferrotorch_b200 import cubecl as Q
from ferrotorch_b200.errors import DeviceUnavailable, InvalidArgument, ShapeMismatch
from ferrotorch_b200.serialize import dequantize_gguf


def _client():
    return Q.CubeRuntime.new(Q.CubeDevice.Cuda(0), allow_host=True).client()


def test_runtime_variants():
    for d in (Q.CubeDevice.Wgpu(0), Q.CubeDevice.Rocm(1)):
        assert not d.is_available()
        with pytest.raises(DeviceUnavailable):
            Q.CubeRuntime.new(d)
    if not torch.cuda.is_available():
        with pytest.raises(DeviceUnavailable):
            Q.CubeRuntime.new(Q.CubeDevice.Cuda(0))
    rt = Q.CubeRuntime.new(Q.CubeDevice.Cuda(0), allow_host=True)
    h = Q.upload_f32([1.0, 2.0, 3.0], rt)
    assert h.len() == 3 and h.read_to_host().tolist() == [1.0, 2.0, 3.0] and Q.cubecl_handle_of(h) is h and Q.cubecl_handle_of(3) is None
    w = Q.wrap_kernel_output(torch.arange(6.0), [2, 3], rt)
    assert w.tensor.shape == (2, 3) and rt.device() == Q.CubeDevice.Cuda(0)
    with pytest.raises(ShapeMismatch):
        Q.wrap_kernel_output(torch.arange(6.0), [4], rt)


@pytest.mark.parametrize("kind,ggml", [("Q4_0", 2), ("Q4_1", 3), ("Q5_0", 6), ("Q5_1", 7), ("Q8_0", 8)])
def test_block_dequantisation_matches_the_file_reader(kind, ggml):
    k = Q.GgufBlockKind[kind]
    rng = np.random.default_rng(0)
    nb = 5
    raw = bytearray(rng.integers(0, 256, nb * k.block_bytes(), dtype=np.uint8).tobytes())
    for b in range(nb):                                       # finite f16 scale / min at the head of every block
        raw[b * k.block_bytes(): b * k.block_bytes() + 2] = np.float16(rng.uniform(0.01, 2.0)).tobytes()
        if kind in ("Q4_1", "Q5_1"):
            raw[b * k.block_bytes() + 2: b * k.block_bytes() + 4] = np.float16(rng.uniform(-1.0, 1.0)).tobytes()
    want = dequantize_gguf(bytes(raw), ggml, nb * 32)
    got = Q.dequantize_blocks_to_gpu(_client(), k, bytes(raw), nb * 32)
    assert got.dtype == torch.float32 and torch.allclose(got, want, atol=1e-6)
    assert torch.equal(Q.dequantize_blocks_to_gpu(_client(), k, bytes(raw), nb * 32 - 7), got[: nb * 32 - 7])      # ragged tail
    with pytest.raises(InvalidArgument):
        Q.dequantize_blocks_to_gpu(_client(), k, bytes(raw)[:-1], nb * 32)


def test_q8_1_f32_header_layout_and_size_checks():
    vals = np.arange(-16, 16, dtype=np.int8)
    raw = struct.pack("<ff", 0.5, 2.0) + vals.tobytes()
    s, m, p = Q.split_q8_1_blocks(raw, 1)
    assert s.tolist() == [0.5] and m.tolist() == [2.0] and len(p) == 8 and Q.GgufBlockKind.Q8_1.block_bytes() == 40
    out = Q.dequantize_q8_1_to_gpu(_client(), s, m, p, 32)
    assert torch.equal(out, torch.from_numpy(vals.astype(np.float32)) * 0.5 + 2.0)
    sc, nib = Q.split_q4_0_blocks(np.float16(1.0).tobytes() + bytes([0x21] * 16), 1)
    assert nib.tolist() == [0x21212121] * 4
    deq = Q.dequantize_q4_0_to_gpu(_client(), sc, nib, 32)
    assert deq[:16].tolist() == [1 - 8] * 16 and deq[16:].tolist() == [2 - 8] * 16          # low nibbles first, then high nibbles
    with pytest.raises(ShapeMismatch):
        Q.dequantize_q4_0_to_gpu(_client(), sc, nib[:3], 32)
    with pytest.raises(InvalidArgument):
        Q.dequantize_q4_0_to_gpu(_client(), sc, nib, 33)


def _json_bool_dfa():
    """DFA for the literals ``true`` / ``false`` and every prefix of them: states are positions in the two words."""
    words = ["true", "false"]
    classes = {c: i + 1 for i, c in enumerate(sorted(set("".join(words))))}       # class 0 = every other ASCII character
    states = {"": 0}
    for w in words:
        for i in range(1, len(w) + 1):
            states.setdefault(w[:i], len(states))
    reject = len(states)
    C = len(classes) + 1
    T = [reject] * ((reject + 1) * C)
    for pre, s in states.items():
        for w in words:
            if w.startswith(pre) and len(w) > len(pre):
                T[s * C + classes[w[len(pre)]]] = states[w[: len(pre) + 1]]
    cc = [classes.get(chr(i), 0) for i in range(128)]
    return T, cc, C, states, reject


def test_dfa_token_mask_matches_a_per_token_walk():
    T, cc, C, states, reject = _json_bool_dfa()
    vocab = ["t", "tr", "true", "rue", "fal", "false", "x", "", "trué", "e", "ue", "se", "truex"]
    offs, chars = [0], []
    for tok in vocab:
        chars += [ord(c) for c in tok]
        offs.append(len(chars))
    inp = Q.DfaMaskInputs.new(T, cc, offs, chars, C, 0, reject, 5)

    def walk(tok, s):
        for ch in tok:
            s = reject if ord(ch) >= 128 or s == reject else T[s * C + cc[ord(ch)]]
        return int(s != reject)
    for start_name in ("", "tr", "fals"):
        s0 = states[start_name]
        allow, V = Q.compute_token_mask_dfa_to_gpu(_client(), inp, s0)
        assert V == len(vocab) and allow.dtype == torch.int32 and allow.tolist() == [walk(t, s0) for t in vocab], start_name
    allow, _ = Q.compute_token_mask_dfa_to_gpu(_client(), inp)
    assert [v for v, a in zip(vocab, allow.tolist()) if a] == ["t", "tr", "true", "fal", "false", ""]
    dev_state, _ = Q.compute_token_mask_dfa_to_gpu(_client(), inp, torch.tensor([states["tr"]]))          # state held in a device tensor
    assert [v for v, a in zip(vocab, dev_state.tolist()) if a] == ["", "ue"]
    for bad in (dict(char_classes=cc[:100]), dict(vocab_offsets=offs[:-1]), dict(start_state=99), dict(max_token_len=3), dict(transitions=T[:-1])):
        kw = dict(transitions=T, char_classes=cc, vocab_offsets=offs, vocab_chars=chars, num_classes=C, start_state=0, reject_state=reject, max_token_len=5)
        kw.update(bad)
        with pytest.raises(InvalidArgument):
            Q.DfaMaskInputs.new(**kw)


def test_per_format_split_and_dequantise_entry_points():
    """The per-format pair (``split_*_blocks`` -> ``dequantize_*_to_gpu``) for every format against the file-format reader."""
    rng = np.random.default_rng(1)
    nb = 3

    def blocks(kind, with_min):
        k = Q.GgufBlockKind[kind]
        raw = bytearray(rng.integers(0, 256, nb * k.block_bytes(), dtype=np.uint8).tobytes())
        for b in range(nb):
            raw[b * k.block_bytes(): b * k.block_bytes() + 2] = np.float16(rng.uniform(0.01, 2.0)).tobytes()
            if with_min:
                raw[b * k.block_bytes() + 2: b * k.block_bytes() + 4] = np.float16(rng.uniform(-1.0, 1.0)).tobytes()
        return bytes(raw)
    c = _client()
    assert isinstance(c, Q.CubeClient)
    raw = blocks("Q4_1", True)
    s, m, nib = Q.split_q4_1_blocks(raw, nb)
    assert len(s) == len(m) == nb and len(nib) == 4 * nb
    assert torch.allclose(Q.dequantize_q4_1_to_gpu(c, s, m, nib, nb * 32), dequantize_gguf(raw, 3, nb * 32), atol=1e-6)
    raw = blocks("Q5_0", False)
    s, qh, nib = Q.split_q5_0_blocks(raw, nb)
    assert len(qh) == nb and len(nib) == 4 * nb
    assert torch.allclose(Q.dequantize_q5_0_to_gpu(c, s, qh, nib, nb * 32), dequantize_gguf(raw, 6, nb * 32), atol=1e-6)
    raw = blocks("Q5_1", True)
    s, m, qh, nib = Q.split_q5_1_blocks(raw, nb)
    assert torch.allclose(Q.dequantize_q5_1_to_gpu(c, s, m, qh, nib, nb * 32), dequantize_gguf(raw, 7, nb * 32), atol=1e-6)
    raw = blocks("Q8_0", False)
    s, packed = Q.split_q8_0_blocks(raw, nb)
    assert len(packed) == 8 * nb
    out = Q.dequantize_q8_0_to_gpu(c, s, packed, nb * 32)
    assert torch.allclose(out, dequantize_gguf(raw, 8, nb * 32), atol=1e-6)
    h = Q.wrap_kernel_output(out, [nb, 32], Q.CubeRuntime.new(Q.CubeDevice.Cuda(0), allow_host=True))
    assert isinstance(h, Q.CubeclStorageHandle) and h.len() == nb * 32


def test_dfa_walk_kernel_on_raw_tables():
    T, cc, C, states, reject = _json_bool_dfa()
    vocab = ["tr", "ue", "x", "false"]
    offs, chars = [0], []
    for tok in vocab:
        chars += [ord(ch) for ch in tok]
        offs.append(len(chars))
    lt = lambda a: torch.tensor(a, dtype=torch.long)     # noqa: E731
    allow = torch.empty(len(vocab), dtype=torch.int32)
    Q.kernel_compute_token_mask_dfa(lt(T), lt(cc), lt(offs), lt(chars), allow, C, 0, reject, 5)
    assert allow.tolist() == [1, 0, 0, 1]
    Q.kernel_compute_token_mask_dfa(lt(T), lt(cc), lt(offs), lt(chars), allow, C, torch.tensor([states["tr"]]), reject, 5)
    assert allow.tolist() == [0, 1, 0, 0]
