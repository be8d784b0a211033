"""Byte-level checks of the native state-dict / checkpoint layout against the reference's documented format, the pickle-free RPC payload
codec, and optimizer steps on parameters whose memory is not row-major."""
import json
import pickle
import struct

import pytest
import torch

from ferrotorch_b200 import errors
from ferrotorch_b200.serialize import formats as F


def test_state_dict_bytes_are_the_reference_layout(tmp_path):
    # ferrotorch-serialize/src/state_dict.rs:59-161: compact JSON line per tensor (name, shape, dtype, byte_offset, byte_length), names
    # sorted, every line newline-terminated, "\n---\n", raw little-endian bodies in header order
    w = torch.tensor([[1.0, 2.0], [3.0, 4.0]])
    b = torch.tensor([0.5, -0.5], dtype=torch.float64)
    fixture = (b'{"name":"b","shape":[2],"dtype":"f64","byte_offset":0,"byte_length":16}\n'
               b'{"name":"w","shape":[2,2],"dtype":"f32","byte_offset":16,"byte_length":16}\n'
               b"\n---\n" + b.numpy().tobytes() + w.numpy().tobytes())
    assert F.dumps_state_dict({"w": w, "b": b}) == fixture          # insertion order does not matter: names are sorted
    back = F.loads_state_dict(fixture)
    assert torch.equal(back["w"], w) and torch.equal(back["b"], b) and back["b"].dtype == torch.float64
    # files of the earlier layout of this package still load
    legacy = (json.dumps({"name": "w", "dtype": "F32", "shape": [2, 2], "offset": 0, "nbytes": 16}).encode() + b"\n---\n" + w.numpy().tobytes())
    assert torch.equal(F.loads_state_dict(legacy)["w"], w)
    with pytest.raises(errors.InvalidArgument):
        F.loads_state_dict(fixture[:-4])                            # body shorter than the header says
    half = torch.randn(5).bfloat16()
    assert torch.equal(F.loads_state_dict(F.dumps_state_dict({"h": half}))["h"], half)


def test_checkpoint_sections_have_the_reference_shape(tmp_path):
    m = torch.nn.Linear(3, 2)
    opt = torch.optim.AdamW(m.parameters(), lr=1e-3, betas=(0.8, 0.9))
    m(torch.randn(4, 3)).sum().backward()
    opt.step()
    path = tmp_path / "c.ftc"
    F.save_checkpoint(path, m, opt, epoch=2, step=7)
    data = path.read_bytes()
    (n1,) = struct.unpack_from("<Q", data, 0)
    assert data[8:8 + n1] == b'{"epoch":2,"step":7}'               # checkpoint.rs:86-90
    (n2,) = struct.unpack_from("<Q", data, 8 + n1)
    sec2 = json.loads(data[16 + n1:16 + n1 + n2])
    # checkpoint.rs:198-229: {"<key>": {"<name>": [numbers]}} and nothing else, keys sorted
    assert list(sec2) == sorted(sec2)
    for inner in sec2.values():
        assert isinstance(inner, dict) and all(isinstance(v, list) and all(isinstance(x, (int, float)) for x in v) for v in inner.values())
    assert sec2["0"]["step"] == [1] and len(sec2["0"]["exp_avg"]) == 6
    ck = F.TrainingCheckpoint.load(path)
    opt2 = torch.optim.AdamW(m.parameters(), lr=9.0)
    opt2.load_state_dict(ck.optimizer_state)
    assert opt2.param_groups[0]["lr"] == 1e-3 and opt2.param_groups[0]["betas"] == (0.8, 0.9)
    a, b = opt.state_dict()["state"], opt2.state_dict()["state"]
    assert all(torch.equal(a[k]["exp_avg_sq"], b[k]["exp_avg_sq"]) and a[k]["exp_avg"].shape == b[k]["exp_avg"].shape for k in a)
    # a section that already has the reference's shape passes through unchanged
    F.TrainingCheckpoint({"w": torch.ones(2)}, {"p0": {"momentum": [0.5, 0.25]}}, 1, 2, {"note": "x"}).save(path)
    ck = F.TrainingCheckpoint.load(path)
    assert ck.optimizer_state == {"p0": {"momentum": [0.5, 0.25]}} and ck.extra == {"note": "x"} and (ck.epoch, ck.step) == (1, 2)


def test_rpc_payloads_are_parsed_never_executed():
    from ferrotorch_b200.distributed.extras import wire_dumps, wire_loads
    msg = ("call", "f", (1, -5, 2 ** 70, 3.5, "x", b"y", [torch.arange(6).reshape(2, 3), torch.randn(3).bfloat16()], None, True), {"k": {"a": (1, 2)}})
    back = wire_loads(wire_dumps(msg))
    assert back[:2] == msg[:2] and back[2][:6] == msg[2][:6] and back[2][7:] == (None, True) and back[3] == msg[3]
    assert torch.equal(back[2][6][0], msg[2][6][0]) and torch.equal(back[2][6][1], msg[2][6][1])

    class Evil:
        def __reduce__(self):
            return (print, ("executed",))
    with pytest.raises(errors.InvalidArgument):
        wire_loads(pickle.dumps(Evil()))                            # a pickle stream is just an unknown tag
    with pytest.raises(errors.InvalidArgument):
        wire_dumps(Evil())                                          # and objects cannot be sent
    with pytest.raises(errors.InvalidArgument):
        wire_loads(wire_dumps([1, 2, 3])[:-2])                      # truncated
    deep = []
    for _ in range(200):
        deep = [deep]
    with pytest.raises(errors.InvalidArgument):
        wire_dumps(deep)


def test_rpc_round_trip_over_the_simulated_backend():
    import threading
    from ferrotorch_b200.distributed import SimulatedBackend
    from ferrotorch_b200.distributed.extras import RpcAgent
    bs = SimulatedBackend.create_group(2)
    server, client = RpcAgent(bs[1]), RpcAgent(bs[0])
    server.register("scale", lambda t, k=2: t * k)
    th = threading.Thread(target=lambda: server.serve(0, idle_timeout=5.0))
    th.start()
    out = client.rpc_sync(1, "scale", torch.arange(4.0), k=3)
    with pytest.raises(errors.WorkerPanic):
        client.rpc_sync(1, "missing")
    client.shutdown(1)
    th.join(10)
    assert torch.equal(out, torch.arange(4.0) * 3)


@pytest.mark.parametrize("amsgrad", [False, True])
def test_adamw_updates_channels_last_parameters(amsgrad):
    from ferrotorch_b200.optim import AdamW
    torch.manual_seed(0)
    ours = torch.nn.Conv2d(3, 4, 3).to(memory_format=torch.channels_last)
    theirs = torch.nn.Conv2d(3, 4, 3)
    theirs.load_state_dict(ours.state_dict())
    o1, o2 = AdamW(ours.parameters(), lr=1e-2, amsgrad=amsgrad), torch.optim.AdamW(theirs.parameters(), lr=1e-2, amsgrad=amsgrad)
    x = torch.randn(2, 3, 8, 8)
    for _ in range(3):
        for c, o in ((ours, o1), (theirs, o2)):
            o.zero_grad()
            c(x).pow(2).sum().backward()
            o.step()
    assert ours.weight.is_contiguous(memory_format=torch.channels_last)
    assert torch.allclose(ours.weight, theirs.weight, atol=1e-6) and torch.allclose(ours.bias, theirs.bias, atol=1e-6)
