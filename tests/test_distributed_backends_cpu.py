"""Process-group backends (gloo ranks on CPU), bounded receives, the RPC byte transport and the distributed-checkpoint object."""
import multiprocessing as mp
import os
import traceback

import pytest
import torch

from ferrotorch_b200 import distributed as D
from ferrotorch_b200 import errors as E


def _gloo_worker(rank, world, port, q):
    try:
        torch.set_num_threads(1)
        b = D.GlooBackend(rank, world, f"tcp://127.0.0.1:{port}", timeout=30.0)
        out = {"rank": b.rank(), "world": b.world_size()}
        peer = 1 - rank
        # bytes both ways (lower rank sends first)
        if rank == 0:
            b.send(b"hello from 0", peer)
            out["bytes"] = b.recv(12, peer)
        else:
            out["bytes"] = b.recv(12, peer)
            b.send(b"hello from 1", peer)
        t = torch.arange(6.0) + 10 * rank
        out["allreduce"] = b.allreduce_(t.clone(), D.ReduceOp.Sum).tolist()
        out["max"] = b.allreduce_(t.clone(), D.ReduceOp.Max).tolist()
        out["bcast"] = b.broadcast_(t.clone(), 1).tolist()
        out["gather"] = b.all_gather_into(torch.empty(12), t).tolist()
        out["rs"] = b.reduce_scatter_into(torch.empty(3), t).tolist()
        out["gpu_allreduce"] = D.gpu_allreduce(t, b).tolist()            # no NCCL here: the staged path over the same group
        out["gpu_broadcast"] = D.gpu_broadcast(t, b, 0).tolist()
        # tensor receive with a deadline that is met, then one that cannot be met (nobody sends)
        if rank == 0:
            b.send_tensor(torch.full((2, 2), 7.0), peer)
        else:
            buf = torch.zeros(2, 2)
            D.recv_into_with_timeout(buf, peer, b, 10.0)
            out["recv_into"] = buf.tolist()
        b.barrier()
        if rank == 1:
            try:
                D.recv_with_timeout((4,), torch.float32, peer, b, 0.5)
                out["timeout"] = "no error"
            except E.Timeout:
                out["timeout"] = "Timeout"
            except E.FerrotorchError as e:
                out["timeout"] = type(e).__name__ + ": " + str(e)
        for bad, name in ((5, "InvalidRank"), (rank, "SelfSend")):
            try:
                D.recv_into(torch.zeros(1), bad, b)
            except E.FerrotorchError as e:
                out[name] = type(e).__name__
        try:
            D.nccl_allreduce(t, b)
        except E.InvalidArgument as e:
            out["needs_nccl"] = "NcclBackend" in str(e)
        q.put(out)
        if rank == 0:
            import time
            time.sleep(2.0)                                  # stay connected while rank 1 lets its deadline pass
    except BaseException:
        q.put({"rank": rank, "error": traceback.format_exc()})
    finally:
        q.close()
        q.join_thread()                                      # flush the result before leaving
        os._exit(0)                                          # the unmet receive leaves gloo with a pending operation: skip its teardown


def test_gloo_backend_two_ranks():
    assert D.is_gloo_available()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 200
    ps = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    got = {}
    for _ in range(2):
        o = q.get(timeout=120)
        assert "error" not in o, o.get("error")
        got[o["rank"]] = o
    [p.join(30) for p in ps]
    a, b = got[0], got[1]
    assert a["bytes"] == b"hello from 1" and b["bytes"] == b"hello from 0" and a["world"] == 2
    base = [float(i) for i in range(6)]
    for o in (a, b):
        assert o["allreduce"] == [2 * v + 10 for v in base] == o["gpu_allreduce"] and o["max"] == [v + 10 for v in base]
        assert o["bcast"] == [v + 10 for v in base] and o["gpu_broadcast"] == base and o["gather"] == base + [v + 10 for v in base]
        assert o["InvalidRank"] == "InvalidRank" and o["SelfSend"] == "SelfSend" and o["needs_nccl"] is True
    assert a["rs"] == [10.0, 12.0, 14.0] and b["rs"] == [16.0, 18.0, 20.0]
    assert b["recv_into"] == [[7.0, 7.0], [7.0, 7.0]] and b["timeout"] == "Timeout"


def test_unavailable_backends_say_so():
    assert D.is_mpi_available() is False or True
    if not D.is_mpi_available():
        with pytest.raises(E.BackendUnavailable):
            D.MpiBackend(0, 1)
    if not D.is_nccl_available():
        with pytest.raises(E.BackendUnavailable):
            D.NcclBackend(0, 1)
        with pytest.raises(E.BackendUnavailable):
            D.NcclUniqueId.generate()
    uid = D.NcclUniqueId.from_bytes(bytes(range(128)))
    assert uid.to_bytes() == bytes(range(128)) and D.NcclUniqueId.from_bytes(uid.to_bytes()) == uid
    with pytest.raises(E.InvalidArgument):
        D.NcclUniqueId(b"short")


def test_rpc_transport_and_errors():
    sim = D.SimulatedBackend.create_group(2)
    a, b = D.TcpRpcBackend(sim[0]), D.TcpRpcBackend(sim[1])
    a.send(b"payload", 1)
    assert b.recv(7, 0) == b"payload" and (a.rank(), b.rank(), a.world_size()) == (0, 1, 2)
    with pytest.raises(D.RpcError) as e:
        b.recv((1 << 30) + 1, 0)
    assert e.value.kind == "invalid_message" and "1 GiB" in str(e.value)
    with pytest.raises(D.RpcError) as e:
        b.recv(4, 0, timeout=0.2)
    assert e.value.kind == "timeout"
    assert D.RpcError.function_not_found("f").kind == "function_not_found" and "rank 3" in str(D.RpcError.no_connection(3))
    assert isinstance(D.RpcError.internal("x"), E.InvalidArgument)


def test_distributed_checkpoint_object(tmp_path):
    world = 2
    shards = [{"flat": torch.arange(4.0) + 4 * r, "bias": torch.full((3,), float(r))} for r in range(world)]
    meta = D.flat_shard_metadata(shards[0], world)
    assert meta.num_ranks == 2 and meta.tensor_specs["flat"].full_shape == [8] and meta.tensor_specs["bias"].shard_sizes == [3, 3]
    ck = D.DistributedCheckpoint(tmp_path / "ck", meta)
    for r in range(world):
        ck.save(shards[r], r)
    again = D.DistributedCheckpoint.open(tmp_path / "ck")
    assert again.shard_metadata.tensor_specs["flat"].full_shape == [8]
    assert torch.equal(again.load(1)["flat"], shards[1]["flat"])
    whole = again.load(0, world_size=1)
    assert torch.equal(whole["flat"], torch.arange(8.0)) and whole["bias"].tolist() == [0, 0, 0, 1, 1, 1]
    quarter = again.load(3, world_size=4)
    assert quarter["flat"].tolist() == [6.0, 7.0]
    with pytest.raises(D.DistCheckpointError) as e:
        ck.save({"flat": torch.zeros(5), "bias": torch.zeros(3)}, 0)
    assert e.value.kind == "tensor"
    with pytest.raises(D.DistCheckpointError) as e:
        ck.save({"other": torch.zeros(1)}, 0)
    assert e.value.kind == "metadata"
    (tmp_path / "ck" / "rank_1.safetensors").unlink()
    with pytest.raises(D.DistCheckpointError) as e:
        again.load(0, world_size=1)
    assert e.value.kind == "missing_shard" and "shard file missing" in str(e.value)
    with pytest.raises(D.DistCheckpointError) as e:
        D.DistributedCheckpoint.open(tmp_path / "nowhere")
    assert e.value.kind == "io"
    with pytest.raises(D.DistCheckpointError):
        D.flat_shard_metadata(shards[0], 0)
    assert D.CheckpointFuture is not None
