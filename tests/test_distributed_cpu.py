"""CPU control plane: backends, collectives, DDP (world size 2 over TCP, MLP 784-256-10), failure detection on the host."""
import multiprocessing as mp
import os
import threading
import time

import pytest
import torch

import ferrotorch_b200.distributed as fd
from ferrotorch_b200 import errors


def _threads(world, fn):
    backs = fd.SimulatedBackend.create_group(world)
    out, errs = [None] * world, []

    def run(r):
        try:
            out[r] = fn(backs[r], r)
        except BaseException as e:  # noqa
            errs.append(e)
    ts = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    if errs:
        raise errs[0]
    return out


@pytest.mark.parametrize("world", [1, 2, 4])
@pytest.mark.parametrize("algo", ["star", "ring"])
def test_allreduce_sum_mean(world, algo):
    def fn(b, r):
        x = torch.arange(10, dtype=torch.float32) + r
        return fd.allreduce(x, b, fd.ReduceOp.Sum, algorithm=algo), fd.allreduce(x, b, fd.ReduceOp.Mean, algorithm=algo)
    res = _threads(world, fn)
    exp = sum(torch.arange(10, dtype=torch.float32) + r for r in range(world))
    for s, m in res:
        assert torch.equal(s, exp)
        assert torch.allclose(m, exp / world)
    for s, m in res[1:]:
        assert torch.equal(m, res[0][1])       # bit-identical on every rank


def test_all_gather_reduce_scatter_all_to_all_broadcast():
    world = 4

    def fn(b, r):
        x = torch.full((2, 3), float(r))
        g = fd.all_gather(x, b)
        s = fd.all_gather(torch.tensor(float(r)), b)
        rs = fd.reduce_scatter(torch.arange(8, dtype=torch.float32).reshape(8, 1) * (r + 1), b, fd.ReduceOp.Sum)
        a2a = fd.all_to_all(torch.arange(4, dtype=torch.float32) + 10 * r, b)
        bc = fd.broadcast(torch.full((3,), float(r)), b, root=2)
        bt = fd.broadcast(torch.full((3,), float(r)), b, root=1, algorithm="tree")
        return g, s, rs, a2a, bc, bt
    res = _threads(world, fn)
    for r, (g, s, rs, a2a, bc, bt) in enumerate(res):
        assert g.shape == (8, 3) and torch.equal(g[::2, 0], torch.arange(4.0))
        assert torch.equal(s, torch.arange(4.0))
        assert torch.equal(rs.flatten(), torch.arange(8.0)[2 * r: 2 * r + 2] * 10)
        assert torch.equal(a2a, torch.tensor([r + 10.0 * p for p in range(4)]))
        assert torch.equal(bc, torch.full((3,), 2.0)) and torch.equal(bt, torch.full((3,), 1.0))


def test_world1_identity_and_empty_and_errors():
    (b,) = fd.SimulatedBackend.create_group(1)
    x = torch.randn(4, 2)
    assert torch.equal(fd.allreduce(x, b, fd.ReduceOp.Mean), x)
    assert torch.equal(fd.all_gather(x, b), x)
    assert fd.all_gather(torch.empty(0, 3), b).shape == (0, 3)
    b2 = fd.SimulatedBackend.create_group(2)
    with pytest.raises(errors.ShapeMismatch):
        fd.reduce_scatter(torch.zeros(3, 2), b2[0])
    with pytest.raises(errors.SelfSend):
        b2[0].send(b"x", 0)
    with pytest.raises(errors.InvalidRank):
        b2[0].send(b"x", 5)


def test_recv_timeout_and_fault_injection():
    a, b = fd.SimulatedBackend.create_group(2)
    t0 = time.time()
    with pytest.raises(errors.Timeout):
        a.recv_timeout(4, 1, 0.2)
    assert 0.15 < time.time() - t0 < 2.0
    # a dropped message: the receiver's collective times out instead of hanging
    b.inject_fault(fd.FAULT_DROP_NEXT_SEND)
    b.send(b"abcd", 0)
    with pytest.raises(errors.Timeout):
        a.recv_timeout(4, 1, 0.2)
    # a corrupted frame length is reported as a size mismatch
    b.inject_fault(fd.FAULT_CORRUPT_LENGTH)
    b.send(b"abcd", 0)
    with pytest.raises(errors.SizeMismatch):
        a.recv_timeout(4, 1, 1.0)
    # a closed channel is reported as such
    b.inject_fault(fd.FAULT_CLOSE)
    with pytest.raises(errors.ChannelClosed):
        b.send(b"abcd", 0)
    with pytest.raises(errors.ChannelClosed):
        a.recv_timeout(4, 1, 1.0)


def test_rank_that_never_joins_times_out_collective():
    backs = fd.SimulatedBackend.create_group(2)
    with pytest.raises(errors.Timeout):
        fd.allreduce(torch.ones(4), backs[1], fd.ReduceOp.Sum, timeout=0.3)   # rank 0 never shows up


def test_sub_backend_and_async():
    def fn(b, r):
        if r in (1, 3):
            sub = fd.SubBackend(b, [1, 3])
            return fd.allreduce(torch.tensor([float(r)]), sub, fd.ReduceOp.Sum)
        return None
    res = _threads(4, fn)
    assert res[1].item() == 4.0 and res[3].item() == 4.0

    def fn2(b, r):
        h = fd.async_all_gather(torch.tensor([float(r)]), b)
        return h.wait(10)
    res = _threads(2, fn2)
    assert torch.equal(res[0], torch.tensor([0.0, 1.0]))


def test_bucket_plan_reverse_order():
    ps = [torch.zeros(10), torch.zeros(20), torch.zeros(30), torch.zeros(5)]
    assert fd.compute_buckets(ps, bucket_size_bytes=4 * 35) == [[3, 2], [1, 0]]
    assert fd.compute_buckets(ps, bucket_size_bytes=1) == [[3], [2], [1], [0]]


def _mlp(seed=0):
    torch.manual_seed(seed)
    m = torch.nn.Sequential(torch.nn.Linear(784, 256), torch.nn.ReLU(), torch.nn.Linear(256, 10))
    for l in (m[0], m[2]):
        torch.nn.init.kaiming_uniform_(l.weight, nonlinearity="relu")   # the reference's Linear init: Kaiming-uniform, ReLU gain, zero bias
        torch.nn.init.zeros_(l.bias)
    return m


def _ddp_worker(rank, world, port, q):
    torch.set_num_threads(1)
    backend = fd.TcpBackend(rank, world, f"127.0.0.1:{port}")
    model = _mlp(0)
    ddp = fd.DDP(model, backend)
    ddp.broadcast_parameters(0)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    g = torch.Generator().manual_seed(1234)
    X = torch.randn(100, 128, 784, generator=g)
    Y = torch.randint(0, 10, (100, 128), generator=g)
    grads = None
    for step in range(100):
        x, y = X[step, rank * 64:(rank + 1) * 64], Y[step, rank * 64:(rank + 1) * 64]
        opt.zero_grad()
        loss = torch.nn.functional.cross_entropy(ddp(x), y)
        loss.backward()
        ddp.sync_gradients()
        if step == 99:
            grads = [p.grad.numpy().copy() for p in model.parameters()]
        opt.step()
    q.put((rank, [p.detach().numpy().copy() for p in model.parameters()], grads))
    backend.barrier()


def test_config1_ddp_world2_tcp_matches_single_process():
    """World size 2 over TCP, MLP 784->256->10, batch 64 per rank, SGD lr 0.01 momentum 0.9, 100 steps: gradients and
    parameters bit-identical across ranks and within 1e-5 of single-process batch-128 training."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29800 + os.getpid() % 100
    ps = [ctx.Process(target=_ddp_worker, args=(r, 2, port, q)) for r in range(2)]
    [p.start() for p in ps]
    got = {}
    for _ in range(2):
        r, params, grads = q.get(timeout=180)
        got[r] = (params, grads)
    [p.join(30) for p in ps]
    import numpy as np
    for a, b in zip(got[0][0], got[1][0]):
        assert np.array_equal(a, b)
    for a, b in zip(got[0][1], got[1][1]):
        assert np.array_equal(a, b)
    # single process, batch 128
    torch.set_num_threads(1)
    model = _mlp(0)
    opt = torch.optim.SGD(model.parameters(), lr=0.01, momentum=0.9)
    g = torch.Generator().manual_seed(1234)
    X = torch.randn(100, 128, 784, generator=g)
    Y = torch.randint(0, 10, (100, 128), generator=g)
    for step in range(100):
        opt.zero_grad()
        torch.nn.functional.cross_entropy(model(X[step]), Y[step]).backward()
        opt.step()
    for a, b in zip(got[0][0], model.parameters()):
        assert np.abs(a - b.detach().numpy()).max() < 1e-5


def test_device_mesh_and_dtensor_redistribute():
    mesh = fd.DeviceMesh([2, 2], ["dp", "tp"])
    assert mesh.coordinates(3) == (1, 1) and mesh.rank_of((1, 0)) == 2
    assert mesh.group_ranks(1, "dp") == [1, 3] and mesh.group_ranks(2, "tp") == [2, 3]
    full = torch.arange(24.).reshape(4, 6)

    def fn(b, r):
        dt = fd.DTensor.from_full(full, b, fd.Shard(1))
        assert dt.local.shape == (4, 3) and dt.full_shape() == (4, 6)
        rep = dt.redistribute(fd.Replicate())
        part = fd.DTensor(torch.full((2, 2), float(r + 1)), b, fd.Partial())
        rs = part.redistribute(fd.Shard(0))
        return rep.local, dt.redistribute(fd.Shard(0)).local, part.redistribute(fd.Replicate()).local, rs.local
    res = _threads(2, fn)
    for r, (rep, s0, ar, rs) in enumerate(res):
        assert torch.equal(rep, full) and torch.equal(s0, full[2 * r:2 * r + 2])
        assert torch.equal(ar, torch.full((2, 2), 3.0)) and torch.equal(rs, torch.full((1, 2), 3.0))


@pytest.mark.parametrize("sched", [fd.PipelineSchedule.GPipe, fd.PipelineSchedule.OneFOneB])
def test_pipeline_matches_single_process(sched):
    torch.manual_seed(0)
    s0, s1 = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh()), torch.nn.Linear(8, 3)
    x, y = torch.randn(8, 6), torch.randn(8, 3)
    ref0, ref1 = torch.nn.Sequential(torch.nn.Linear(6, 8), torch.nn.Tanh()), torch.nn.Linear(8, 3)
    ref0.load_state_dict(s0.state_dict()); ref1.load_state_dict(s1.state_dict())
    torch.nn.functional.mse_loss(ref1(ref0(x)), y).backward()

    def fn(b, r):
        p = fd.Pipeline(s0 if r == 0 else s1, b, 4, sched, timeout=20)
        return p.step(x if r == 0 else None, y if r == 1 else None, torch.nn.functional.mse_loss)
    res = _threads(2, fn)
    assert res[1] is not None
    assert torch.allclose(s0[0].weight.grad, ref0[0].weight.grad, atol=1e-5)       # a real gradient reached the first stage
    assert torch.allclose(s1.weight.grad, ref1.weight.grad, atol=1e-5)


def test_rpc_roundtrip_and_remote_error():
    def fn(b, r):
        ag = fd.RpcAgent(b, timeout=10)
        if r == 1:
            ag.register("add", lambda a, c: a + c)
            ag.register("boom", lambda: 1 / 0)
            return ag.serve(0)
        out = ag.rpc_sync(1, "add", torch.ones(3), 2)
        fut = ag.rpc_async(1, "add", 1, 2)
        v = fut.wait(10)
        try:
            ag.rpc_sync(1, "boom")
            bad = False
        except errors.WorkerPanic:
            bad = True
        ag.shutdown(1)
        return out, v, bad
    res = _threads(2, fn)
    assert torch.equal(res[0][0], torch.full((3,), 3.0)) and res[0][1] == 3 and res[0][2] and res[1] == 3


@pytest.mark.parametrize("strategy", [fd.ShardingStrategy.FullShard, fd.ShardingStrategy.ShardGradOp, fd.ShardingStrategy.NoShard])
def test_cpu_fsdp_matches_averaged_gradients(strategy):
    torch.manual_seed(1)
    base = torch.nn.Linear(4, 2)
    xs = [torch.randn(3, 4), torch.randn(3, 4)]
    ref = torch.nn.Linear(4, 2)
    ref.load_state_dict(base.state_dict())
    (ref(xs[0]).sum() / 2 + ref(xs[1]).sum() / 2).backward()

    def fn(b, r):
        m = torch.nn.Linear(4, 2)
        m.load_state_dict(base.state_dict())
        f = fd.FSDP(m, b, strategy, timeout=20)
        f(xs[r]).sum().backward()
        f.sync_gradients()
        return [s.grad.clone() for s in f.shard_parameters()]
    res = _threads(2, fn)
    full_w = ref.weight.grad.reshape(-1)
    if strategy == fd.ShardingStrategy.NoShard:
        assert torch.allclose(res[0][0], full_w, atol=1e-6)
    else:
        assert torch.allclose(torch.cat([res[0][0], res[1][0]]), full_w, atol=1e-6)


def test_distributed_checkpoint_reshards_on_world_change(tmp_path):
    full = {"w": torch.arange(24.).reshape(6, 4), "b": torch.arange(6.)}
    for r in range(2):
        fd.save_distributed(tmp_path, {k: v.chunk(2, 0)[r] for k, v in full.items()}, r, 2)
    same = fd.load_distributed(tmp_path, 1, 2)
    assert torch.equal(same["w"], full["w"][3:])
    parts = [fd.load_distributed(tmp_path, r, 3) for r in range(3)]
    assert torch.equal(torch.cat([p["w"] for p in parts]), full["w"]) and torch.equal(torch.cat([p["b"] for p in parts]), full["b"])
    ck = fd.AsyncCheckpointer()
    ck.save_async(tmp_path / "a", {"w": full["w"]}, 0, 1).wait(10)
    assert torch.equal(fd.load_distributed(tmp_path / "a", 0, 1)["w"], full["w"])


def _tp_worker(rank, world, port, q):
    import torch.distributed as dist
    from ferrotorch_b200.parallel import ColumnParallelLinear, ParallelEmbedding, RowParallelLinear
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        M, D, Fd = 8 * world, 16, 24
        w1, w2, x = torch.randn(Fd, D), torch.randn(D, Fd), torch.randn(M, D)
        col = ColumnParallelLinear(D, Fd, dtype=torch.float32)
        row = RowParallelLinear(Fd, D, dtype=torch.float32)
        col.load_full_weight(w1)
        row.load_full_weight(w2)
        xs = x[rank * (M // world): (rank + 1) * (M // world)]
        y = row(col(xs))
        ref = (x @ w1.t() @ w2.t())[rank * (M // world): (rank + 1) * (M // world)]
        emb = ParallelEmbedding(10 * world, 4, dtype=torch.float32)
        full = torch.arange(10 * world * 4, dtype=torch.float32).view(10 * world, 4)
        emb.load_full_weight(full)
        ids = torch.tensor([[0, 10 * world - 1, 7], [3, 11 % (10 * world), 5]])
        q.put((rank, float((y - ref).abs().max()), bool(torch.equal(emb(ids), full[ids]))))
    finally:
        dist.destroy_process_group()


def test_tensor_parallel_layers_world2_gloo():
    """Column/row-parallel linears (sequence-parallel) and the vocabulary-parallel embedding over a CPU group equal the dense computation."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29741
    ps = [ctx.Process(target=_tp_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(60)
        assert p.exitcode == 0
    for rank, err, emb_ok in res:
        assert err < 1e-4 and emb_ok, (rank, err, emb_ok)


def _cp_worker(rank, world, port, q):
    import torch.distributed as dist
    from ferrotorch_b200.parallel import UlyssesAttention, ring_attention
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        S, Hq, Hkv, D = 16 * world, 4, 2, 8
        Q, K, V = torch.randn(S, Hq, D), torch.randn(S, Hkv, D), torch.randn(S, Hkv, D)
        sl = slice(rank * (S // world), (rank + 1) * (S // world))
        errs = []
        for causal in (True, False):
            rep = Hq // Hkv
            ref = torch.nn.functional.scaled_dot_product_attention(Q.transpose(0, 1)[None], K.repeat_interleave(rep, 1).transpose(0, 1)[None],
                                                                   V.repeat_interleave(rep, 1).transpose(0, 1)[None], is_causal=causal)[0].transpose(0, 1)[sl]
            ql = Q[sl].clone().requires_grad_()
            u = UlyssesAttention(causal=causal)(ql, K[sl], V[sl])
            u.sum().backward()
            errs.append(float((u - ref).abs().max()))
            errs.append(float((ring_attention(Q[sl], K[sl], V[sl], causal=causal) - ref).abs().max()))
            assert ql.grad is not None and ql.grad.shape == ql.shape
        q.put((rank, max(errs)))
    finally:
        dist.destroy_process_group()


def test_ulysses_and_ring_attention_world2_gloo():
    """Sequence-parallel attention (head exchange and K/V ring) equals dense attention on the gathered sequence, causal and not."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_cp_worker, args=(r, 2, 29743, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(60)
        assert p.exitcode == 0
    for rank, err in res:
        assert err < 1e-5, (rank, err)


def test_heartbeat_failure_detection_and_elastic_restart(tmp_path):
    """Three rank threads train; rank 2 stops between steps (no GPU involved). The survivors notice through the heartbeat store within the
    timeout, re-rendezvous as a world of two with new ranks, and reload the distributed checkpoint re-sharded for the new world."""
    import threading
    from ferrotorch_b200.distributed import load_distributed, save_distributed
    from ferrotorch_b200.distributed.elastic import DistributedMonitor, ElasticCoordinator, HeartbeatMonitor, MemoryStore, RankFailure, resume_from_checkpoint
    store = MemoryStore()
    full = torch.arange(24, dtype=torch.float32).view(6, 4)
    for r in range(3):
        save_distributed(str(tmp_path), {"w": full[r * 2:(r + 1) * 2].clone()}, r, 3, {"w": 0})
    results, errors = {}, []

    def rank_fn(rank):
        try:
            hb = HeartbeatMonitor(store, rank, 3, interval_s=0.01, timeout_s=0.15).start()
            if rank == 2:
                time.sleep(0.05)
                hb.stop()                                  # "dies" between steps: stops heartbeating and never joins again
                return
            t0 = time.monotonic()
            failed = None
            while time.monotonic() - t0 < 5:
                try:
                    hb.check()
                except RankFailure as e:
                    failed = e.ranks
                    break
                time.sleep(0.01)
            hb.stop()
            assert failed == [2], failed
            m = ElasticCoordinator(store, min_world=2, timeout_s=5).rendezvous(rank, 3, failed, generation=0)
            state = resume_from_checkpoint(str(tmp_path), m)
            results[rank] = (m, state["w"], time.monotonic() - t0)
        except Exception as e:                             # noqa: BLE001
            errors.append((rank, repr(e)))
    import time
    ts = [threading.Thread(target=rank_fn, args=(r,)) for r in range(3)]
    for t in ts:
        t.start()
    for t in ts:
        t.join(20)
    assert not errors, errors
    assert set(results) == {0, 1}
    for old in (0, 1):
        m, w, dt = results[old]
        assert (m.generation, m.rank, m.world, m.old_ranks) == (1, old, 2, [0, 1]) and dt < 2.0
        assert torch.equal(w, full[old * 3:(old + 1) * 3])                 # 6 rows over 2 ranks now
    with pytest.raises(Exception):
        ElasticCoordinator(store, min_world=3).rendezvous(0, 3, [2], 0)
    with pytest.raises(Exception):
        ElasticCoordinator(MemoryStore(), timeout_s=0.1).rendezvous(0, 3, [2], 0)   # rank 1 never joins -> Timeout, not a hang
    mon = DistributedMonitor("tokens", roofline_ms=1.0)
    for _ in range(3):
        with mon.span("step"):
            with mon.span("compute"):
                time.sleep(0.002)
            with mon.span("comm"):
                time.sleep(0.001)
        mon.end_step(1000)
    s = mon.summary(skip=1)
    assert s["tokens_per_s"] > 0 and 0 < s["comm_to_compute"] < 2 and 0 < s["fraction_of_roofline"] < 1


def test_comm_trace_decoding_and_chrome_events():
    """The phase-stamp ring of the collective kernels, decoded on the host: empty and torn records are dropped, phases add up."""
    from ferrotorch_b200.parallel.symm import CommTrace
    ring = [0] * (4 * CommTrace.WORDS)
    ring[0:5] = [7 | (1 << 32), 1_000_000, 1_004_000, 1_054_000, 1_056_000]          # all-reduce, launch 7
    ring[5:10] = [8 | (8 << 32), 2_000_000, 2_001_000, 2_301_000, 2_302_500]         # fused FSDP kernel, launch 8
    ring[10:15] = [9 | (3 << 32), 3_000_000, 2_999_000, 0, 0]                        # torn: still running when the ring was read
    recs = CommTrace.decode(ring)
    assert [r["kind"] for r in recs] == ["all_reduce", "fsdp_rs_adamw_ag"] and recs[0]["seq"] == 7
    assert recs[0]["wait_peers_us"] == 4.0 and recs[0]["body_us"] == 50.0 and recs[0]["drain_us"] == 2.0 and recs[0]["total_us"] == 56.0
    ev = CommTrace.chrome_events(recs, pid=3)
    assert len(ev) == 6 and ev[0]["name"] == "all_reduce:wait_peers" and ev[1]["ts"] == 1004.0 and ev[5]["dur"] == 1.5 and ev[0]["pid"] == 3


def test_cpu_fsdp_hybrid_shard_world4_nodes_of_2():
    """HybridShard on 4 ranks with nodes of 2: shards live inside a node (contiguous ranks), are replicated across nodes (strided ranks),
    and the shard gradients are the global mean."""
    torch.manual_seed(3)
    base = torch.nn.Linear(4, 2)
    xs = [torch.randn(3, 4) for _ in range(4)]
    ref = torch.nn.Linear(4, 2)
    ref.load_state_dict(base.state_dict())
    sum(ref(x).sum() / 4 for x in xs).backward()

    def fn(b, r):
        m = torch.nn.Linear(4, 2)
        m.load_state_dict(base.state_dict())
        f = fd.FSDP(m, b, fd.ShardingStrategy.HybridShard, timeout=20, intra_node_size=2)
        assert f.shard_world == 2 and f.shard_rank == r % 2 and f.shard_parameters()[0].numel() == 4
        f(xs[r]).sum().backward()
        f.sync_gradients()
        return [s.grad.clone() for s in f.shard_parameters()], [s.detach().clone() for s in f.shard_parameters()]
    res = _threads(4, fn)
    full_w = ref.weight.grad.reshape(-1)
    for node in range(2):
        assert torch.allclose(torch.cat([res[2 * node][0][0], res[2 * node + 1][0][0]]), full_w, atol=1e-6)
    assert torch.equal(res[0][1][0], res[2][1][0]) and torch.equal(res[1][1][0], res[3][1][0])          # replicas across nodes
    assert torch.equal(res[0][0][0], res[2][0][0])                                                         # and their gradients
    with pytest.raises(Exception):
        _threads(4, lambda b, r: fd.FSDP(torch.nn.Linear(4, 2), b, fd.ShardingStrategy.HybridShard, intra_node_size=3))


def _syncbn_worker(rank, world, port, q):
    import torch.distributed as dist
    from ferrotorch_b200 import nn
    from ferrotorch_b200.parallel import SyncBatchNorm2d
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        full = torch.randn(4 * world, 6, 5, 5) * 2 + 1                     # the batch of all ranks; this rank holds its slice
        w = torch.randn(4 * world, 6, 5, 5)
        ref_bn = torch.nn.BatchNorm2d(6)
        with torch.no_grad():
            ref_bn.weight.uniform_(0.5, 1.5)
            ref_bn.bias.uniform_(-0.5, 0.5)
        plain = nn.Sequential(nn.Conv2d(6, 6, 1), nn.BatchNorm2d(6))
        plain[1].load_state_dict(ref_bn.state_dict())
        conv = SyncBatchNorm2d.convert(plain)
        assert isinstance(conv[1], SyncBatchNorm2d) and isinstance(conv[0], nn.Conv2d) and conv[1].training
        sbn = conv[1]
        sl = slice(4 * rank, 4 * (rank + 1))
        x = full[sl].clone().requires_grad_()
        y = sbn(x)
        (y * w[sl]).sum().backward()
        xr = full.clone().requires_grad_()
        yr = ref_bn(xr)
        (yr * w).sum().backward()
        errs = (float((y - yr[sl]).abs().max()), float((x.grad - xr.grad[sl]).abs().max()),
                float((sbn.running_mean - ref_bn.running_mean).abs().max()), float((sbn.running_var - ref_bn.running_var).abs().max()))
        gw = sbn.weight.grad.clone()
        dist.all_reduce(gw)                                                # parameter gradients are local sums: DDP adds them up
        errs += (float((gw - ref_bn.weight.grad).abs().max()),)
        sbn.eval()
        errs += (float((sbn(full[sl]) - ref_bn.eval()(full[sl])).abs().max()),)
        q.put((rank, errs, int(sbn.num_batches_tracked)))
    finally:
        dist.destroy_process_group()


def test_sync_batch_norm_world2_gloo_equals_batch_norm_over_the_global_batch():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    ps = [ctx.Process(target=_syncbn_worker, args=(r, 2, 29747, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = [q.get(timeout=120) for _ in ps]
    for p in ps:
        p.join(60)
        assert p.exitcode == 0
    for rank, errs, tracked in res:
        assert max(errs) < 1e-4 and tracked == 1, (rank, errs, tracked)
