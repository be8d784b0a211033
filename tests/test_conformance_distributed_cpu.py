"""Per-symbol behaviour checks of ``ferrotorch_b200.distributed`` on in-process simulated ranks: timeouts, asynchronous collectives, uneven
all-to-all, send/receive pairs, resharding records, error types and the device-collective wrappers' argument checks."""
import threading

import pytest
import torch

import ferrotorch_b200.distributed as fd
from ferrotorch_b200 import errors


def _ranks(world, fn):
    backs = fd.SimulatedBackend.create_group(world)
    out, errs = [None] * world, []

    def run(r):
        try:
            out[r] = fn(backs[r], r)
        except BaseException as e:  # noqa: BLE001
            errs.append(e)
    ts = [threading.Thread(target=run, args=(r,)) for r in range(world)]
    [t.start() for t in ts]
    [t.join(30) for t in ts]
    if errs:
        raise errs[0]
    return out


def test_timed_collectives_match_the_untimed_math():
    W = 3

    def fn(b, r):
        x = torch.arange(6, dtype=torch.float32) + r
        ar = fd.allreduce_with_timeout(x.clone(), b, fd.ReduceOp.Sum, 10.0)
        ag = fd.all_gather_with_timeout(torch.full((2,), float(r)), b, 10.0)
        rs = fd.reduce_scatter_with_timeout(x.clone(), b, fd.ReduceOp.Sum, 10.0)
        rs2 = fd.reduce_scatter_tensor(x.clone(), b)
        a2a = fd.all_to_all_with_timeout(torch.arange(W, dtype=torch.float32) + 10 * r, b, 10.0)
        return ar, ag, rs, rs2, a2a
    out = _ranks(W, fn)
    total = sum(torch.arange(6, dtype=torch.float32) + r for r in range(W))
    for r, (ar, ag, rs, rs2, a2a) in enumerate(out):
        assert torch.equal(ar, total)
        assert torch.equal(torch.as_tensor(ag).reshape(-1), torch.tensor([0.0, 0.0, 1.0, 1.0, 2.0, 2.0]))
        assert torch.equal(rs, total[2 * r: 2 * r + 2]) and torch.equal(rs2, rs)
        assert torch.equal(torch.as_tensor(a2a).reshape(-1), torch.tensor([r + 10.0 * p for p in range(W)]))


def test_async_collectives_and_pending_handles():
    def fn(b, r):
        h = fd.async_allreduce(torch.ones(4) * (r + 1), b)
        assert isinstance(h, fd.PendingCollective)
        rs = fd.async_reduce_scatter(torch.arange(4.0), b)
        return h.wait(), rs.wait()
    for r, (ar, rs) in enumerate(_ranks(2, fn)):
        assert torch.equal(ar, torch.full((4,), 3.0)) and torch.equal(rs, 2 * torch.arange(4.0)[2 * r: 2 * r + 2])
    p = fd.PendingCollective(lambda: (_ for _ in ()).throw(ValueError("boom")))
    with pytest.raises(errors.WorkerPanic, match="boom"):
        p.wait()


def test_uneven_all_to_all_and_sendrecv():
    send = {0: [1, 2], 1: [3, 0]}          # rank 0 sends 1 row to itself and 2 to rank 1; rank 1 sends 3 rows to rank 0

    def fn(b, r):
        rows = sum(send[r])
        x = torch.arange(rows * 2, dtype=torch.float32).view(rows, 2) + 100 * r
        recv = [send[p][r] for p in range(2)]
        y = fd.all_to_all_single_uneven(x, send[r], recv, b)
        z = fd.sendrecv(torch.full((3,), float(r)), dst=1 - r, src=1 - r, backend=b)
        return y, z
    (y0, z0), (y1, z1) = _ranks(2, fn)
    assert y0.shape == (4, 2) and torch.equal(y0[0], torch.tensor([0.0, 1.0])) and torch.equal(y0[1:], torch.arange(6.0).view(3, 2) + 100)
    assert y1.shape == (2, 2) and torch.equal(y1, torch.tensor([[2.0, 3.0], [4.0, 5.0]]))
    assert torch.equal(z0, torch.ones(3)) and torch.equal(z1, torch.zeros(3))


def test_reshard_and_shard_records():
    full = torch.arange(10.0).view(5, 2)
    parts = [fd.reshard(full, 0, r, 3) for r in range(3)]
    assert [p.shape[0] for p in parts] == [2, 2, 1] and torch.equal(torch.cat(parts), full)
    spec = fd.TensorShardSpec([5, 2], 0, [2, 2, 1])
    meta = fd.ShardMetadata(3, {"w": spec})
    assert meta.tensor_specs["w"].shard_sizes == [2, 2, 1] and meta.num_ranks == 3 and sum(spec.shard_sizes) == spec.full_shape[spec.shard_dim]
    assert issubclass(fd.Shard, fd.Placement) and issubclass(fd.Replicate, fd.Placement) and fd.Shard(1).dim == 1


def test_error_types_and_backend_contracts():
    for e in (fd.InvalidWorldSize, fd.IoError, fd.NoConnection, fd.UnsupportedOp):
        assert issubclass(e, fd.DistributedError) and issubclass(e, errors.FerrotorchError)
    a, b = fd.SimulatedBackend.create_group(2)
    assert isinstance(a, fd.Backend) and a.world_size() == 2 and b.rank() == 1
    assert isinstance(fd.is_ucc_available(), bool)
    if not fd.is_ucc_available():
        with pytest.raises(errors.FerrotorchError):
            fd.UccBackend(0, 1, "tcp://127.0.0.1:29999")
    # the device-buffer wrappers refuse a transport that has no NCCL side
    t = torch.zeros(2)
    for call in (lambda: fd.nccl_broadcast(t, a, 0), lambda: fd.nccl_all_gather(t, torch.zeros(4), a), lambda: fd.nccl_reduce_scatter(torch.zeros(4), t, a)):
        with pytest.raises(errors.InvalidArgument):
            call()

    class FakeNccl(fd.SimulatedBackend.__mro__[1]):            # a Backend whose rank disagrees with the host transport
        def __init__(self):
            pass

        def rank(self):
            return 1

        def world_size(self):
            return 2
    with pytest.raises(errors.InvalidArgument):
        fd.HybridBackend(a, FakeNccl())


def test_several_outstanding_async_collectives_run_in_issue_order():
    """Five handles outstanding at once on each rank, repeated: the ticket of each handle keeps the untagged channels from interleaving."""
    def fn(b, r):
        outs = []
        for rep in range(6):
            hs = [fd.async_allreduce(torch.full((3 + k,), float(r + 1 + k + rep)), b) for k in range(3)]
            hs.append(fd.async_all_gather(torch.tensor([float(r), float(rep)]), b))
            hs.append(fd.async_reduce_scatter(torch.arange(4.0) + rep, b))
            outs.append([h.wait() for h in reversed(hs)][::-1])             # waited in reverse: execution order is the issue order all the same
        return outs
    res = _ranks(2, fn)
    for r in range(2):
        for rep, (a0, a1, a2, ag, rs) in enumerate(res[r]):
            for k, a in enumerate((a0, a1, a2)):
                assert a.shape == (3 + k,) and torch.equal(a, torch.full((3 + k,), float(1 + k + rep) + float(2 + k + rep)))
            assert torch.equal(ag.flatten(), torch.tensor([0.0, float(rep), 1.0, float(rep)]))
            assert torch.equal(rs, 2 * (torch.arange(4.0) + rep)[2 * r: 2 * r + 2])
