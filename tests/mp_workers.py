"""Worker entry points for the multi-process tests (launched by torch.distributed.run from test_multigpu.py).

    python -m torch.distributed.run --nproc-per-node N tests/mp_workers.py <case>
"""
import os
import sys
import time
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch
import torch.distributed as dist


def _init():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    return rank, world, dev


def case_collectives():
    from ferrotorch_b200.parallel.symm import SymmComm, SymmetricBuffer
    rank, world, dev = _init()
    comm = SymmComm(dev)
    for dtype, tol in ((torch.bfloat16, 2e-2), (torch.float32, 1e-5)):
        for n in (8 * world, 1 << 12, (1 << 20) + 8 * world * 3, 3 * (1 << 22)):
            buf = SymmetricBuffer(n, dtype, dev)
            torch.manual_seed(100 + rank)
            x = (torch.rand(n, device=dev) * 2 - 1).to(dtype)
            ref = x.float().clone()
            dist.all_reduce(ref)
            for nvls in (False, True):
                buf.tensor.copy_(x)
                torch.cuda.synchronize(); dist.barrier()
                comm.all_reduce_(buf, n, scale=1.0, use_nvls=nvls)
                comm.check()
                err = (buf.tensor.float() - ref).abs().max().item()
                assert err <= tol * world, (str(dtype), n, nvls, err)
            # mean via scale, one-shot
            buf.tensor.copy_(x)
            torch.cuda.synchronize(); dist.barrier()
            out = torch.empty(n, device=dev, dtype=dtype)
            comm.all_reduce_small(buf, out, n, scale=1.0 / world)
            comm.check()
            assert (out.float() - ref / world).abs().max().item() <= tol
            # reduce-scatter / all-gather round trip
            chunk = n // world
            if chunk % 8 == 0 and chunk * world == n:
                buf.tensor.copy_(x)
                torch.cuda.synchronize(); dist.barrier()
                rs = torch.empty(chunk, device=dev, dtype=dtype)
                for nvls in (False, True):                      # peer pulls in fixed rank order / in-switch reduction
                    rs.zero_()
                    comm.reduce_scatter(buf, rs, chunk, use_nvls=nvls)
                    comm.check()
                    assert (rs.float() - ref[rank * chunk:(rank + 1) * chunk]).abs().max().item() <= tol * world, (str(dtype), n, nvls)
                comm.all_gather(buf, rs, chunk)
                comm.check()
                assert (buf.tensor.float() - ref).abs().max().item() <= tol * world
            del buf
    comm.barrier()
    comm.check()
    # bit-identical across ranks (fixed reduction order)
    n = 1 << 16
    buf = SymmetricBuffer(n, torch.float32, dev)
    torch.manual_seed(7 + rank)
    buf.tensor.copy_(torch.randn(n, device=dev))
    torch.cuda.synchronize(); dist.barrier()
    comm.all_reduce_(buf, n, scale=1.0 / world, use_nvls=False)
    comm.check()
    gathered = [torch.empty(n, device=dev) for _ in range(world)]
    dist.all_gather(gathered, buf.tensor)
    for g in gathered[1:]:
        assert torch.equal(g, gathered[0])
    if True:
        # phase stamps written from inside the kernels: four launches, four ordered records
        from ferrotorch_b200.parallel.symm import CommTrace
        with CommTrace(dev, capacity=64) as tr:
            for _ in range(3):
                comm.all_reduce_(buf, n, scale=1.0, use_nvls=False)
            comm.barrier()
        recs = tr.records()
        assert [r["kind"] for r in recs] == ["all_reduce"] * 3 + ["barrier"], recs
        assert all(0 <= r["wait_peers_us"] < 2e6 and r["total_us"] > 0 for r in recs)
        comm.all_reduce_(buf, n, scale=1.0, use_nvls=False)          # stamps off again: the ring stays as it was
        assert len(tr.records()) == 4
        comm.check()
    if rank == 0:
        print("COLLECTIVES_OK")


def case_fsdp():
    """Every sharding strategy and transport of the device engine trains the same model to the same losses and parameters; the fully sharded
    engine holds no replicated parameter copy; a checkpoint written by one configuration loads into another, also at world size 1."""
    import shutil
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.models import LlamaConfig, LlamaForCausalLM
    from ferrotorch_b200.parallel import FSDP, AdamWConfig, ShardingStrategy
    rank, world, dev = _init()
    cfg = LlamaConfig.tiny(layers=3, hidden=256, heads=2, kv_heads=1, ffn=512, vocab=512)
    opt = AdamWConfig(lr=3e-3, betas=(0.9, 0.95), weight_decay=0.01)
    torch.manual_seed(11 + rank)
    ids = torch.randint(0, cfg.vocab_size, (2, 129), device=dev)
    modes = [("nccl", ShardingStrategy.SHARD_GRAD_OP), ("fused", ShardingStrategy.SHARD_GRAD_OP), ("fused", ShardingStrategy.FULL_SHARD),
             ("nccl", ShardingStrategy.FULL_SHARD)]
    results, engines = {}, {}
    for comm, strat in modes:
        key = f"{comm}/{strat.value}"
        model = LlamaForCausalLM(cfg, device=dev, world=world, rank=rank, seed=0)
        eng = FSDP(model, opt, comm=comm, strategy=strat)
        assert eng.comm == comm, (key, eng.comm)
        losses = [eng.train_step(ids[:, :-1], ids[:, 1:]).item() for _ in range(6)]
        eng.synchronize()
        torch.cuda.synchronize()
        assert _lib.read_status() == 0, key
        params = eng.full_parameters()
        torch.cuda.synchronize()
        assert _lib.read_status() == 0, key
        w = torch.cat([params[u.name][: u.numel].float() for u in eng.units])
        results[key] = (losses, w)
        engines[key] = (model, eng)
        ws = [torch.empty_like(w) for _ in range(world)]
        dist.all_gather(ws, w)
        for o in ws[1:]:
            assert torch.equal(o, ws[0]), key                      # parameters identical on every rank after the updates
        assert losses[-1] < losses[0], (key, losses)
        if strat == ShardingStrategy.FULL_SHARD:
            assert all(u.full is None for u in eng.units), key      # no replicated copy is kept
            if comm == "fused":
                # units that stay resident between forward and backward are not gathered twice
                assert eng.sharded.gathers < 6 * 2 * len(eng.units), (eng.sharded.gathers, len(eng.units))
    base_l, base_w = results["nccl/shard_grad_op"]
    for key, (l, w) in results.items():
        assert all(abs(a - b) < 5e-2 for a, b in zip(base_l, l)), (key, base_l, l)
        rel = (base_w - w).norm() / base_w.norm()
        assert rel.item() < 2e-2, (key, rel.item())
    # ---- checkpoints: written by the fully sharded engine, read by a shard-grad-op engine at the same world size and by a single-rank engine ----
    ck = Path(f"/tmp/ft_fsdp_ck_{os.environ.get('MASTER_PORT', '0')}")
    if rank == 0:
        shutil.rmtree(ck, ignore_errors=True)
    dist.barrier()
    src_model, src = engines["fused/full_shard"]
    src.save(ck / "a")
    m2 = LlamaForCausalLM(cfg, device=dev, world=world, rank=rank, seed=123)           # different initial values
    e2 = FSDP(m2, opt, comm="fused", strategy=ShardingStrategy.SHARD_GRAD_OP)
    e2.load(ck / "a")
    la = [src.train_step(ids[:, :-1], ids[:, 1:]).item() for _ in range(2)]
    lb = [e2.train_step(ids[:, :-1], ids[:, 1:]).item() for _ in range(2)]
    assert all(abs(a - b) < 2e-2 for a, b in zip(la, lb)), (la, lb)                    # training resumes on the restored state
    # single-rank engine reads the multi-rank files (every rank does so on its own GPU)
    src.save(ck / "b")
    m1 = LlamaForCausalLM(cfg, device=dev, world=1, rank=0, seed=5)
    e1 = FSDP(m1, opt, local=True)
    e1.load(ck / "b")
    for u_src, u1 in zip(src.units, e1.units):
        parts = [torch.empty_like(u_src.master) for _ in range(world)]
        dist.all_gather(parts, u_src.master)
        whole = torch.cat(parts)[: u1.numel]
        assert torch.equal(whole, u1.master[: u1.numel]), u1.name
        assert u1.step == u_src.step
    full_src = src.full_parameters()
    for u1 in e1.units:
        assert torch.equal(full_src[u1.name][: u1.numel], u1.full[: u1.numel]), u1.name
    # and back: a single-rank checkpoint (written by rank 0) loads into the sharded engine
    if rank == 0:
        e1.save(ck / "c")
    dist.barrier()
    m3 = LlamaForCausalLM(cfg, device=dev, world=world, rank=rank, seed=77)
    e3 = FSDP(m3, opt, comm="fused", strategy=ShardingStrategy.FULL_SHARD)
    e3.load(ck / "c")
    full3 = e3.full_parameters()
    for u1 in e1.units:
        assert torch.equal(full3[u1.name][: u1.numel], u1.full[: u1.numel]), u1.name
    torch.cuda.synchronize()
    assert _lib.read_status() == 0
    dist.barrier()
    if rank == 0:
        shutil.rmtree(ck, ignore_errors=True)
        print("FSDP_OK", base_l, results["fused/full_shard"][0])


def case_timeout():
    """A peer that does not show up: the waiting rank's kernel gives up after its deadline and reports it."""
    from ferrotorch_b200.parallel.symm import SymmComm
    from ferrotorch_b200.errors import Timeout
    rank, world, dev = _init()
    comm = SymmComm(dev)
    comm.barrier()
    comm.check()
    if rank == 0:
        comm.barrier()                 # nobody else joins this one
        try:
            comm.check()
            raise AssertionError("expected a timeout")
        except Timeout:
            pass
    else:
        comm.seq += 1                  # stay in step with rank 0's sequence numbers without launching anything
        time.sleep(3.0)
    torch.cuda.synchronize()
    dist.barrier()
    # the context is still usable and the fabric still works after the timeout
    comm.barrier()
    comm.check()
    # the same with a many-CTA collective: every CTA of rank 0's all-reduce runs out of time at its opening rendezvous; the CTA counter and the
    # sequence numbers must come out of it consistent, so that the next all-reduce (all ranks present) elects its last CTA and succeeds
    from ferrotorch_b200.parallel.symm import SymmetricBuffer
    n = 1 << 22
    buf = SymmetricBuffer(n, torch.float32, dev)
    buf.tensor.fill_(float(rank + 1))
    torch.cuda.synchronize(); dist.barrier()
    SymmComm.set_timeout(0.5)
    if rank == 0:
        comm.all_reduce_(buf, n, use_nvls=False)
        try:
            comm.check()
            raise AssertionError("expected a timeout")
        except Timeout:
            pass
        assert float(buf.tensor[0]) == 1.0 and float(buf.tensor[-1]) == 1.0       # nothing was reduced
    else:
        comm.seq += 1
        time.sleep(1.5)
    torch.cuda.synchronize()
    dist.barrier()
    SymmComm.set_timeout(2.0)
    comm.all_reduce_(buf, n, use_nvls=False)
    comm.check()
    want = float(sum(range(1, world + 1)))
    assert float(buf.tensor[0]) == want and float(buf.tensor[n // 2 + 3]) == want and float(buf.tensor[-1]) == want
    x = torch.ones(4, device=dev)
    dist.all_reduce(x)
    assert x[0].item() == world
    if rank == 0:
        print("TIMEOUT_OK")


def case_tp_decode():
    """Tensor-parallel engine (prefill + graph-replayed decode) against the dense f32 reference, identical tokens on every rank."""
    from ferrotorch_b200.models import LlamaConfig
    from ferrotorch_b200.models.llama_infer import LlamaTPEngine, TPContext, random_hf_weights, reference_last_logits
    rank, world, dev = _init()
    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256)
    W = random_hf_weights(cfg, dev, seed=1, std=0.05)
    eng = LlamaTPEngine(cfg, TPContext(dev), max_batch=4, max_seq=128, device=dev, weights=W, use_graph=True)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (4, 40), device=dev)
    seq = ids.clone()
    tok = eng.prefill(ids)
    for step in range(6):
        ref = reference_last_logits(cfg, W, seq)
        mine = ref[:, rank * eng.V:(rank + 1) * eng.V]
        err = (eng.logits - mine).abs().max().item()
        assert err < 0.06 * ref.abs().max().item() + 0.02, (step, err)
        toks = [torch.empty_like(tok) for _ in range(world)]
        dist.all_gather(toks, tok.contiguous())
        for t in toks[1:]:
            assert torch.equal(t, toks[0])
        seq = torch.cat([seq, tok[:, None]], 1)
        tok = eng.decode_step().clone()
    eng.check()
    if rank == 0:
        print("TP_DECODE_OK")


def case_ddp():
    """Fused bucket all-reduce DDP: gradients equal the NCCL-averaged ones and are bit-identical across ranks; SyncBatchNorm matches torch's."""
    from ferrotorch_b200.parallel import DDP, SyncBatchNorm2d
    rank, world, dev = _init()
    torch.manual_seed(0)

    def make():
        torch.manual_seed(0)
        return torch.nn.Sequential(torch.nn.Conv2d(3, 8, 3, padding=1), torch.nn.BatchNorm2d(8), torch.nn.ReLU(), torch.nn.Flatten(),
                                   torch.nn.Linear(8 * 8 * 8, 32), torch.nn.ReLU(), torch.nn.Linear(32, 10)).to(dev)
    torch.manual_seed(100 + rank)
    x, y = torch.randn(16, 3, 8, 8, device=dev), torch.randint(0, 10, (16,), device=dev)
    grads = {}
    for mode in ("nccl", "fused"):
        m = make()
        ddp = DDP(m, bucket_cap_bytes=8192, comm=mode)
        assert len(ddp.buckets) > 1
        for _ in range(2):
            ddp.zero_grad()
            torch.nn.functional.cross_entropy(ddp(x), y).backward()
        torch.cuda.synchronize()
        grads[mode] = [p.grad.clone() for p in m.parameters()]
        for g in grads[mode]:
            gs = [torch.empty_like(g) for _ in range(world)]
            dist.all_gather(gs, g.contiguous())
            for o in gs[1:]:
                assert torch.equal(o, gs[0]), mode
    for a, b in zip(grads["nccl"], grads["fused"]):
        assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
    # reference: plain model, gradients averaged by hand
    m = make()
    torch.nn.functional.cross_entropy(m(x), y).backward()
    for p, g in zip(m.parameters(), grads["fused"]):
        r = p.grad.clone()
        dist.all_reduce(r)
        assert torch.allclose(r / world, g, rtol=1e-4, atol=1e-6)
    # SyncBatchNorm
    torch.manual_seed(5)
    ours, theirs = SyncBatchNorm2d(8).to(dev), torch.nn.SyncBatchNorm(8).to(dev)
    xa = x.clone().requires_grad_(True)
    xb = x.clone().requires_grad_(True)
    conv = torch.nn.Conv2d(3, 8, 1).to(dev)
    oa, ob = ours(conv(xa)), theirs(conv(xb))
    assert torch.allclose(oa, ob, atol=1e-4)
    oa.square().sum().backward()
    ob.square().sum().backward()
    assert torch.allclose(xa.grad, xb.grad, atol=1e-3)
    assert torch.allclose(ours.running_var, theirs.running_var, atol=1e-4)
    # channels-last activations: fused statistics kernels, sums reduced by the one-shot peer-memory kernel; several layers in a row
    # (staging slots rotate) and three steps
    torch.manual_seed(6)
    fused = [SyncBatchNorm2d(16).to(dev) for _ in range(3)]
    ref = [torch.nn.SyncBatchNorm(16).to(dev) for _ in range(3)]
    for step in range(3):
        xs = (torch.randn(4, 16, 6, 5, device=dev) * (rank + 1) + rank).contiguous(memory_format=torch.channels_last)
        xa, xb = xs.clone().requires_grad_(True), xs.clone().requires_grad_(True)
        ha, hb = xa, xb
        for fa, fb in zip(fused, ref):
            ha, hb = fa(ha) * 1.5, fb(hb) * 1.5
        assert torch.allclose(ha, hb, atol=1e-4), (ha - hb).abs().max().item()
        ha.square().sum().backward()
        hb.square().sum().backward()
        assert torch.allclose(xa.grad, xb.grad, atol=2e-3, rtol=1e-3), (xa.grad - xb.grad).abs().max().item()
        for fa, fb in zip(fused, ref):
            assert torch.allclose(fa.weight.grad, fb.weight.grad, atol=2e-3, rtol=1e-3)
            assert torch.allclose(fa.running_mean, fb.running_mean, atol=1e-4) and torch.allclose(fa.running_var, fb.running_var, atol=1e-3)
            fa.weight.grad = fb.weight.grad = None
    from ferrotorch_b200 import _lib
    assert _lib.read_status() == 0
    if rank == 0:
        print("DDP_OK")


def case_tp_gemm():
    """Fused all-gather->GEMM and GEMM->reduce-scatter against the unfused library path, several launches in a row (flag / parity reuse)."""
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.parallel import ColumnParallelLinear, RowParallelLinear, ParallelEmbedding
    rank, world, dev = _init()
    M, D, Fdim = 128 * world * 3, 512, 1024 + 256
    torch.manual_seed(0)
    w1, w2 = (torch.randn(Fdim, D, device=dev) * 0.05).bfloat16(), (torch.randn(D, Fdim, device=dev) * 0.05).bfloat16()
    col_f, col_n = ColumnParallelLinear(D, Fdim, device=dev, comm="fused"), ColumnParallelLinear(D, Fdim, device=dev, comm="nccl")
    row_f, row_n = RowParallelLinear(Fdim, D, device=dev, comm="fused"), RowParallelLinear(Fdim, D, device=dev, comm="nccl")
    for m in (col_f, col_n):
        m.load_full_weight(w1)
    for m in (row_f, row_n):
        m.load_full_weight(w2)
    with torch.no_grad():
        for it in range(5):
            torch.manual_seed(10 + it)
            x_full = torch.randn(M, D, device=dev).bfloat16()               # same on every rank
            xs = x_full[rank * (M // world): (rank + 1) * (M // world)].contiguous()
            h_f, h_n = col_f(xs), col_n(xs)
            ref_h = (x_full.float() @ w1.float().t())[:, rank * (Fdim // world): (rank + 1) * (Fdim // world)]
            assert h_f.shape == (M, Fdim // world)
            assert (h_f.float() - ref_h).abs().max() < 0.05 and (h_f.float() - h_n.float()).abs().max() < 0.02, it
            y_f, y_n = row_f(h_n), row_n(h_n)
            hf_all = [torch.empty_like(h_n) for _ in range(world)]
            dist.all_gather(hf_all, h_n)
            ref_y = (torch.cat(hf_all, 1).float() @ w2.float().t())[rank * (M // world): (rank + 1) * (M // world)]
            assert y_f.shape == (M // world, D)
            tol = 2.0 * 2.0 ** -8 * float(ref_y.abs().max())          # two bf16 steps at the largest magnitude (the partial products are rounded to bf16)
            assert (y_f.float() - ref_y).abs().max() < tol, (it, float((y_f.float() - ref_y).abs().max()), tol)
            assert (y_f.float() - y_n.float()).abs().max() < tol, (it, float((y_f.float() - y_n.float()).abs().max()), tol)
    emb = ParallelEmbedding(64 * world, 32, device=dev)
    full = torch.arange(64 * world * 32, device=dev, dtype=torch.float32).view(64 * world, 32).bfloat16()
    emb.load_full_weight(full)
    ids = torch.randint(0, 64 * world, (4, 9), device=dev, generator=torch.Generator(device=dev).manual_seed(1))
    assert torch.equal(emb(ids), full[ids])
    assert _lib.read_status() == 0
    dist.barrier()
    if rank == 0:
        print("TP_GEMM_OK")


def case_cp():
    """Peer-memory all-to-all / broadcast kernels, Ulysses attention over them and ring attention pulling K/V blocks from peers."""
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.parallel import UlyssesAttention, ring_attention
    from ferrotorch_b200.parallel.symm import SymmComm, SymmetricBuffer
    rank, world, dev = _init()
    comm = SymmComm(dev)
    for dtype in (torch.bfloat16, torch.float32):
        chunk = 4096 + 64
        buf = SymmetricBuffer(world * chunk, dtype, dev)
        buf.tensor.copy_((torch.arange(world * chunk, device=dev) % 251 + rank * 1000).to(dtype))
        out = torch.empty(world * chunk, device=dev, dtype=dtype)
        comm.all_to_all(buf, out, chunk)
        for q in range(world):
            exp = (torch.arange(rank * chunk, (rank + 1) * chunk, device=dev) % 251 + q * 1000).to(dtype)
            assert torch.equal(out[q * chunk:(q + 1) * chunk], exp), (dtype, q)
        b = torch.empty(chunk, device=dev, dtype=dtype)
        comm.broadcast(buf, b, chunk, root=world - 1)
        assert torch.equal(b, (torch.arange(chunk, device=dev) % 251 + (world - 1) * 1000).to(dtype))
    torch.manual_seed(0)
    S, Hq, Hkv, D = 256 * world, 8, 2 * world, 128
    Q, K, V = (torch.randn(S, h, D, device=dev).bfloat16() for h in (Hq, Hkv, Hkv))
    sl = slice(rank * (S // world), (rank + 1) * (S // world))
    rep = Hq // Hkv
    for causal in (True, False):
        ref = torch.nn.functional.scaled_dot_product_attention(Q.float().transpose(0, 1)[None], K.float().repeat_interleave(rep, 1).transpose(0, 1)[None],
                                                               V.float().repeat_interleave(rep, 1).transpose(0, 1)[None], is_causal=causal)[0].transpose(0, 1)[sl]
        with torch.no_grad():
            u = UlyssesAttention(causal=causal)(Q[sl].contiguous(), K[sl].contiguous(), V[sl].contiguous())
        assert (u.float() - ref).abs().max() < 3e-2, ("ulysses", causal, float((u.float() - ref).abs().max()))
        kvbuf = SymmetricBuffer(2 * K[sl].numel(), torch.bfloat16, dev)
        r = ring_attention(Q[sl].contiguous(), K[sl].contiguous(), V[sl].contiguous(), causal=causal, fabric=(comm, kvbuf))
        assert (r.float() - ref).abs().max() < 3e-2, ("ring", causal, float((r.float() - ref).abs().max()))
    assert _lib.read_status() == 0
    dist.barrier()
    if rank == 0:
        print("CP_OK")


def case_pipeline():
    """Device point-to-point channel (more messages than slots, so slots are re-used behind acknowledgements) and a two-stage GPipe step whose
    parameter gradients equal the single-process ones (the upstream stage receives the real input gradient)."""
    from ferrotorch_b200 import _lib
    from ferrotorch_b200.parallel import GpuPipelineStage, P2PChannel
    rank, world, dev = _init()
    ch = P2PChannel(4096, slots=2, device=dev)
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    for i in range(7):
        msg = torch.full((1024,), float(rank * 100 + i), device=dev)
        ch.send(msg, nxt)
        got = ch.recv(torch.empty(1024, device=dev), prv)
        assert float(got[0]) == prv * 100 + i and float(got[-1]) == prv * 100 + i, (i, float(got[0]))
    torch.manual_seed(0)
    full = torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.Tanh(), torch.nn.Linear(64, 48), torch.nn.Tanh(), torch.nn.Linear(48, 8)).to(dev)
    cut = 2 if world == 2 else None
    assert world == 2
    stage_mod = torch.nn.Sequential(*list(full.children())[:cut]) if rank == 0 else torch.nn.Sequential(*list(full.children())[cut:])
    import copy
    stage_mod = copy.deepcopy(stage_mod)
    stage = GpuPipelineStage(stage_mod, (32,) if rank == 0 else (64,), (64,) if rank == 0 else (8,), micro_batch=4)
    g = torch.Generator(device=dev).manual_seed(1)
    X = torch.randn(3, 4, 32, device=dev, generator=g)
    T = torch.randn(3, 4, 8, device=dev, generator=g)
    losses = stage.forward_backward([X[i] for i in range(3)] if rank == 0 else None, 3, (lambda o, i: ((o - T[i]) ** 2).mean()) if rank == 1 else None)
    torch.cuda.synchronize()
    for i in range(3):
        ((full(X[i]) - T[i]) ** 2).mean().backward()
    ref = list(full.children())[:cut] if rank == 0 else list(full.children())[cut:]
    for a, b in zip(stage_mod.parameters(), torch.nn.Sequential(*ref).parameters()):
        assert torch.allclose(a.grad, b.grad, atol=1e-5), float((a.grad - b.grad).abs().max())
    if rank == 1:
        assert len(losses) == 3
    assert _lib.read_status() == 0
    dist.barrier()
    if rank == 0:
        print("PIPELINE_OK")


if __name__ == "__main__":
    try:
        {"collectives": case_collectives, "fsdp": case_fsdp, "timeout": case_timeout, "tp_decode": case_tp_decode, "ddp": case_ddp, "tp_gemm": case_tp_gemm, "cp": case_cp, "pipeline": case_pipeline}[sys.argv[1]]()
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()
