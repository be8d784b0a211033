"""Decode path: split-K GEMM, paged attention, fused epilogues and the TP engine against dense f32 PyTorch evaluations."""
import math

import pytest
import torch

from ferrotorch_b200 import _lib, ops
from ferrotorch_b200.models import LlamaConfig
from ferrotorch_b200.models.llama_infer import LlamaTPEngine, random_hf_weights, reference_last_logits

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("N,K,splits", [(1280, 1024, 8), (520, 8192, 16), (256, 200, 3)])
def test_splitk_gemm_planes_sum_to_product(N, K, splits):
    torch.manual_seed(N + K)
    x = torch.zeros(16, K, device="cuda", dtype=torch.bfloat16)
    x[:5] = torch.randn(5, K, device="cuda").to(torch.bfloat16)
    w = torch.randn(N, K, device="cuda").to(torch.bfloat16)
    planes = torch.full((splits, 16, N), float("nan"), device="cuda", dtype=torch.float32)
    _lib.call("ft_gemm_bf16_splitk", x, w, planes, 16, N, K, K, K, N, 0, 0, splits, _lib.S())
    ref = x.float() @ w.float().t()
    got = planes.sum(0)
    assert torch.isfinite(got).all()
    assert (got - ref).abs().max().item() <= 2e-3 * ref.abs().max().item() + 1e-3
    out = torch.empty(5, N, device="cuda", dtype=torch.bfloat16)
    _lib.call("ft_splitk_reduce", planes, splits, 5, N, N, 16 * N, None, out, N, 0, _lib.S())
    assert (out.float() - ref[:5]).abs().max().item() <= 2e-2 * ref.abs().max().item()


@pytest.mark.parametrize("Hq,Hkv,nsplit", [(8, 1, 4), (4, 2, 4), (2, 2, 4), (8, 1, 1), (8, 1, 13), (8, 1, 16), (8, 1, 37), (4, 2, 64)])
def test_paged_attention_decode(Hq, Hkv, nsplit):
    """Split counts on both sides of the combining pass's batch of sixteen, and more splits than a short sequence has pages (empty splits)."""
    torch.manual_seed(Hq * 10 + Hkv)
    B, D, max_blocks = 3, 128, 12
    lens = torch.tensor([1, 37, 160], device="cuda", dtype=torch.int32)
    nblk = B * max_blocks
    kc = torch.randn(nblk, 16, Hkv, D, device="cuda").to(torch.bfloat16)
    vc = torch.randn(nblk, 16, Hkv, D, device="cuda").to(torch.bfloat16)
    perm = torch.randperm(nblk, device="cuda").to(torch.int32).view(B, max_blocks).contiguous()     # scattered pages
    q = torch.randn(B, Hq, D, device="cuda").to(torch.bfloat16)
    out = torch.empty_like(q)
    ws = torch.zeros(B * Hkv * nsplit * (Hq // Hkv) * 132, device="cuda")
    ctr = torch.zeros(B * Hkv, device="cuda", dtype=torch.int32)
    for _ in range(2):      # second call checks that the counters reset themselves
        _lib.call("ft_paged_attn_decode", q, kc, vc, perm, max_blocks, lens, B, Hq, Hkv, D, 1.0 / math.sqrt(D), nsplit, ws, ctr, out, _lib.S())
    for b in range(B):
        n = int(lens[b])
        k = kc[perm[b].long()].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, 1)
        v = vc[perm[b].long()].reshape(-1, Hkv, D)[:n].float().repeat_interleave(Hq // Hkv, 1)
        s = torch.einsum("hd,thd->ht", q[b].float(), k) / math.sqrt(D)
        ref = torch.einsum("ht,thd->hd", torch.softmax(s, -1), v)
        assert (out[b].float() - ref).abs().max().item() < 2e-2
    assert int(ctr.sum()) == 0


@pytest.mark.parametrize("use_graph", [False, True])
def test_tp_engine_single_gpu_matches_dense_reference(use_graph):
    cfg = LlamaConfig(vocab_size=1024, hidden_size=512, intermediate_size=1024, num_hidden_layers=2, num_attention_heads=4,
                      num_key_value_heads=2, max_position_embeddings=256)
    W = random_hf_weights(cfg, "cuda", seed=1, std=0.05)
    eng = LlamaTPEngine(cfg, max_batch=4, max_seq=128, device="cuda", weights=W, use_graph=use_graph)
    torch.manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (4, 40), device="cuda")
    seq = ids.clone()
    tok = eng.prefill(ids)
    ref = reference_last_logits(cfg, W, seq)
    assert (eng.logits - ref).abs().max().item() < 0.06 * ref.abs().max().item() + 0.02
    for _ in range(5):
        seq = torch.cat([seq, tok[:, None]], 1)
        tok = eng.decode_step().clone()
        ref = reference_last_logits(cfg, W, seq)
        assert (eng.logits - ref).abs().max().item() < 0.06 * ref.abs().max().item() + 0.02
    eng.check()
