"""CPU checks of the model families against Hugging Face implementations / dense formulas, and of the generation utilities."""
import math

import pytest
import torch

from ferrotorch_b200.models import LlamaConfig, bert, diffusion, graph, rl, whisper
from ferrotorch_b200.models import llama_gen as G
from ferrotorch_b200.models.llama_infer import random_hf_weights, reference_generate

transformers = pytest.importorskip("transformers")


def _tiny_llama(seed=3):
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      max_position_embeddings=128)
    W = {k: v.float() for k, v in random_hf_weights(cfg, "cpu", seed, 0.2).items()}
    return cfg, G.CachedLlama(cfg, W), W


def test_cached_generation_matches_dense_reference():
    cfg, m, W = _tiny_llama()
    ids = torch.randint(0, 128, (2, 10), generator=torch.Generator().manual_seed(0))
    out = G.generate(m, m.new_cache, ids, G.GenerationConfig(max_new_tokens=8))
    assert torch.equal(out[:, 10:], reference_generate(cfg, W, ids, 8))


def test_sampling_filters_and_seed():
    logits = torch.tensor([[1.0, 2.0, 3.0, 4.0]])
    assert torch.isinf(G.top_k_filter(logits, 2)[0, :2]).all() and torch.isfinite(G.top_k_filter(logits, 2)[0, 2:]).all()
    f = G.top_p_filter(logits, 0.5)                       # p(4)=0.64 >= 0.5: only the top token survives
    assert torch.isfinite(f[0, 3]) and torch.isinf(f[0, :3]).all()
    pen = G.apply_repetition_penalty(torch.tensor([[2.0, -2.0, 1.0]]), torch.tensor([[0, 1]]), 2.0)
    assert pen.tolist() == [[1.0, -4.0, 1.0]]
    cfg, m, _ = _tiny_llama()
    ids = torch.randint(0, 128, (1, 6), generator=torch.Generator().manual_seed(1))
    c = G.GenerationConfig(max_new_tokens=6, seed=7).with_top_k(20).with_top_p(0.95).with_temperature(0.9)
    a, b = G.generate(m, m.new_cache, ids, c), G.generate(m, m.new_cache, ids, c)
    assert torch.equal(a, b) and a.shape == (1, 12)


def test_streamer_eos_and_beam():
    cfg, m, _ = _tiny_llama()
    ids = torch.randint(0, 128, (1, 6), generator=torch.Generator().manual_seed(2))
    greedy = G.generate(m, m.new_cache, ids, G.GenerationConfig(max_new_tokens=5))
    seen = []
    eos = int(greedy[0, 8])
    out = G.generate(m, m.new_cache, ids, G.GenerationConfig(max_new_tokens=5, eos_token_id=eos), streamer=lambda t: seen.append(int(t)))
    assert out.shape[1] <= 9 and int(out[0, -1]) == eos and seen == out[0, 6:].tolist()
    beam = G.generate(m, m.new_cache, ids, G.GenerationConfig(max_new_tokens=5, num_beams=3))
    # the best beam scores at least as well as greedy under the model
    def score(seq):
        lp = m(seq[:, :-1], m.new_cache()).log_softmax(-1)
        return float(lp[0, 5:].gather(1, seq[0, 6:, None]).sum())
    assert beam.shape == greedy.shape and score(beam) >= score(greedy) - 1e-4


def test_speculative_decoding_equals_greedy():
    cfg, m, _ = _tiny_llama(3)
    _, d, _ = _tiny_llama(4)
    ids = torch.randint(0, 128, (1, 8), generator=torch.Generator().manual_seed(5))
    greedy = G.generate(m, m.new_cache, ids, G.GenerationConfig(max_new_tokens=12))
    sp, st = G.speculative_generate(m, m.new_cache, d, d.new_cache, ids, G.SpecDecodeConfig(3, 12))
    assert torch.equal(sp, greedy)
    sp2, st2 = G.speculative_generate(m, m.new_cache, m, m.new_cache, ids, G.SpecDecodeConfig(4, 12))
    assert torch.equal(sp2, greedy) and st2.acceptance_rate() == 1.0


def test_quant_loaders_and_gguf_names():
    gen = torch.Generator().manual_seed(0)
    w = torch.randint(0, 16, (64, 16), generator=gen)
    z = torch.randint(1, 16, (1, 16), generator=gen)
    sc = torch.rand(1, 16, generator=gen)
    qw = torch.zeros(8, 16, dtype=torch.int32)
    for r in range(64):
        qw[r // 8] |= w[r].to(torch.int32) << (4 * (r % 8))
    qz = torch.zeros(1, 2, dtype=torch.int32)
    for c in range(16):
        qz[0, c // 8] |= (z[0, c] - 1).to(torch.int32) << (4 * (c % 8))
    assert torch.allclose(G.dequantize_gptq_q4(qw, qz, sc, group_size=64), ((w.float() - z.float()) * sc).t())
    # AWQ: [in, out/8] with the interleaved nibble order
    wa = torch.randint(0, 16, (32, 8), generator=gen)
    za = torch.randint(0, 16, (1, 8), generator=gen)
    sa = torch.rand(1, 8, generator=gen)
    order = [0, 2, 4, 6, 1, 3, 5, 7]                 # AutoAWQ's packing order: nibble i of a word holds channel order[i]
    qwa, qza = torch.zeros(32, 1, dtype=torch.int32), torch.zeros(1, 1, dtype=torch.int32)
    for i, o in enumerate(order):
        qwa[:, 0] |= wa[:, o].to(torch.int32) << (4 * i)
        qza[:, 0] |= za[:, o].to(torch.int32) << (4 * i)
    assert torch.allclose(G.dequantize_awq_q4(qwa, qza, sa, group_size=32), ((wa.float() - za.float()) * sa).t())
    q = torch.randint(0, 16, (8, 4), generator=gen).to(torch.uint8)
    packed = (q[:4] << 4) | q[4:]
    assert torch.allclose(G.dequantize_hqq(packed, torch.tensor(0.5), torch.tensor(8.0), (8, 4)), (q.float() - 8) * 0.5)
    assert G.gguf_to_hf_name("blk.3.ffn_gate.weight") == "model.layers.3.mlp.gate_proj.weight"
    assert G.gguf_to_hf_name("output_norm.weight") == "model.norm.weight" and G.gguf_to_hf_name("rope_freqs.weight") is None
    w = torch.arange(8 * 3, dtype=torch.float32).view(8, 3)
    un = G.gguf_unpermute_qk(w, 2)
    assert un.shape == w.shape and torch.equal(un[0], w[0]) and torch.equal(un[1], w[2]) and torch.equal(un[2], w[1])


def test_bert_matches_hf():
    c = bert.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, max_position_embeddings=32)
    hc = transformers.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, max_position_embeddings=32)
    hm, m = transformers.BertModel(hc).eval(), bert.BertModel(c).eval()
    m.load_state_dict(hm.state_dict(), strict=False)
    ids = torch.randint(0, 100, (2, 10))
    mask = torch.ones(2, 10, dtype=torch.long)
    mask[1, 6:] = 0
    with torch.no_grad():
        o, (h, p) = hm(input_ids=ids, attention_mask=mask), m(ids, mask)
        assert (o.last_hidden_state - h)[mask.bool()].abs().max() < 1e-5 and (o.pooler_output - p).abs().max() < 1e-5
        e = bert.SentenceTransformer(m)(ids, mask)
    assert torch.allclose(e.norm(dim=-1), torch.ones(2), atol=1e-5)


def test_whisper_encoder_and_mel_match_hf():
    wc = whisper.WhisperConfig(d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128)
    hwc = transformers.WhisperConfig(num_mel_bins=80, d_model=64, encoder_layers=2, encoder_attention_heads=4, encoder_ffn_dim=128, max_source_positions=1500,
                                     decoder_layers=1, decoder_attention_heads=4, decoder_ffn_dim=128, vocab_size=100, pad_token_id=0, bos_token_id=1,
                                     eos_token_id=2, decoder_start_token_id=1)
    hwe, we = transformers.WhisperModel(hwc).encoder.eval(), whisper.WhisperEncoder(wc).eval()
    we.load_state_dict(hwe.state_dict(), strict=False)
    audio = torch.randn(16000, generator=torch.Generator().manual_seed(0))
    mel = whisper.log_mel_spectrogram(audio)
    ref = torch.tensor(transformers.WhisperFeatureExtractor()(audio.numpy(), sampling_rate=16000, return_tensors="np").input_features)
    assert mel.shape == (1, 80, 3000) and (mel - ref).abs().max() < 1e-4
    with torch.no_grad():
        assert (hwe(mel).last_hidden_state - we(mel)).abs().max() < 1e-4


def test_diffusion_shapes_param_counts_and_clip_parity():
    assert sum(p.numel() for p in diffusion.UNet2DConditionModel().parameters()) == 859_520_964      # SD-1.5 UNet
    assert sum(p.numel() for p in diffusion.AutoencoderKL().parameters()) == 83_653_863              # SD-1.5 VAE
    hc = transformers.CLIPTextConfig(vocab_size=1000, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, max_position_embeddings=77)
    hm, mine = transformers.CLIPTextModel(hc).eval(), diffusion.ClipTextEncoder(diffusion.ClipTextConfig.tiny()).eval()
    mine.load_state_dict(hm.state_dict(), strict=False)
    ids = torch.randint(0, 1000, (2, 77))
    with torch.no_grad():
        assert (hm(ids).last_hidden_state - mine(ids)).abs().max() < 1e-5
    u, v = diffusion.UNet2DConditionModel(diffusion.UNetConfig.tiny()).eval(), diffusion.AutoencoderKL(diffusion.VaeConfig.tiny()).eval()
    img = diffusion.StableDiffusionPipeline(mine, u, v)(ids[:1], height=64, width=64, num_inference_steps=3)
    assert img.shape == (1, 3, 16, 16) and 0 <= float(img.min()) and float(img.max()) <= 1
    s = diffusion.DDIMScheduler()
    s.set_timesteps(50)
    assert s.timesteps[0] == 981 and s.timesteps[-1] == 1 and abs(float(s.alphas_cumprod[0]) - 0.99915) < 1e-5


def test_gcn_matches_dense_and_policy_shapes():
    g = graph.Graph(torch.tensor([[0, 1, 2, 3], [1, 2, 3, 0]]), 4)
    net = graph.GcnNet(8, 4, 3).eval()
    A = torch.zeros(4, 4)
    A[g.edge_index[1], g.edge_index[0]] = 1
    A += torch.eye(4)
    d = A.sum(1).pow(-0.5)
    An = d[:, None] * A * d[None]
    x = torch.randn(4, 8)
    assert (net.conv1(x, g) - (An @ net.conv1.lin(x) + net.conv1.bias)).abs().max() < 1e-5
    with pytest.raises(Exception):
        graph.Graph(torch.tensor([[0], [9]]), 4)
    pol = rl.MlpPolicy(rl.MlpPolicyConfig())
    a, v, lp = pol(torch.randn(5, 4))
    assert a.shape == v.shape == lp.shape == (5,) and "mlp_extractor.policy_net.0.weight" in pol.state_dict()
    pol2 = rl.MlpPolicy(rl.MlpPolicyConfig(discrete=False, action_dim=3))
    a, v, lp = pol2(torch.randn(5, 4))
    assert a.shape == (5, 3) and lp.shape == (5,)
    loss = rl.ppo_loss(pol, torch.randn(5, 4), torch.randint(0, 2, (5,)), torch.zeros(5), torch.randn(5), torch.randn(5))
    loss.backward()
    assert all(p.grad is not None for n, p in pol.named_parameters())


def test_llama_training_model_matches_hf_transformers_through_hf_state_dict():
    """The training model (flat per-layer units) against transformers' LlamaForCausalLM: weights go across under the HF key names in both
    directions and the losses agree (half-rotation RoPE, GQA, pre-norm residual blocks, untied head)."""
    import torch
    from transformers import LlamaConfig as HFConfig, LlamaForCausalLM as HFModel
    from ferrotorch_b200.models import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig.tiny(layers=2, hidden=256, heads=2, kv_heads=1, ffn=512, vocab=1024)
    ours = LlamaForCausalLM(cfg, device="cpu", seed=0)
    hf_cfg = HFConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size,
                      num_hidden_layers=cfg.num_hidden_layers, num_attention_heads=cfg.num_attention_heads, num_key_value_heads=cfg.num_key_value_heads,
                      rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, max_position_embeddings=cfg.max_position_embeddings,
                      tie_word_embeddings=False, attention_bias=False, mlp_bias=False)
    hf = HFModel(hf_cfg).to(torch.bfloat16)
    missing, unexpected = hf.load_state_dict(ours.hf_state_dict(), strict=False)
    assert not missing and not unexpected
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, cfg.vocab_size, (2, 33), generator=g)
    with torch.no_grad():
        loss = float(ours(ids[:, :-1], labels=ids[:, 1:]))
        ref = float(torch.nn.functional.cross_entropy(hf(input_ids=ids[:, :-1]).logits.float().reshape(-1, cfg.vocab_size), ids[:, 1:].reshape(-1)))
    assert abs(loss - ref) < 5e-3 * ref, (loss, ref)
    # and back: a freshly initialised HF model loaded into a second instance of ours
    hf2 = HFModel(hf_cfg).to(torch.bfloat16)
    other = LlamaForCausalLM(cfg, device="cpu", seed=1)
    other.load_hf_state_dict(hf2.state_dict())
    with torch.no_grad():
        loss2 = float(other(ids[:, :-1], labels=ids[:, 1:]))
        ref2 = float(torch.nn.functional.cross_entropy(hf2(input_ids=ids[:, :-1]).logits.float().reshape(-1, cfg.vocab_size), ids[:, 1:].reshape(-1)))
    assert abs(loss2 - ref2) < 5e-3 * ref2, (loss2, ref2)


def test_rope_scaling_types_match_transformers():
    """Inverse frequencies and table scale of the rope-scaling descriptions found in HF configs (linear, llama3 as in Llama 3.1+, yarn) against
    transformers' rotary embedding; unknown types are refused."""
    import pytest
    import torch
    from transformers import LlamaConfig as HFConfig
    from transformers.models.llama.modeling_llama import LlamaRotaryEmbedding
    from ferrotorch_b200 import ops
    from ferrotorch_b200.errors import InvalidArgument
    D = 128
    for rs in (None, dict(rope_type="linear", factor=4.0),
               dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=8192),
               dict(rope_type="yarn", factor=8.0, original_max_position_embeddings=2048, beta_fast=32.0, beta_slow=1.0)):
        emb = LlamaRotaryEmbedding(HFConfig(hidden_size=D * 4, num_attention_heads=4, rope_theta=500000.0, max_position_embeddings=16384,
                                            rope_scaling=dict(rs) if rs else None))
        inv, att = ops.llama.rope_inv_freq(D, 500000.0, rs)
        assert float(((emb.inv_freq.double() - inv).abs() / inv).max()) < 1e-6, rs
        assert abs(float(emb.attention_scaling) - att) < 1e-9
        cos, sin = ops.rope_tables(64, D, 500000.0, "cpu", rs)
        ang = torch.outer(torch.arange(64, dtype=torch.float64), inv)
        assert torch.allclose(cos.double(), ang.cos() * att, atol=1e-6) and torch.allclose(sin.double(), ang.sin() * att, atol=1e-6)
    from transformers.modeling_rope_utils import ROPE_INIT_FUNCTIONS
    dyn = HFConfig(hidden_size=D * 4, num_attention_heads=4, rope_theta=10000.0, max_position_embeddings=2048, rope_scaling=dict(rope_type="dynamic", factor=4.0))
    for length in (1024, 2048, 5000, 16384):
        inv_hf, _ = ROPE_INIT_FUNCTIONS["dynamic"](dyn, "cpu", seq_len=length)
        inv, _ = ops.llama.rope_inv_freq(D, 10000.0, dict(rope_type="dynamic", factor=4.0, original_max_position_embeddings=2048), seq_len=length)
        assert float(((inv_hf.double() - inv).abs() / inv).max()) < 1e-6
    # this framework's own descriptions: static NTK base scaling, YaRN without a table scale (ferrotorch-nn/src/transformer.rs:210-266)
    inv_ntk, _ = ops.llama.rope_inv_freq(D, 10000.0, {"type": "ntk", "factor": 4.0})
    assert abs(float(inv_ntk[0]) - 1.0) < 1e-12 and float(inv_ntk[-1]) < 1.0 / 10000.0 ** ((D - 2) / D) / 3.9
    _, att = ops.llama.rope_inv_freq(D, 10000.0, {"type": "yarn", "factor": 8.0, "original_max_position": 2048})
    assert att == 1.0
    with pytest.raises(InvalidArgument):
        ops.rope_tables(8, D, 10000.0, "cpu", {"rope_type": "longrope", "factor": 2.0})


def test_cached_generation_and_sampling_filters_match_transformers():
    """Greedy generation with the KV-cache model from a transformers checkpoint equals ``generate(do_sample=False)``; the top-k, top-p and
    repetition-penalty filters equal transformers' logits processors."""
    import torch
    from transformers import LlamaConfig as HFConfig, LlamaForCausalLM as HFModel
    from transformers.generation.logits_process import RepetitionPenaltyLogitsProcessor, TopKLogitsWarper, TopPLogitsWarper
    from ferrotorch_b200.models import LlamaConfig, llama_gen as G
    torch.manual_seed(0)
    cfg = LlamaConfig.tiny(layers=2, hidden=256, heads=2, kv_heads=1, ffn=512, vocab=512)
    hf = HFModel(HFConfig(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, num_hidden_layers=2,
                          num_attention_heads=2, num_key_value_heads=1, rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta,
                          max_position_embeddings=2048, tie_word_embeddings=False)).float().eval()
    model = G.CachedLlama(cfg, {k: v.clone() for k, v in hf.state_dict().items()})
    ids = torch.randint(0, 512, (2, 9))
    out = G.generate(model, model.new_cache, ids, G.GenerationConfig().with_max_new_tokens(12))
    ref = hf.generate(ids, max_new_tokens=12, do_sample=False, pad_token_id=0)
    assert torch.equal(out[:, -12:], ref[:, -12:])
    logits, seq = torch.randn(3, 512), torch.randint(0, 512, (3, 20))
    assert torch.equal(G.top_k_filter(logits.clone(), 7), TopKLogitsWarper(7)(seq, logits.clone()))
    assert torch.equal(G.top_p_filter(logits.clone(), 0.8), TopPLogitsWarper(0.8)(seq, logits.clone()))
    assert torch.allclose(G.apply_repetition_penalty(logits.clone(), seq, 1.3), RepetitionPenaltyLogitsProcessor(1.3)(seq, logits.clone()))


def test_gptq_and_awq_dequantisation_match_vllm_reference_packers():
    """Weights quantised and packed by vLLM's reference utilities (GPTQ: rows of eight along the input dimension, stored zero = zero point - 1;
    AWQ: interleaved channel order, explicit zero points) come back as the reference's dequantised weights."""
    import pytest
    import torch
    try:
        from vllm.model_executor.layers.quantization.utils import quant_utils as Q
        from vllm.scalar_type import scalar_types
    except Exception as e:                            # the library is an optional oracle
        pytest.skip(f"vllm quantisation utilities not importable: {e}")
    from ferrotorch_b200.models import llama_gen as G
    torch.manual_seed(0)
    K, N, gs = 256, 64, 128
    w = torch.randn(K, N)
    w_ref, q_w, s, _, _ = Q.gptq_quantize_weights(w, scalar_types.uint4b8, gs, act_order=False)
    qzeros = Q.pack_cols(torch.full((K // gs, N), 7, dtype=torch.int32), 4, K // gs, N)
    assert torch.equal(G.dequantize_gptq_q4(Q.gptq_pack(q_w, 4, K, N), qzeros, s, None, gs), w_ref.t().contiguous())
    w_ref, q_w, s, zp = Q.quantize_weights(w, scalar_types.uint4, gs, zero_points=True)
    out = G.dequantize_awq_q4(Q.awq_pack(q_w, 4, K, N), Q.awq_pack(zp.to(torch.int32), 4, K // gs, N), s, gs)
    assert torch.allclose(out, w_ref.t(), atol=1e-6)
