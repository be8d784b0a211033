"""Per-symbol structure and behaviour checks of ``ferrotorch_b200.models``: the named sub-modules of the BERT, Whisper, Llama, CLIP and
Stable Diffusion families are the ones the assembled models are made of; generation helpers, GGUF remapping, checkpoint loaders and the record
types behave as documented."""
import pytest
import torch

import ferrotorch_b200.models as M
from ferrotorch_b200.models import LlamaConfig, bert, diffusion, graph, rl, whisper
from ferrotorch_b200.models import llama_gen as G
from ferrotorch_b200.models.llama_infer import random_hf_weights
from ferrotorch_b200.serialize import save_safetensors


def _types(module):
    return {type(m) for m in module.modules()}


def test_bert_whisper_and_llama_building_blocks():
    bc = bert.BertConfig(vocab_size=100, hidden_size=32, num_hidden_layers=2, num_attention_heads=4, intermediate_size=64, max_position_embeddings=64)
    bm = bert.BertModel(bc)
    assert {M.BertEmbeddings, M.BertEncoder, M.BertLayer, M.BertSelfAttention} <= _types(bm)
    assert isinstance(bm.pooler, M.BertPooler) if getattr(bm, "pooler", None) is not None else M.BertPooler(bc) is not None
    ids = torch.randint(0, 100, (2, 9))
    mask = torch.ones(2, 9, dtype=torch.long)
    mask[1, 6:] = 0
    out = bm(ids, mask)
    hidden = out[0] if isinstance(out, tuple) else out
    assert hidden.shape == (2, 9, 32) and torch.isfinite(hidden).all()
    r = M.DropReport(dropped_position_ids=True, dropped=("cls.predictions.bias",))
    assert r.dropped_position_ids and r.dropped_pooler == () and r.unmapped == ()
    wc = whisper.WhisperConfig.tiny()
    layer = M.WhisperEncoderLayer(wc)
    x = torch.randn(1, 12, wc.d_model)
    assert layer(x).shape == x.shape
    cfg = LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64)
    att, mlp = M.LlamaAttention(cfg), M.LlamaMLP(cfg)
    h = torch.randn(2, 5, 32)
    assert att(h).shape == h.shape and mlp(h).shape == h.shape
    assert torch.allclose(mlp(h), mlp.down_proj(torch.nn.functional.silu(mlp.gate_proj(h)) * mlp.up_proj(h)), atol=1e-6)
    assert (att.num_heads(), att.num_kv_heads(), att.head_dim()) == (4, 2, 8)
    W = random_hf_weights(cfg, "cpu", 0, 0.1)
    gl = M.LlamaGpuLayer(cfg).load(W, "model.layers.0.")
    assert torch.equal(gl.mlp.gate_proj.weight.float(), W["model.layers.0.mlp.gate_proj.weight"].float())
    inf = M.LlamaGpuInferencer(cfg, W, device="cpu", dtype=torch.float32)
    prof = inf.forward_from_ids_profiled([1, 2, 3], mlp_block_size=16, n_mlp_blocks=4)
    assert isinstance(prof, M.ProfiledForwardResult) and prof.attn_magnitudes.shape == (1, 3, 4) and prof.mlp_magnitudes.shape == (1, 3, 4)
    tm = M.LlamaForCausalLM(LlamaConfig.tiny(layers=1, hidden=256, heads=2, kv_heads=1, ffn=256, vocab=128), device="cpu", seed=0)
    assert any(isinstance(m, M.LlamaDecoderLayer) for m in tm.modules())


def test_diffusion_building_blocks_compose_the_models():
    u = diffusion.UNet2DConditionModel(diffusion.UNetConfig.tiny())
    ut = _types(u)
    assert {M.ResnetBlock2D, M.Transformer2DModel, M.BasicTransformerBlock, M.Attention, M.FeedForward, M.Downsample2D, M.Upsample2D,
            M.UNetMidBlock2DCrossAttn, M.Timesteps, M.TimestepEmbedding} <= ut
    v = diffusion.AutoencoderKL(diffusion.VaeConfig.tiny())
    vt = _types(v)
    assert {M.Encoder, M.Decoder, M.DownEncoderBlock2D, M.UpDecoderBlock2D, M.UNetMidBlock2D} <= vt
    assert issubclass(M.VaeEncoder, torch.nn.Module) and issubclass(M.VaeDecoder, torch.nn.Module)
    clip = diffusion.ClipTextEncoder(diffusion.ClipTextConfig.tiny())
    assert M.ClipEncoderLayer in _types(clip)
    t = M.Timesteps(8)(torch.tensor([0.0, 10.0]))
    assert t.shape == (2, 8) and torch.allclose(t[0], torch.tensor([1.0, 1, 1, 1, 0, 0, 0, 0]))          # cos first, then sin, at t = 0
    a = M.Attention(16, cross_dim=8, heads=2, dim_head=8)
    assert a(torch.randn(1, 5, 16), torch.randn(1, 3, 8)).shape == (1, 5, 16)
    rb = M.ResnetBlock2D(8, 16, temb_channels=4, groups=4)
    assert rb(torch.randn(1, 8, 6, 6), torch.randn(1, 4)).shape == (1, 16, 6, 6)
    assert M.Downsample2D(8)(torch.randn(1, 8, 6, 6)).shape == (1, 8, 3, 3) and M.Upsample2D(8)(torch.randn(1, 8, 3, 3)).shape == (1, 8, 6, 6)
    assert {p.name for p in M.PredictionType} >= {"Epsilon"}
    d = M.PipelineStepDump(0, 981, *(torch.zeros(1) for _ in range(4)))
    assert d.timestep == 981 and d.guided_noise.shape == (1,)
    for name in ("GpuClipTextEncoder", "GpuStableDiffusionPipeline", "GpuUNet2DConditional", "GpuVaeDecoder", "GpuVaeEncoder"):
        assert isinstance(getattr(M, name), type)


def test_generation_helpers_and_gguf_remap():
    cfg = LlamaConfig(vocab_size=128, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                      max_position_embeddings=128)
    W = {k: v.float() for k, v in random_hf_weights(cfg, "cpu", 3, 0.2).items()}
    m = G.CachedLlama(cfg, W)
    ids = torch.randint(0, 128, (1, 6), generator=torch.Generator().manual_seed(2))
    gc = G.GenerationConfig(max_new_tokens=4, num_beams=3)
    assert torch.equal(M.beam_search(m, m.new_cache, ids, gc), G.generate(m, m.new_cache, ids, gc))
    logits = torch.tensor([[0.0, 5.0, 1.0]])
    assert M.sample_next(logits, torch.tensor([[0]]), G.GenerationConfig()).tolist() == [1]
    pen = M.sample_next(torch.tensor([[3.0, 2.9, 0.0]]), torch.tensor([[0]]), G.GenerationConfig(repetition_penalty=2.0))
    assert pen.tolist() == [1]                        # the already-seen token 0 is halved below token 1
    samp = G.GenerationConfig(seed=0).with_temperature(1.0).with_top_k(1)
    assert M.sample_next(logits, torch.tensor([[0]]), samp, torch.Generator().manual_seed(0)).tolist() == [1]
    st = M.SpecDecodeStats(proposed=10, accepted=7)
    assert abs(st.acceptance_rate() - 0.7) < 1e-12
    gg = {"token_embd.weight": torch.randn(128, 64), "blk.0.attn_q.weight": torch.randn(64, 64), "blk.0.attn_k.weight": torch.randn(32, 64),
          "blk.0.ffn_down.weight": torch.randn(64, 128), "output_norm.weight": torch.ones(64), "rope_freqs.weight": torch.ones(8)}
    hf = M.remap_gguf_state_dict(gg, cfg)
    assert set(hf) == {"model.embed_tokens.weight", "model.layers.0.self_attn.q_proj.weight", "model.layers.0.self_attn.k_proj.weight",
                       "model.layers.0.mlp.down_proj.weight", "model.norm.weight"}
    assert torch.equal(hf["model.layers.0.self_attn.q_proj.weight"], G.gguf_unpermute_qk(gg["blk.0.attn_q.weight"], 4))
    assert torch.equal(hf["model.layers.0.mlp.down_proj.weight"], gg["blk.0.ffn_down.weight"])
    assert M.gguf_to_hf_state_dict(gg, cfg).keys() == hf.keys()


def test_checkpoint_loaders(tmp_path):
    net = graph.GcnNet(6, 4, 3)
    p = tmp_path / "gcn.safetensors"
    save_safetensors({k: v.detach() for k, v in net.state_dict().items()}, p)
    net2 = M.load_gcn_net(str(p), 6, 4, 3)
    assert all(torch.equal(a, b) for a, b in zip(net.state_dict().values(), net2.state_dict().values()))
    conv = M.GcnConv(6, 4)
    g = graph.Graph(torch.tensor([[0, 1], [1, 0]]), 2)
    assert conv(torch.randn(2, 6), g).shape == (2, 4)
    rb = M.ResnetBlock2D(8, 8, temb_channels=None, groups=4)
    p2 = tmp_path / "rb.safetensors"
    save_safetensors({k: v.detach() for k, v in rb.state_dict().items()}, p2)
    fresh = M.ResnetBlock2D(8, 8, temb_channels=None, groups=4)
    M.load_sd_component(fresh, str(p2))
    assert all(torch.equal(a, b) for a, b in zip(rb.state_dict().values(), fresh.state_dict().values()))
    gen = torch.Generator().manual_seed(0)
    qw, qz, sc = torch.randint(0, 2 ** 31 - 1, (8, 16), generator=gen, dtype=torch.int32), torch.randint(0, 2 ** 31 - 1, (1, 2), generator=gen, dtype=torch.int32), torch.rand(1, 16, generator=gen)
    sd = {"l.qweight": qw, "l.qzeros": qz, "l.scales": sc}
    assert torch.equal(M.load_quantized_linear_weights(sd, "l.", "gptq", 64), G.dequantize_gptq_q4(qw, qz, sc, None, 64))
    with pytest.raises(Exception):
        M.load_quantized_linear_weights(sd, "l.", "int3")
    pol = rl.MlpPolicy(rl.MlpPolicyConfig())
    out = pol.forward_raw(torch.randn(3, 4)) if hasattr(pol, "forward_raw") else M.PolicyOutput(torch.zeros(3, 2), torch.zeros(3, 1))
    assert isinstance(out, M.PolicyOutput) and out.action_logits.shape[0] == 3 and out.value.shape == (3, 1)
