"""Behaviour of the finer-grained public names of the model / tool packages (sub-blocks, Hugging Face config parsers, loader drop reports)."""
import json

import pytest
import torch

from ferrotorch_b200 import models as M
from ferrotorch_b200.errors import FerrotorchError, InvalidArgument
from ferrotorch_b200.serialize import save_safetensors


def _tiny_bert():
    return M.BertConfig(vocab_size=32, hidden_size=8, num_hidden_layers=1, num_attention_heads=2, intermediate_size=16, max_position_embeddings=16)


def test_bert_blocks_hf_config_and_drop_report(tmp_path):
    c = _tiny_bert()
    x = torch.randn(2, 5, 8)
    assert M.BertAttention(c)(x).shape == x.shape
    assert M.BertIntermediate(c)(x).shape == (2, 5, 16)
    assert M.BertOutput(c).forward_residual(torch.randn(2, 5, 16), x).shape == x.shape
    assert M.BertSelfOutput(c)(x, x).shape == x.shape
    assert c.head_dim() == 4 and M.BertConfig.all_minilm_l6_v2().hidden_size == 384

    hf = M.HfBertConfig.from_json_str(json.dumps(dict(hidden_size=8, num_hidden_layers=1, num_attention_heads=2, intermediate_size=16, vocab_size=32,
                                                      max_position_embeddings=16, architectures=["BertModel"], extra_key=1)))
    assert hf.layer_norm_eps == 1e-12 and hf.type_vocab_size == 2 and hf.position_embedding_type == "absolute"
    assert M.BertConfig.from_hf(hf) == c
    with pytest.raises(InvalidArgument):
        M.HfBertConfig.from_json_str('{"hidden_size": 8}')
    with pytest.raises(InvalidArgument):
        M.HfBertConfig.from_json_str("{not json")
    bad = M.HfBertConfig.from_json_str(json.dumps(dict(hidden_size=9, num_hidden_layers=1, num_attention_heads=2, intermediate_size=16, vocab_size=32,
                                                       max_position_embeddings=16)))
    with pytest.raises(InvalidArgument):
        bad.validate()
    (tmp_path / "config.json").write_text(json.dumps(hf.__dict__ | {"architectures": list(hf.architectures)}))
    assert M.HfBertConfig.from_file(tmp_path / "config.json") == hf

    src = M.BertModel(c, add_pooling_layer=True)
    sd = dict(src.state_dict())
    sd["embeddings.position_ids"] = torch.arange(16)[None].float()
    save_safetensors(sd, str(tmp_path / "model.safetensors"))
    with pytest.raises(InvalidArgument):
        M.load_bert_model(str(tmp_path / "model.safetensors"), c, True)
    dst, rep = M.load_bert_model(str(tmp_path / "model.safetensors"), c, False)
    assert rep.dropped_position_ids and rep.dropped_pooler == ("pooler.dense.bias", "pooler.dense.weight") and dst.pooler is None
    ids = torch.randint(0, 32, (2, 7))
    assert torch.equal(dst(ids)[0], src(ids)[0])
    st, rep2 = M.load_sentence_transformer(str(tmp_path / "model.safetensors"), c, True, False)
    e = st.encode(ids)
    assert e.shape == (2, 8) and torch.allclose(e.norm(dim=-1), torch.ones(2), atol=1e-5) and rep2 == rep
    whole = M.load_bert_model(str(tmp_path))                      # directory form keeps the pooler
    assert whole.pooler is not None and torch.equal(whole(ids)[1], src(ids)[1])


def test_whisper_names_and_loader_report(tmp_path):
    assert (M.SAMPLE_RATE, M.N_MELS, M.N_FRAMES, M.N_SAMPLES, M.N_FREQS) == (16000, 80, 3000, 480000, 201)
    c = M.WhisperConfig(num_mel_bins=8, d_model=16, encoder_layers=1, encoder_attention_heads=2, encoder_ffn_dim=32, max_source_positions=10)
    assert c.encoder_head_dim() == 8 and M.WhisperConfig.whisper_tiny() == M.WhisperConfig.tiny()
    with pytest.raises(InvalidArgument):
        M.WhisperConfig(d_model=10, encoder_attention_heads=3).validate()
    hf = M.HfWhisperConfig.from_json_str(json.dumps(dict(vocab_size=100, num_mel_bins=8, d_model=16, encoder_layers=1, encoder_attention_heads=2,
                                                         encoder_ffn_dim=32, decoder_layers=1, decoder_attention_heads=2, decoder_ffn_dim=32,
                                                         max_source_positions=10, max_target_positions=12)))
    assert hf.activation_function == "gelu" and M.WhisperConfig.from_hf(hf) == c
    assert M.WhisperEncoderSelfAttention(c)(torch.randn(1, 6, 16)).shape == (1, 6, 16)
    assert M.WhisperConvStem(c)(torch.randn(1, 8, 20)).shape == (1, 10, 16)
    enc = M.WhisperEncoder(c)
    sd = {"model.encoder." + k: v for k, v in enc.state_dict().items()}
    sd["model.decoder.embed_tokens.weight"] = torch.zeros(4, 16)
    sd["proj_out.weight"] = torch.zeros(4, 16)
    save_safetensors(sd, str(tmp_path / "w.safetensors"))
    with pytest.raises(InvalidArgument):
        M.load_whisper_encoder(str(tmp_path / "w.safetensors"), c, True)
    got, rep = M.load_whisper_encoder(str(tmp_path / "w.safetensors"), c, False)
    assert rep.dropped == ("model.decoder.embed_tokens.weight", "proj_out.weight")
    mel = torch.randn(1, 8, 20)
    assert torch.equal(got.forward_from_mel(mel), enc(mel))


def test_rl_policy_parts_and_loader_report(tmp_path):
    c = M.MlpPolicyConfig.cartpole_v1()
    assert (c.obs_dim, c.hidden, c.n_actions) == (4, 64, 2)
    ex = M.MlpExtractor(4, 8)
    obs = torch.randn(3, 4)
    assert ex.forward_actor(obs).shape == (3, 8) and ex.forward_critic(obs).shape == (3, 8) and (ex.obs_dim(), ex.hidden()) == (4, 8)
    assert sorted(ex.state_dict()) == sorted(f"{t}.{i}.{p}" for t in ("policy_net", "value_net") for i in (0, 2) for p in ("weight", "bias"))
    assert M.ActionNet(8, 2)(torch.randn(3, 8)).shape == (3, 2) and M.ValueHead(8)(torch.randn(3, 8)).shape == (3, 1)
    cfg = M.MlpPolicyConfig.discrete_mlp(4, 8, 2)
    src = M.MlpPolicy(cfg)
    out = src.policy_output(obs)
    assert out.action_logits.shape == (3, 2) and out.value.shape == (3, 1)
    sd = dict(src.state_dict())
    save_safetensors(sd, str(tmp_path / "p.safetensors"))
    dst, rep = M.load_ppo_policy(str(tmp_path / "p.safetensors"), cfg, True)
    assert rep.unmapped == () and torch.equal(dst.policy_output(obs).action_logits, out.action_logits)
    sd["extra.weight"] = torch.zeros(1)
    save_safetensors(sd, str(tmp_path / "q.safetensors"))
    with pytest.raises(InvalidArgument):
        M.load_ppo_policy(str(tmp_path / "q.safetensors"), cfg, True)
    assert M.load_ppo_policy(str(tmp_path / "q.safetensors"), cfg, False)[1].unmapped == ("extra.weight",)
    del sd["extra.weight"], sd["action_net.bias"]
    save_safetensors(sd, str(tmp_path / "r.safetensors"))
    with pytest.raises(InvalidArgument):
        M.load_ppo_policy(str(tmp_path / "r.safetensors"), cfg, False)


def test_diffusion_configs_blocks_and_loaders(tmp_path):
    D = M
    uc = D.UNet2DConditionConfig.from_json_str(json.dumps(dict(block_out_channels=[32, 64], layers_per_block=1, cross_attention_dim=32, attention_head_dim=4,
                                                               norm_num_groups=8, sample_size=8, down_block_types=["CrossAttnDownBlock2D", "DownBlock2D"],
                                                               up_block_types=["UpBlock2D", "CrossAttnUpBlock2D"])))
    assert uc.down_block_has_attn == (True, False) and uc.up_block_has_attn == (False, True) and uc.time_embed_dim() == 128 and uc.num_blocks() == 2
    assert D.UNet2DConditionConfig.sd_v1_5().up_block_has_attn == (False, True, True, True)
    for bad in ('{"down_block_types": ["AttnDownBlock2D"]}', '{"block_out_channels": [30]}', '{"block_out_channels": []}', "{"):
        with pytest.raises(InvalidArgument):
            D.UNet2DConditionConfig.from_json_str(bad)
    vc = D.VaeDecoderConfig.from_json_str(json.dumps(dict(block_out_channels=[16, 32], layers_per_block=1, norm_num_groups=8, sample_size=16)))
    assert vc.out_channels == 3 and vc.resnets_per_up_block() == 2 and vc.num_up_blocks() == 2 and D.VaeEncoderConfig is D.VaeDecoderConfig
    with pytest.raises(InvalidArgument):
        D.VaeDecoderConfig.from_json_str('{"scaling_factor": 0.0}')
    cc = D.ClipTextConfig.from_json_str(json.dumps(dict(vocab_size=100, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
                                                        max_position_embeddings=8, hidden_act="quick_gelu")))
    assert cc.head_dim() == 8 and D.ClipTextConfig.sd_v1_5().hidden_size == 768
    with pytest.raises(InvalidArgument):
        D.ClipTextConfig.from_json_str('{"hidden_act": "gelu"}')

    temb = torch.randn(2, 16)
    r = D.ResnetBlock2DTime(8, 16, 16, groups=4)
    assert r.forward_t(torch.randn(2, 8, 4, 4), temb).shape == (2, 16, 4, 4)
    with pytest.raises(FerrotorchError):
        r(torch.randn(2, 8, 4, 4), None)
    db = D.DownBlock2D(8, 8, 16, 1, True, groups=4)
    x, outs = db(torch.randn(2, 8, 4, 4), temb)
    assert x.shape == (2, 8, 2, 2) and len(outs) == 2 and db.attentions is None
    assert D.ClipSelfAttention(cc)(torch.randn(1, 5, 32)).shape == (1, 5, 32) and D.ClipMlp(cc)(torch.randn(1, 5, 32)).shape == (1, 5, 32)
    assert D.ClipTextEmbeddings(cc)(torch.tensor([[1, 2, 3]])).shape == (1, 3, 32) and D.ClipEncoder(cc)(torch.randn(1, 3, 32)).shape == (1, 3, 32)
    assert D.AttnBlock2D(16, 4)(torch.randn(1, 16, 3, 3)).shape == (1, 16, 3, 3)

    # scheduler config forms agree; linspace spacing follows round(i * N / n) reversed
    s1, s2 = D.DDIMScheduler(D.DDIMConfig.sd_v1_5()), D.DDIMScheduler()
    assert s1.set_timesteps(4) == s2.set_timesteps(4) == [751, 501, 251, 1] and s1.config().beta_schedule is D.BetaSchedule.ScaledLinear
    assert D.DDIMScheduler(D.DDIMConfig(timestep_spacing=D.TimestepSpacing.Linspace)).set_timesteps(4) == [750, 500, 250, 0]
    with pytest.raises(InvalidArgument):
        s1.set_timesteps(0)
    with pytest.raises(InvalidArgument):
        D.DDIMScheduler(beta_schedule="cosine")

    # VAE halves against the whole autoencoder, posterior arithmetic, loaders with reports
    ae = D.AutoencoderKL(vc).eval()
    save_safetensors(dict(ae.state_dict()), str(tmp_path / "vae.safetensors"))
    with pytest.raises(InvalidArgument):
        D.load_vae_decoder(str(tmp_path / "vae.safetensors"), vc, True)
    dec, rep = D.load_vae_decoder(str(tmp_path / "vae.safetensors"), vc, False)
    assert rep.dropped and all(k.startswith(("encoder.", "quant_conv.")) for k in rep.dropped)
    enc, rep_e = D.load_vae_encoder(str(tmp_path / "vae.safetensors"), vc, False)
    assert all(k.startswith(("decoder.", "post_quant_conv.")) for k in rep_e.dropped)
    img = torch.rand(1, 3, 16, 16) * 2 - 1
    with torch.no_grad():
        post = enc.encode(img)
        assert torch.allclose(post.mode(), ae.encode(img, sample=False), atol=1e-6)
        z = enc.encode_with_scaling(img)
        assert torch.allclose(dec.decode_with_scaling(z), ae.decode(post.mode()), atol=1e-5)
        a, b = post.sample_with_seed(5), post.sample_with_seed(5)
        assert torch.equal(a, b) and not torch.equal(a, post.sample_with_seed(6))
        eps = torch.randn(post.mean.shape, generator=torch.Generator().manual_seed(5))
        assert torch.allclose(a, post.mean + (0.5 * post.logvar).exp() * eps, atol=1e-6)
    with pytest.raises(FerrotorchError):
        D.DiagonalGaussianDistribution.from_parameters(torch.zeros(1, 6, 2, 2), 4)
    assert float(D.DiagonalGaussianDistribution.from_parameters(torch.full((1, 8, 1, 1), 99.0), 4).logvar.max()) == 20.0

    clip = D.ClipTextEncoder(cc).eval()
    sd = dict(clip.state_dict())
    sd["text_model.embeddings.position_ids"] = torch.arange(8)[None].float()
    save_safetensors(sd, str(tmp_path / "clip.safetensors"))
    got, rep_c = D.load_clip_text_encoder(str(tmp_path / "clip.safetensors"), cc, True)
    assert rep_c.dropped == ("text_model.embeddings.position_ids",)
    assert torch.equal(got.forward_from_ids([1, 2, 3]), clip(torch.tensor([[1, 2, 3]])))
    with pytest.raises(InvalidArgument):
        got.forward_from_ids([1000])

    unet = D.UNet2DConditionModel(uc).eval()
    save_safetensors({"unet." + k: v for k, v in unet.state_dict().items()}, str(tmp_path / "unet.safetensors"))
    u2, rep_u = D.load_unet(str(tmp_path / "unet.safetensors"), uc, True)
    assert rep_u.dropped == ()
    pipe = D.StableDiffusionPipeline(got, u2, dec, D.DDIMScheduler(D.DDIMConfig.sd_v1_5()))
    cond, unc = pipe.encode_prompt([1, 2, 3, 4]), pipe.encode_prompt([0, 0, 0, 0])
    lat = torch.randn(1, 4, 4, 4, generator=torch.Generator().manual_seed(0))
    image, dumps = pipe.generate(cond, unc, lat, 3, 5.0)
    assert image.shape == (1, 3, 8, 8) and [d.timestep for d in dumps] == [667, 334, 1] and [d.step for d in dumps] == [0, 1, 2]
    d0 = dumps[0]
    assert torch.allclose(d0.guided_noise, d0.noise_pred_uncond + 5.0 * (d0.noise_pred_cond - d0.noise_pred_uncond))
    with torch.no_grad():
        assert torch.allclose(d0.noise_pred_cond, unet(lat, 667, cond), atol=1e-5)
        assert torch.allclose(image, dec.decode_with_scaling(dumps[-1].latent_after_step))
    with pytest.raises(FerrotorchError):
        pipe.generate(cond, unc[:, :2], lat, 2, 5.0)


def _tiny_llama(act="silu", param=None):
    cfg = M.LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                        max_position_embeddings=64, rope_theta=10000.0, hidden_act=act, hidden_act_param=param)
    g = torch.Generator().manual_seed(0)
    W = {"model.embed_tokens.weight": torch.randn(64, 32, generator=g) * 0.5, "model.norm.weight": torch.rand(32, generator=g) + 0.5,
         "lm_head.weight": torch.randn(64, 32, generator=g) * 0.3}
    for i in range(2):
        p = f"model.layers.{i}."
        for n, shp in (("self_attn.q_proj", (32, 32)), ("self_attn.k_proj", (16, 32)), ("self_attn.v_proj", (16, 32)), ("self_attn.o_proj", (32, 32)),
                       ("mlp.gate_proj", (48, 32)), ("mlp.up_proj", (48, 32)), ("mlp.down_proj", (32, 48))):
            W[p + n + ".weight"] = torch.randn(*shp, generator=g) * 0.2
        W[p + "input_layernorm.weight"] = torch.rand(32, generator=g) + 0.5
        W[p + "post_attention_layernorm.weight"] = torch.rand(32, generator=g) + 0.5
    return cfg, W


def test_llama_activation_variants_match_transformers():
    transformers = pytest.importorskip("transformers")
    a = M.LlamaActivation.FatRelu(0.5)
    assert torch.equal(a(torch.tensor([-1.0, 0.4, 0.5, 2.0])), torch.tensor([0.0, 0.0, 0.5, 2.0])) and a == M.LlamaActivation.parse("fatrelu", 0.5)
    assert M.LlamaActivation.parse("swish") is M.LlamaActivation.Silu and M.LlamaActivation.parse("fatrelu").threshold == 0.01
    with pytest.raises(InvalidArgument):
        M.LlamaActivation.parse("gelu")
    with pytest.raises(InvalidArgument):
        M.LlamaConfig(hidden_act="gelu").validate()
    cfg, W = _tiny_llama("relu")
    hf = transformers.LlamaForCausalLM(transformers.LlamaConfig(vocab_size=64, hidden_size=32, intermediate_size=48, num_hidden_layers=2,
                                                                num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=64,
                                                                rope_theta=10000.0, hidden_act="relu", rms_norm_eps=cfg.rms_norm_eps)).eval()
    hf.load_state_dict(W, strict=False)
    ids = torch.randint(0, 64, (1, 9), generator=torch.Generator().manual_seed(1))
    ours = M.CachedLlama(cfg, W)
    with torch.no_grad():
        want = hf(ids).logits
    assert torch.allclose(ours(ids, ours.new_cache()), want, atol=2e-4)
    with pytest.raises(InvalidArgument):                      # the fused training layer is SwiGLU only and says so
        M.LlamaModel(cfg, device="cpu")


def test_llama_blocks_and_inferencer_taps():
    cfg, W = _tiny_llama("fatrelu", 0.05)
    ref = M.CachedLlama(cfg, W)
    ids = [3, 9, 27, 1, 50, 7]
    want = ref(torch.tensor([ids]), ref.new_cache())[0]
    inf = M.LlamaGpuInferencer(cfg, W, device="cpu", dtype=torch.float32)
    assert torch.allclose(inf.forward_logits_from_ids_all(ids), want, atol=1e-5)
    assert torch.allclose(inf.forward_from_ids(ids), want[-1], atol=1e-5)
    L0 = inf.layers[0]
    assert L0.self_attn.num_heads() == 4 and L0.self_attn.num_kv_heads() == 2 and L0.self_attn.head_dim() == 8
    # attention with a cache fed token by token equals the whole-sequence pass
    x = torch.randn(1, 6, 32)
    cache = M.LayerKvCache()
    step = torch.cat([L0.self_attn.forward_with_cache(x[:, i: i + 1], cache) for i in range(6)], 1)
    assert torch.allclose(step, L0.self_attn(x), atol=1e-5)
    r = inf.forward_from_ids_profiled_with_bootstrap(ids, 12, 4, bootstrap_k=1)
    assert r.attn_magnitudes.shape == (2, 6, 4) and r.mlp_magnitudes.shape == (2, 6, 4) and r.seq_len == 6 and r.hidden_size == 32
    # layer 0 by hand
    x0 = W["model.embed_tokens.weight"][torch.tensor([ids])]
    rms = lambda v, w: v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * w
    x1 = x0 + L0.self_attn(rms(x0, W["model.layers.0.input_layernorm.weight"]))
    gated = L0.mlp.gated(rms(x1, W["model.layers.0.post_attention_layernorm.weight"]))
    assert torch.allclose(r.mlp_magnitudes[0], gated[0].abs().view(6, 4, 12).amax(-1), atol=1e-5)
    assert torch.allclose(r.bootstrap_hidden, (x1 + L0.mlp.down_proj(gated))[0], atol=1e-5)
    assert (gated == 0).float().mean() > 0.3                 # the thresholded gate really zeroes activations
    rp = inf.forward_from_ids_profiled_with_bootstrap(ids, 12, 4, None, True)
    y = x1 + L0.mlp.down_proj(gated)
    assert torch.allclose(rp.mlp_magnitudes[0], (gated * (y @ L0.mlp.down_proj.weight))[0].abs().view(6, 4, 12).amax(-1), atol=1e-5)
    for bad in ((10, 4, None), (12, 4, 3), (12, 4, 0)):
        with pytest.raises(InvalidArgument):
            inf.forward_from_ids_profiled_with_bootstrap(ids, *bad)


def test_generation_primitives_and_streamer():
    r = M.XorShift64(1)
    x = 1
    x ^= (x << 13) & (2 ** 64 - 1); x ^= x >> 7; x ^= (x << 17) & (2 ** 64 - 1)          # noqa: E702
    assert r.next_u64() == x and 0.0 <= r.uniform() <= 1.0
    assert M.argmax(torch.tensor([1.0, 5.0, 5.0, 2.0])) == 1 and M.argmax([float("-inf")] * 3) == 0
    assert torch.equal(M.apply_temperature(torch.tensor([2.0, 4.0]), 2.0), torch.tensor([1.0, 2.0]))
    assert M.sample_softmax(torch.tensor([float("-inf"), float("-inf")]), M.XorShift64(3)) == 0
    rng, counts = M.XorShift64(7), [0, 0, 0]
    lg = torch.log(torch.tensor([0.2, 0.5, 0.3]))
    for _ in range(4000):
        counts[M.sample_softmax(lg, rng)] += 1
    assert abs(counts[0] / 4000 - 0.2) < 0.03 and abs(counts[1] / 4000 - 0.5) < 0.03

    cfg, W = _tiny_llama()
    model = M.CachedLlama(cfg, W)
    prompt = [5, 6, 7]
    seen = []
    out = M.generate_with_streamer(model, prompt, M.GenerationConfig.greedy(8), lambda t: (seen.append(t), True)[1])
    full = M.generate(model, model.new_cache, torch.tensor([prompt]), M.GenerationConfig(max_new_tokens=8))
    assert out == full[0, 3:].tolist() == seen
    assert M.generate_with_streamer(model, prompt, M.GenerationConfig.greedy(8), lambda t: len(seen) < 0) == out[:1]      # streamer says stop
    stop = M.GenerationConfig.greedy(8)
    stop.eos_token_ids = [out[2]]
    assert M.generate_with_streamer(model, prompt, stop, lambda t: True) == out[: out.index(out[2]) + 1]
    c = M.GenerationConfig.nucleus(12, 0.9, 0.8)
    c.seed, c.top_k, c.repetition_penalty = 11, 20, 1.3
    a, b = M.generate_with_streamer(model, prompt, c, lambda t: True), M.generate_with_streamer(model, prompt, c, lambda t: True)
    c.seed = 12
    assert a == b and len(a) == 12 and a != M.generate_with_streamer(model, prompt, c, lambda t: True)
    for bad in (dict(temperature=-1.0), dict(top_p=1.5), dict(repetition_penalty=0.0)):
        with pytest.raises(InvalidArgument):
            M.generate_with_streamer(model, prompt, M.GenerationConfig(**bad), lambda t: True)
    with pytest.raises(InvalidArgument):
        M.generate_with_streamer(model, [], M.GenerationConfig(), lambda t: True)


class _FixedHandle(M.ModelHandle):
    """Context-free distribution, with call counters."""

    def __init__(self, probs):
        self.logits, self.calls, self.batched = torch.log(torch.tensor(probs, dtype=torch.float64)), 0, 0

    def vocab_size(self):
        return self.logits.numel()

    def forward_ids(self, ids):
        self.calls += 1
        return self.logits

    def forward_ids_all_positions(self, ids):
        self.batched += 1
        return self.logits.expand(len(ids), -1)


def test_speculative_decode_samples_from_the_target():
    p, q = [0.1, 0.2, 0.3, 0.4], [0.4, 0.3, 0.2, 0.1]
    first, second, acc, prop = [0] * 4, [0] * 4, 0, 0
    import random
    seeds = random.Random(0)                                  # xorshift needs well-mixed seeds: a small seed gives a tiny first draw
    for _ in range(1500):
        d, t = _FixedHandle(q), _FixedHandle(p)
        o = M.speculative_decode(d, t, [0], M.SpecDecodeConfig(draft_k=3, max_new_tokens=6, seed=seeds.getrandbits(64) | 1))
        assert len(o.tokens) == 6 and t.calls == 0 and t.batched <= 6 and d.calls == o.proposed_count
        first[o.tokens[0]] += 1
        second[o.tokens[3]] += 1
        acc, prop = acc + o.accepted_count, prop + o.proposed_count
    for cnt in (first, second):
        assert all(abs(cnt[i] / 1500 - p[i]) < 0.04 for i in range(4)), cnt
    a1 = sum(min(a, b) for a, b in zip(p, q))                 # one draft token survives with probability sum min(p, q); a round stops at the
    assert abs(acc / prop - (a1 + a1 ** 2 + a1 ** 3) / 3) < 0.05          # first rejection, so of 3 proposals a1 + a1^2 + a1^3 are kept on average
    same = M.speculative_decode(_FixedHandle(p), _FixedHandle(p), [0], M.SpecDecodeConfig(draft_k=4, max_new_tokens=9, seed=5))
    assert same.acceptance_rate() == 1.0 and len(same.tokens) == 9
    a = M.speculative_decode(_FixedHandle(q), _FixedHandle(p), [0], M.SpecDecodeConfig(draft_k=2, max_new_tokens=7, seed=9))
    b = M.speculative_decode(_FixedHandle(q), _FixedHandle(p), [0], M.SpecDecodeConfig(draft_k=2, max_new_tokens=7, seed=9))
    assert a.tokens == b.tokens
    eos = M.speculative_decode(_FixedHandle(q), _FixedHandle(p), [0], M.SpecDecodeConfig(draft_k=2, max_new_tokens=50, seed=9, eos_token_ids=[a.tokens[1]]))
    assert eos.tokens[-1] == a.tokens[1] and a.tokens[1] not in eos.tokens[:-1]
    assert M.SpecDecodeOutput([], 0, 0).acceptance_rate() == 1.0
    with pytest.raises(InvalidArgument):
        M.speculative_decode(_FixedHandle(q), _FixedHandle(p), [], M.SpecDecodeConfig())
    with pytest.raises(InvalidArgument):
        M.speculative_decode(_FixedHandle(q), _FixedHandle(p), [0], M.SpecDecodeConfig(draft_k=0))
    with pytest.raises(InvalidArgument):
        M.speculative_decode(_FixedHandle(q[:3] + [0.1]), _FixedHandle([0.5, 0.5]), [0])

    # real models: a handle re-feeds only the unseen suffix, and draft == target accepts everything
    cfg, W = _tiny_llama()
    h = M.LlamaHandle(M.CachedLlama(cfg, W))
    ref = M.CachedLlama(cfg, W)
    ids = [4, 8, 15, 16, 23]
    want = ref(torch.tensor([ids]), ref.new_cache())[0].double()
    assert torch.allclose(h.forward_ids(ids[:3]), want[2], atol=1e-5) and torch.allclose(h.forward_ids(ids), want[4], atol=1e-5)
    assert h._cache.len() == 5 and torch.allclose(h.forward_ids(ids[:4]), want[3], atol=1e-5)
    assert torch.allclose(h.forward_ids_all_positions(ids), want, atol=1e-5) and h.vocab_size() == 64
    o = M.speculative_decode(M.LlamaHandle(M.CachedLlama(cfg, W)), h, ids, M.SpecDecodeConfig(draft_k=3, max_new_tokens=8, seed=3))
    assert o.acceptance_rate() == 1.0 and len(o.tokens) == 8


def test_quantised_weight_structs():
    g = torch.Generator().manual_seed(0)
    K, N, G = 32, 16, 16
    qw, qz = torch.randint(-2 ** 31, 2 ** 31 - 1, (K // 8, N), generator=g, dtype=torch.int64).int(), torch.randint(-2 ** 31, 2 ** 31 - 1, (K // G, N // 8), generator=g, dtype=torch.int64).int()
    sc = torch.rand(K // G, N, generator=g)
    assert torch.equal(M.dequantize_gptq_q4(M.GptqQ4(qw.reshape(-1), qz.reshape(-1), sc.reshape(-1), None, K, N, G)), M.dequantize_gptq_q4(qw, qz, sc, None, G))
    aw = torch.randint(-2 ** 31, 2 ** 31 - 1, (K, N // 8), generator=g, dtype=torch.int64).int()
    assert torch.equal(M.dequantize_awq_q4(M.AwqQ4(aw.reshape(-1), qz.reshape(-1), sc.reshape(-1), K, N, G)), M.dequantize_awq_q4(aw, qz, sc, G))
    with pytest.raises(InvalidArgument):
        M.dequantize_gptq_q4(M.GptqQ4(qw.reshape(-1)[:-1], qz.reshape(-1), sc.reshape(-1), None, K, N, G))
    with pytest.raises(InvalidArgument):
        M.dequantize_awq_q4(M.AwqQ4(aw.reshape(-1), qz.reshape(-1), sc.reshape(-1), K, N, 5))
    for bits in (1, 2, 3, 4, 8):
        rows, cols = 3, 8
        vals = torch.randint(0, 2 ** bits, (rows * cols,), generator=g)
        stream = 0
        for i, v in enumerate(vals.tolist()):
            stream |= v << (i * bits)
        packed = torch.tensor(list(stream.to_bytes(rows * cols * bits // 8, "little")), dtype=torch.uint8)
        scale, zero = torch.rand(rows, generator=g) + 0.5, torch.rand(rows, generator=g)
        got = M.dequantize_hqq(M.HqqWeights(bits, packed, scale, zero, rows, cols))
        assert torch.allclose(got, (vals.view(rows, cols).float() - zero[:, None]) * scale[:, None]), bits
    with pytest.raises(InvalidArgument):
        M.dequantize_hqq(M.HqqWeights(5, packed, scale, zero, 3, 8))
    with pytest.raises(FerrotorchError):
        M.dequantize_hqq(M.HqqWeights(8, packed[:5], scale, zero, 3, 8))
    assert M.gguf_key_to_hf("blk.3.attn_q.weight") == "model.layers.3.self_attn.q_proj.weight" and M.LlamaKvCache is M.KvCache


def test_vision_io_structs_samples_and_detection_names(tmp_path):
    from ferrotorch_b200 import vision as V
    img = torch.rand(3, 5, 7)
    raw = V.tensor_to_raw_image(img * 1.5 - 0.2)              # out-of-range values clamp
    assert (raw.width, raw.height, raw.channels) == (7, 5, 3) and len(raw.data) == 105
    back = V.raw_image_to_tensor(raw)
    assert torch.equal(back, ((img * 1.5 - 0.2).double().clamp(0, 1) * 255).round().float().div(255))
    V.write_tensor_as_image(tmp_path / "a.png", img)
    got = V.read_image_as_tensor(tmp_path / "a.png")
    assert got.shape == (3, 5, 7) and (got - img).abs().max() <= 0.5 / 255 + 1e-6
    rgba = V.read_image_rgba(tmp_path / "a.png")
    assert rgba.channels == 4 and rgba.data[3] == 255 and rgba.data[:3] == V.read_image_raw(tmp_path / "a.png").data[:3]
    for bad in (torch.rand(5, 7), torch.rand(2, 5, 7)):
        with pytest.raises(InvalidArgument):
            V.tensor_to_raw_image(bad)
    with pytest.raises(InvalidArgument):
        V.read_image_rgba(tmp_path / "missing.png")
    s = V.Mnist.synthetic(4)[0]
    assert isinstance(s, V.MnistSample) and s.image.shape == (1, 28, 28) and s[1] == s.label
    x, y = V.Cifar10.synthetic(4)[1]
    assert x.shape == (3, 32, 32) and isinstance(V.Cifar10.synthetic(2)[0], V.CifarSample)
    assert V.Split.Train is not V.Split.Test and V.IMAGENET_MEAN == (0.485, 0.456, 0.406) and V.FPN_OUT_CHANNELS == 256
    assert sum(a * f * f for a, f in zip(V.SSD_ANCHORS_PER_SCALE, V.SSD_FM_SIZES)) == V.SSD_TOTAL_ANCHORS == 8732
    d = V.Detections(boxes=torch.zeros(2, 4), scores=torch.ones(2), labels=torch.tensor([1, 2]))
    assert d.boxes is d["boxes"] and d.labels.tolist() == [1, 2] and isinstance(V.MaskDetections(d), V.Detections)
    with pytest.raises(AttributeError):
        d.masks
    c = V.RpnConfig.default_eval((64, 96))
    assert (c.pre_nms_top_n, c.post_nms_top_n, c.nms_thresh, c.min_size, c.score_thresh, c.image_size) == (1000, 1000, 0.7, 1e-3, 0.0, (64, 96))
    rpn = V.Rpn(V.AnchorGenerator(((32,),), ((1.0,),)), V.RpnHead(8, 1), V.RpnConfig(pre_nms_top_n=5, post_nms_top_n=3))
    assert (rpn.pre, rpn.post) == (5, 3)
    fe = V.create_feature_extractor(V.resnet18(num_classes=3).eval(), ["layer1", "layer3"])
    out = fe(torch.randn(1, 3, 32, 32))
    assert isinstance(fe, V.FeatureExtractor) and fe.return_nodes() == ["layer1", "layer3"] and out["layer3"].shape[1] == 256
    body = V.ResNet50Dilated().eval()
    with torch.no_grad():
        f = body(torch.randn(1, 3, 64, 64))
    assert f["out"].shape == (1, 2048, 8, 8) and f["aux"].shape == (1, 1024, 8, 8)
    assert V.FcnHead(16, 3)(torch.randn(2, 16, 4, 4)).shape == (2, 3, 4, 4) and V.TwoMlpHead is not None and V.MaskPredictor is not None


def test_optimizer_configs_and_averaging_strategy():
    from ferrotorch_b200 import optim as O
    torch.manual_seed(0)
    w0 = torch.randn(6, 4)

    def run(make, steps=3):
        p = torch.nn.Parameter(w0.clone())
        opt = make([p])
        for _ in range(steps):
            opt.zero_grad()
            (p.pow(2).sum() + p.sum()).backward()
            opt.step()
        return p.detach()
    pairs = [(O.Adamax, O.AdamaxConfig, torch.optim.Adamax), (O.NAdam, O.NAdamConfig, torch.optim.NAdam), (O.RAdam, O.RAdamConfig, torch.optim.RAdam),
             (O.Adagrad, O.AdagradConfig, torch.optim.Adagrad), (O.Adadelta, O.AdadeltaConfig, torch.optim.Adadelta), (O.Rmsprop, O.RmspropConfig, torch.optim.RMSprop),
             (O.Rprop, O.RpropConfig, torch.optim.Rprop), (O.Asgd, O.AsgdConfig, torch.optim.ASGD)]
    for ours, cfg, ref in pairs:
        c = cfg().with_lr(0.05)
        assert c.lr == 0.05 and cfg().lr != 0.05 or cfg().lr == 0.05
        import dataclasses
        # own implementations of the update rules: the same numbers up to the rounding of a different operation order
        assert torch.allclose(run(lambda ps: ours(ps, c)), run(lambda ps: ref(ps, **dataclasses.asdict(c))), rtol=0, atol=1e-6), ours.__name__
    assert O.RmspropConfig().with_centered(True).with_momentum(0.5).centered and O.NAdamConfig().momentum_decay == 4e-3 and O.AsgdConfig().t0 == 1e6
    assert torch.allclose(run(lambda ps: O.Adamax(ps, lr=0.01)), run(lambda ps: torch.optim.Adamax(ps, lr=0.01)), rtol=0, atol=1e-6)
    lb = O.Lbfgs([torch.nn.Parameter(w0.clone())], O.LbfgsConfig(line_search_fn="strong_wolfe", history_size=5))
    assert lb.param_groups[0]["history_size"] == 5 and lb.param_groups[0]["line_search_fn"] == "strong_wolfe"

    # Adafactor under the reference's relative-step rule: first step moves every entry by about t^-0.5 * max(rms, eps_rms) in the gradient's sign
    p = torch.nn.Parameter(w0.clone())
    opt = O.Adafactor([p], O.AdafactorConfig())
    (p * torch.ones_like(p)).sum().backward()
    opt.step()
    rms = float(w0.norm() / w0.numel() ** 0.5)
    assert torch.allclose(w0 - p.detach(), torch.full_like(w0, rms), rtol=1e-3)
    small = w0 * 1e-3                                         # small weights, so that a 1e-6-relative step survives f32 rounding
    p2 = torch.nn.Parameter(small.clone())
    opt2 = O.Adafactor([p2], O.AdafactorConfig(warmup_init=True))
    (p2 * torch.ones_like(p2)).sum().backward()
    opt2.step()
    assert torch.allclose(small - p2.detach(), torch.full_like(w0, 1e-6 * max(rms * 1e-3, 1e-3)), rtol=0.1, atol=0)
    fixed = O.AdafactorConfig(lr=0.1, relative_step=False)
    p3 = torch.nn.Parameter(w0.clone())
    o3 = O.Adafactor([p3], fixed)
    (p3 * torch.ones_like(p3)).sum().backward()
    o3.step()
    assert torch.allclose(w0 - p3.detach(), torch.full_like(w0, 0.1), rtol=1e-3)

    # K-FAC config: momentum on the preconditioned step, L2 decay, maximize
    def kfac(cfg):
        torch.manual_seed(1)
        net = torch.nn.Sequential(torch.nn.Linear(4, 3))
        opt = O.Kfac(net, cfg)
        x, y = torch.randn(16, 4), torch.randn(16, 3)
        losses = []
        for _ in range(6):
            opt.zero_grad()
            l = (net(x) - y).pow(2).mean()
            l.backward()
            opt.step()
            losses.append(float(l))
        return losses, net
    base, _ = kfac(O.KfacConfig(lr=0.05, momentum=0.0, update_freq=1))
    assert base[-1] < base[0]
    mom, _ = kfac(O.KfacConfig(lr=0.05, momentum=0.5, update_freq=1))
    assert mom[-1] < mom[0] and mom[2] != base[2]
    up, _ = kfac(O.KfacConfig(lr=0.05, momentum=0.0, update_freq=1, maximize=True))
    assert up[-1] > up[0]
    _, heavy = kfac(O.KfacConfig(lr=0.05, momentum=0.0, update_freq=1, weight_decay=5.0))
    _, light = kfac(O.KfacConfig(lr=0.05, momentum=0.0, update_freq=1))
    assert heavy[0].weight.norm() < light[0].weight.norm()

    k = O.ParamKey(2, 7)
    assert str(k) == "g2_p7" and O.ParamKey.parse("g2_p7") == k and O.ParamKey(0, 9) < O.ParamKey(1, 0)
    with pytest.raises(InvalidArgument):
        O.ParamKey.parse("p7")

    net = torch.nn.Linear(2, 2)
    ema = O.AveragedModel(net, O.AveragingStrategy.Ema(0.9))
    swa = O.AveragedModel(net, O.AveragingStrategy.Swa)
    w_first = net.weight.detach().clone()
    ema.update_parameters(net); swa.update_parameters(net)          # noqa: E702
    with torch.no_grad():
        net.weight.add_(1.0)
    ema.update_parameters(net); swa.update_parameters(net)          # noqa: E702
    assert torch.allclose(ema.module.weight, 0.9 * w_first + 0.1 * (w_first + 1)) and torch.allclose(swa.module.weight, w_first + 0.5)
    assert O.AveragingStrategy.Ema(0.9) == O.AveragingStrategy.Ema(0.9) != O.AveragingStrategy.Swa
    with pytest.raises(InvalidArgument):
        O.AveragingStrategy.Ema(1.5)


def test_data_crate_names():
    from ferrotorch_b200 import data as D
    idx = list(range(20))
    D.shuffle_with_seed(idx, 1234)
    again = list(range(20))
    D.shuffle_with_seed(again, 1234)
    assert idx == again and sorted(idx) == list(range(20)) and idx != list(range(20))
    other = list(range(20))
    D.shuffle_with_seed(other, 1235)
    assert other != idx
    zero = list(range(8)); dead = list(range(8))               # noqa: E702
    D.shuffle_with_seed(zero, 0); D.shuffle_with_seed(dead, 0xDEADBEEFCAFE)          # noqa: E702
    assert zero == dead                                         # seed 0 is replaced, xorshift cannot leave state 0
    # first swap by hand: i = 3 of 4 elements, j = high word of xorshift(seed) * 4
    x = 99
    x ^= (x << 13) & (2 ** 64 - 1); x ^= x >> 7; x ^= (x << 17) & (2 ** 64 - 1)      # noqa: E702
    four = [0, 1, 2, 3]
    D.shuffle_with_seed(four, 99)
    assert four.index(3) == (x * 4) >> 64 or four[3] == [0, 1, 2, 3][(x * 4) >> 64]
    counts = [0] * 3
    for s in range(1, 3001):
        t = [0, 1, 2]
        D.shuffle_with_seed(t, s * 0x9E3779B97F4A7C15 % 2 ** 64)
        counts[t[0]] += 1
    assert all(abs(c / 3000 - 1 / 3) < 0.03 for c in counts)

    xs, ys = D.default_collate_pair([(torch.ones(2), torch.tensor(1)), (torch.zeros(2), torch.tensor(0))])
    assert xs.shape == (2, 2) and ys.tolist() == [1, 0]
    with pytest.raises(InvalidArgument):
        D.default_collate_pair([])
    it = D.BatchIter(D.VecDataset([10, 11, 12, 13, 14]), [[0, 1], [2, 3], [4]])
    assert list(it) == [[10, 11], [12, 13], [14]]

    img = torch.arange(2 * 6 * 6.0).view(2, 6, 6)
    D.manual_seed(5)
    a = [D.RandomCrop(4, 3)(img) for _ in range(4)]
    D.manual_seed(5)
    b = [D.RandomCrop(4, 3)(img) for _ in range(4)]
    assert all(torch.equal(p, q) for p, q in zip(a, b)) and a[0].shape == (2, 4, 3) and a[0].is_contiguous()
    assert torch.equal(D.RandomCrop(6)(img), img)
    with pytest.raises(InvalidArgument):
        D.RandomCrop(7, 2)(img)
    with pytest.raises(InvalidArgument):
        D.RandomCrop(1)(torch.zeros(3))
    assert torch.equal(D.RandomHorizontalFlip(1.0)(img), img.flip(-1)) and D.RandomHorizontalFlip(0.0)(img) is img
    D.manual_seed(0)
    flips = sum(not torch.equal(D.RandomHorizontalFlip(0.5).apply(img), img) for _ in range(400))
    assert 150 < flips < 250
    with pytest.raises(InvalidArgument):
        D.RandomHorizontalFlip(0.5)(torch.tensor(1.0))
    hwc = (torch.arange(4 * 5 * 3) % 256).to(torch.uint8).view(4, 5, 3).numpy()
    t = D.ToTensor()(hwc)
    assert t.shape == (3, 4, 5) and torch.allclose(t[1, 2, 3], torch.tensor(float(hwc[2, 3, 1]) / 255)) and D.ToTensor()(img) is img
    pipe = D.Compose([D.ToTensor(), D.RandomCrop(2), D.RandomHorizontalFlip(0.5)])
    assert isinstance(D.RandomCrop(2), D.Transform) and pipe.apply(hwc).shape == (3, 2, 2)


def test_hub_discovery_is_parsed_and_offline_is_loud(monkeypatch):
    from ferrotorch_b200 import hub as H
    q = H.SearchQuery().with_search("llama 3/é").with_pipeline_tag("text-generation").with_library("transformers").with_limit(5).with_sort("downloads")
    assert q.to_query_string() == "/api/models?search=llama%203%2F%C3%A9&pipeline_tag=text-generation&library=transformers&limit=5&sort=downloads"
    assert H.SearchQuery().to_query_string() == "/api/models"
    seen = []
    rows = [{"modelId": "meta-llama/Meta-Llama-3-8B", "downloads": 10, "likes": 2, "tags": ["llama"], "pipeline_tag": "text-generation"},
            {"id": "gpt2", "author": "openai-community"}]

    def fake(url, timeout=30.0):
        seen.append(url)
        return rows if "?" in url or url.endswith("/api/models") else {"id": "a/b", "siblings": [{"rfilename": "config.json"}, {"rfilename": "model.safetensors"}]}
    monkeypatch.setattr(H, "_http_get_json", fake)
    out = H.search_models(q)
    assert seen[0].startswith("https://huggingface.co/api/models?search=") and [r.model_id for r in out] == ["meta-llama/Meta-Llama-3-8B", "gpt2"]
    assert out[0].author == "meta-llama" and out[0].downloads == 10 and out[1].author == "openai-community" and out[1].tags == []
    info = H.get_model("a/b")
    assert seen[-1] == "https://huggingface.co/api/models/a/b" and info.filenames() == ["config.json", "model.safetensors"] and info.author == "a"
    with pytest.raises(InvalidArgument):
        H.get_model("")
    monkeypatch.setattr(H, "_http_get_json", lambda url, timeout=30.0: {"oops": 1})
    with pytest.raises(InvalidArgument):
        H.search_models(H.SearchQuery())
    monkeypatch.undo()
    monkeypatch.setenv("FT_HUB_OFFLINE", "1")
    with pytest.raises(H.HubOffline):
        H.search_models(H.SearchQuery().with_search("x"))
    assert [m.name for m in H.search_models("minilm")] == ["all-MiniLM-L6-v2"]          # the string form stays local
    assert H.get_model_info("resnet50").params == 25_557_032 and H.get_model_info("nope") is None
    assert H.get_model_info("resnet50").weights_format is H.WeightsFormat.SafeTensors and H.get_model_info("resnet50").kind is H.EntryKind.Model
    monkeypatch.setenv("HF_TOKEN", "tok123")
    import urllib.request
    assert H.with_auth(urllib.request.Request("https://huggingface.co/x")).get_header("Authorization") == "Bearer tok123"
    monkeypatch.setenv("FT_HUB_CACHE", "/tmp/some-cache")
    assert str(H.default_cache_dir()) == "/tmp/some-cache"


def test_train_profiler_grammar_nn_small_names():
    from ferrotorch_b200 import train as T, profiler as P, grammar as G, nn, optim as O
    net = torch.nn.Linear(3, 1)
    lr = T.Learner(net, O.Sgd(net.parameters(), lr=0.1), torch.nn.functional.mse_loss).with_metric(T.LossMetric())
    data = [(torch.randn(4, 3), torch.randn(4, 1)) for _ in range(3)]
    r = lr.evaluate(data)
    loss, metrics = r
    assert isinstance(r, T.EvalResult) and r.loss == loss and r.metrics is metrics and str(r).startswith(f"eval_loss={loss:.6f}")
    assert T.EvalResult.new_with_defaults(0.5).metrics == {} and T.checkpoint is not None and T.clip_grad_norm_ is nn.clip_grad_norm_

    s = P.ProfileSchedule(wait=1, warmup=2, active=2, repeat=2)
    assert [str(s.phase(i)) for i in range(11)] == ["Waiting", "Warmup", "Warmup", "Active", "Active"] * 2 + ["Done"]
    assert s.phase() is P.SchedulePhase.Waiting

    pv = G.PackedVocab.pack(["a", "true", "", "né"])
    assert pv.offsets == [0, 1, 5, 5, 7] and pv.max_token_len == 4 and pv.vocab_size() == 4 and pv.token(3) == "né" and pv.token(2) == ""
    off, ch = pv.tensors()
    assert off.dtype == torch.int32 and ch.tolist()[1:5] == [ord(c) for c in "true"] and "7 entries" in repr(pv)
    with pytest.raises(G.GrammarError) as e:
        pv.token(9)
    assert e.value.kind == "invalid_token_id" and "9" in str(e.value)
    proc = G.JsonSchemaProcessor({"type": "boolean"}, ["t", "rue", "x"], eos_id=None)
    with pytest.raises(G.GrammarError):
        proc.advance(17)
    B = G.BooleanEmissionStage
    assert B.of("") == (B.Start, "") and B.of("tr") == (B.PartialTrue, "ue") and B.of("fals") == (B.PartialFalse, "e") and B.of("true") == (B.Done, "") and B.of("tx") is None

    x = torch.linspace(-3, 3, 13)
    assert torch.allclose(nn.GELU(nn.GeluApproximate.Sigmoid)(x), x * torch.sigmoid(1.702 * x))
    assert torch.equal(nn.gelu(x, nn.GeluApproximate.Tanh), torch.nn.functional.gelu(x, approximate="tanh")) and torch.equal(nn.GELU()(x), torch.nn.functional.gelu(x))
    with pytest.raises(InvalidArgument):
        nn.gelu(x, "quick")
    img = torch.rand(1, 2, 4, 4)
    assert torch.equal(nn.interpolate(img, scale_factor=2, mode=nn.InterpolateMode.Nearest), torch.nn.functional.interpolate(img, scale_factor=2))
    grid = torch.rand(1, 3, 3, 2) * 2 - 1
    assert torch.equal(nn.grid_sample(img, grid, nn.GridSampleMode.Nearest, nn.GridSamplePaddingMode.Border),
                       torch.nn.functional.grid_sample(img, grid, mode="nearest", padding_mode="border", align_corners=False))
    assert nn.max_pool2d(img, 2).shape == (1, 2, 2, 2) and nn.adaptive_avg_pool2d(img, 1).shape == (1, 2, 1, 1) and nn.pixel_unshuffle(img, 2).shape == (1, 8, 2, 2)
    assert nn.QatModel is nn.QuantizedModel
    table = torch.arange(7.0)                                   # max_dist 3
    q, k = torch.randn(1, 1, 5, 4), torch.randn(1, 1, 5, 4)
    v = torch.randn(1, 1, 5, 4)
    got = nn.flex_attention(q, k, v, nn.relative_position_bias_score_mod(table, 3))
    qi, ki = torch.arange(5)[:, None], torch.arange(5)[None]
    bias = table[(qi - ki).clamp(-3, 3) + 3]
    want = torch.softmax(q @ k.transpose(-1, -2) / 2.0 + bias, -1) @ v
    assert torch.allclose(got, want, atol=1e-5)


def test_umbrella_package_surface():
    """Top level: sub-packages resolve lazily, the core names are reachable directly, the prelude carries the usual starting set, and the
    backends this framework does not have answer 'unavailable' instead of failing to import (ferrotorch/src/lib.rs:41-150)."""
    import ferrotorch_b200 as F
    from ferrotorch_b200 import prelude
    from ferrotorch_b200.errors import DeviceUnavailable
    assert F.zeros(2, 3).shape == (2, 3) and F.normalize_axis(-1, 2) == 1 and F.DispatchKeySet.empty().is_empty()
    for name in ("Linear", "Conv2d", "BatchNorm2d", "LayerNorm", "Dropout", "Module", "Parameter", "Sequential", "CrossEntropyLoss", "MSELoss", "GELU", "ReLU", "SiLU",
                 "Sigmoid", "Softmax", "Tanh", "GRU", "LSTM", "Adam", "AdamW", "Optimizer", "Sgd", "zeros", "Device", "no_grad"):
        assert hasattr(prelude, name), name
    assert callable(F.jit_script.script) and F.cubecl.GgufBlockKind.Q8_0.block_bytes() == 34 and callable(F.gpu.gpu_softmax)
    assert not F.mps.is_available() and not F.mps.is_mps_available() and F.mps.MpsDevice.count() == 0 and not F.xpu.is_available()
    for ctor in (F.mps.MtlBackend, F.mps.MpsDevice, F.xpu.XpuDevice, F.xpu.make_xpu_tensor):
        with pytest.raises(DeviceUnavailable):
            ctor()
    with pytest.raises(AttributeError):
        F.no_such_thing
