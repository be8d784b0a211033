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
