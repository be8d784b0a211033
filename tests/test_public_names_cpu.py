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
