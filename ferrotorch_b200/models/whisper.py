"""Whisper audio encoder with the log-mel frontend (HF parameter names under ``model.encoder.*``).

Reference parity: ferrotorch-whisper/src/{config.rs:24, audio.rs:174 (log_mel_spectrogram), conv_stem.rs:34, encoder.rs:143,
encoder_layer.rs:19, loader.rs:31}.
"""
from __future__ import annotations

import json
import math
import os
from dataclasses import dataclass
from typing import Dict, Optional

import torch
import torch.nn.functional as F

from .. import nn
from ..nn.functional import scaled_dot_product_attention as sdpa
from ..errors import InvalidArgument, ShapeMismatch
from .bert import DropReport

SAMPLE_RATE, N_FFT, HOP_LENGTH, CHUNK_SECONDS = 16000, 400, 160, 30
# ferrotorch-whisper/src/audio.rs:34-49
CHUNK_LENGTH, N_MELS, N_FRAMES, N_SAMPLES, N_FREQS = CHUNK_SECONDS, 80, 3000, CHUNK_SECONDS * SAMPLE_RATE, N_FFT // 2 + 1


@dataclass
class WhisperConfig:
    num_mel_bins: int = 80
    d_model: int = 384
    encoder_layers: int = 4
    encoder_attention_heads: int = 6
    encoder_ffn_dim: int = 1536
    max_source_positions: int = 1500

    @classmethod
    def tiny(cls): return cls()
    @classmethod
    def base(cls): return cls(d_model=512, encoder_layers=6, encoder_attention_heads=8, encoder_ffn_dim=2048)
    @classmethod
    def small(cls): return cls(d_model=768, encoder_layers=12, encoder_attention_heads=12, encoder_ffn_dim=3072)
    whisper_tiny = tiny                                  # ferrotorch-whisper/src/config.rs:52

    @classmethod
    def from_hf(cls, d):
        if isinstance(d, HfWhisperConfig):
            d.validate()
            d = d.__dict__
        c = cls(**{k: d[k] for k in cls.__dataclass_fields__ if k in d})
        c.validate()
        return c

    def encoder_head_dim(self) -> int:
        return self.d_model // self.encoder_attention_heads

    def validate(self) -> None:
        """ferrotorch-whisper/src/config.rs:104-129."""
        if min(self.num_mel_bins, self.d_model, self.encoder_layers, self.encoder_attention_heads, self.encoder_ffn_dim, self.max_source_positions) <= 0:
            raise InvalidArgument("WhisperConfig: num_mel_bins / d_model / encoder_layers / encoder_attention_heads / encoder_ffn_dim / "
                                  "max_source_positions must all be positive")
        if self.d_model % self.encoder_attention_heads:
            raise InvalidArgument(f"WhisperConfig: d_model ({self.d_model}) must be divisible by encoder_attention_heads ({self.encoder_attention_heads})")


@dataclass
class HfWhisperConfig:
    """The fields of a Hugging Face Whisper ``config.json`` (ferrotorch-whisper/src/config.rs:137-236); the decoder sizes are carried but only
    the encoder is built here."""
    vocab_size: int
    num_mel_bins: int
    d_model: int
    encoder_layers: int
    encoder_attention_heads: int
    encoder_ffn_dim: int
    decoder_layers: int
    decoder_attention_heads: int
    decoder_ffn_dim: int
    max_source_positions: int
    max_target_positions: int
    activation_function: str = "gelu"
    architectures: tuple = ()
    model_type: Optional[str] = None

    @classmethod
    def from_json_str(cls, s: str) -> "HfWhisperConfig":
        try:
            d = json.loads(s)
            return cls(**{k: (tuple(d[k]) if k == "architectures" else d[k]) for k in cls.__dataclass_fields__ if k in d})
        except (ValueError, TypeError) as e:
            raise InvalidArgument(f"failed to parse Whisper config JSON: {e}") from None

    @classmethod
    def from_file(cls, path) -> "HfWhisperConfig":
        try:
            text = open(path, "rb").read().decode("utf-8")
        except (OSError, UnicodeDecodeError) as e:
            raise InvalidArgument(f"failed to read config file {path}: {e}") from None
        return cls.from_json_str(text)

    def validate(self) -> None:
        if min(self.vocab_size, self.num_mel_bins, self.d_model, self.encoder_layers, self.encoder_attention_heads, self.encoder_ffn_dim,
               self.max_source_positions) <= 0:
            raise InvalidArgument("HfWhisperConfig: sizes must all be positive")
        if self.d_model % self.encoder_attention_heads:
            raise InvalidArgument(f"HfWhisperConfig: d_model ({self.d_model}) must be divisible by encoder_attention_heads ({self.encoder_attention_heads})")
        if self.activation_function != "gelu":
            raise InvalidArgument(f"HfWhisperConfig: unsupported activation_function {self.activation_function!r}")


def _hz_to_mel(f):
    f = torch.as_tensor(f, dtype=torch.float64)
    lin = f / (200.0 / 3)
    log = 15.0 + torch.log(f.clamp_min(1e-10) / 1000.0) / (math.log(6.4) / 27.0)
    return torch.where(f >= 1000.0, log, lin)


def _mel_to_hz(m):
    lin = m * (200.0 / 3)
    log = 1000.0 * torch.exp((math.log(6.4) / 27.0) * (m - 15.0))
    return torch.where(m >= 15.0, log, lin)


def mel_filterbank(n_mels: int = 80, n_fft: int = N_FFT, sr: int = SAMPLE_RATE) -> torch.Tensor:
    """Slaney-scale, area-normalised triangular filters ``[n_mels, n_fft//2 + 1]`` (librosa.filters.mel defaults)."""
    freqs = torch.linspace(0, sr / 2, n_fft // 2 + 1, dtype=torch.float64)
    pts = _mel_to_hz(torch.linspace(float(_hz_to_mel(0.0)), float(_hz_to_mel(sr / 2)), n_mels + 2, dtype=torch.float64))
    d = pts[1:] - pts[:-1]
    ramps = pts[:, None] - freqs[None]
    lower, upper = -ramps[:-2] / d[:-1, None], ramps[2:] / d[1:, None]
    fb = torch.clamp_min(torch.minimum(lower, upper), 0)
    return (fb * (2.0 / (pts[2:] - pts[:-2]))[:, None]).float()


def log_mel_spectrogram(audio: torch.Tensor, n_mels: int = 80, pad_to_chunk: bool = True) -> torch.Tensor:
    """``[T]`` or ``[B, T]`` 16 kHz waveform -> ``[B, n_mels, frames]`` log-mel features (Hann STFT 400/160, log10, clamp to max-8,
    (x+4)/4), padded/trimmed to 30 s (3000 frames) when ``pad_to_chunk``."""
    if audio.dim() == 1:
        audio = audio[None]
    if pad_to_chunk:
        n = SAMPLE_RATE * CHUNK_SECONDS
        audio = F.pad(audio, (0, max(0, n - audio.shape[-1])))[..., :n]
    win = torch.hann_window(N_FFT, device=audio.device)
    st = torch.stft(audio.float(), N_FFT, HOP_LENGTH, window=win, return_complex=True)
    mag = st[..., :-1].abs() ** 2
    mel = mel_filterbank(n_mels).to(audio.device) @ mag
    lg = torch.clamp_min(mel, 1e-10).log10()
    lg = torch.maximum(lg, lg.amax(dim=(-2, -1), keepdim=True) - 8.0)
    return (lg + 4.0) / 4.0


def sinusoids(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2))
    t = torch.arange(length)[:, None] * inv[None]
    return torch.cat([t.sin(), t.cos()], 1)


class WhisperConvStem(nn.Module):
    def __init__(self, c: WhisperConfig):
        super().__init__()
        self.conv1 = nn.Conv1d(c.num_mel_bins, c.d_model, 3, padding=1)
        self.conv2 = nn.Conv1d(c.d_model, c.d_model, 3, stride=2, padding=1)

    def forward(self, mel):
        return F.gelu(self.conv2(F.gelu(self.conv1(mel)))).transpose(1, 2)


class WhisperEncoderSelfAttention(nn.Module):
    """Bidirectional self-attention with Whisper's bias-free key projection (ferrotorch-whisper/src/attention.rs:37)."""

    def __init__(self, c):
        super().__init__()
        self.h = c.encoder_attention_heads
        self.q_proj, self.v_proj, self.out_proj = nn.Linear(c.d_model, c.d_model), nn.Linear(c.d_model, c.d_model), nn.Linear(c.d_model, c.d_model)
        self.k_proj = nn.Linear(c.d_model, c.d_model, bias=False)

    def forward(self, x):
        B, S, E = x.shape
        sp = lambda t: t.view(B, S, self.h, E // self.h).transpose(1, 2)
        o = sdpa(sp(self.q_proj(x)), sp(self.k_proj(x)), sp(self.v_proj(x)))
        return self.out_proj(o.transpose(1, 2).reshape(B, S, E))


class WhisperEncoderLayer(nn.Module):
    def __init__(self, c: WhisperConfig):
        super().__init__()
        self.self_attn = WhisperEncoderSelfAttention(c)
        self.self_attn_layer_norm, self.final_layer_norm = nn.LayerNorm(c.d_model), nn.LayerNorm(c.d_model)
        self.fc1, self.fc2 = nn.Linear(c.d_model, c.encoder_ffn_dim), nn.Linear(c.encoder_ffn_dim, c.d_model)

    def forward(self, x):
        x = x + self.self_attn(self.self_attn_layer_norm(x))
        return x + self.fc2(F.gelu(self.fc1(self.final_layer_norm(x))))


class WhisperEncoder(nn.Module):
    def __init__(self, c: WhisperConfig):
        super().__init__()
        self.config = c
        self.conv1 = nn.Conv1d(c.num_mel_bins, c.d_model, 3, padding=1)
        self.conv2 = nn.Conv1d(c.d_model, c.d_model, 3, stride=2, padding=1)
        self.embed_positions = nn.Embedding(c.max_source_positions, c.d_model)
        with torch.no_grad():
            self.embed_positions.weight.copy_(sinusoids(c.max_source_positions, c.d_model))
        self.layers = nn.ModuleList([WhisperEncoderLayer(c) for _ in range(c.encoder_layers)])
        self.layer_norm = nn.LayerNorm(c.d_model)

    def forward(self, mel):
        x = F.gelu(self.conv2(F.gelu(self.conv1(mel)))).transpose(1, 2)
        x = x + self.embed_positions.weight[: x.shape[1]]
        for l in self.layers:
            x = l(x)
        return self.layer_norm(x)

    forward_from_mel = forward

    def load_hf_state_dict(self, hf_state: Dict[str, torch.Tensor], strict: bool = True) -> DropReport:
        """Takes the ``encoder.*`` / ``model.encoder.*`` keys of a Hugging Face checkpoint; every other key (decoder, ``proj_out``) is refused
        under ``strict`` and otherwise listed in the report (ferrotorch-whisper/src/encoder.rs:257-290)."""
        own, keep, dropped = self.state_dict(), {}, []
        for k, v in hf_state.items():
            rest = k[8:] if k.startswith("encoder.") else (k[14:] if k.startswith("model.encoder.") else None)
            if rest is None:
                if strict:
                    raise InvalidArgument(f"WhisperEncoder.load_hf_state_dict: key {k!r} is not under `encoder.*` or `model.encoder.*`; "
                                          "pass strict=False to drop decoder / proj_out keys")
                dropped.append(k)
            elif rest in own:
                if tuple(v.shape) != tuple(own[rest].shape):
                    raise ShapeMismatch(f"{rest}: checkpoint {tuple(v.shape)} vs model {tuple(own[rest].shape)}")
                keep[rest] = v
            elif strict:
                raise InvalidArgument(f'unexpected key in WhisperEncoder state_dict: "{rest}"')
        if strict and len(keep) != len(own):
            raise InvalidArgument(f"WhisperEncoder.load_hf_state_dict: missing keys {[k for k in own if k not in keep][:4]}")
        self.load_state_dict(keep, strict=False)
        return DropReport(dropped=tuple(sorted(dropped)))


def load_whisper_encoder(path: str, cfg: Optional[WhisperConfig] = None, strict: bool = False, device="cpu", dtype=torch.float32):
    """``load_whisper_encoder(directory)`` reads ``config.json`` + ``model.safetensors`` and returns the encoder;
    ``load_whisper_encoder(weights_file, cfg, strict)`` is the reference's form and also returns the :class:`DropReport`
    (ferrotorch-whisper/src/safetensors_loader.rs:31)."""
    from ..serialize import load_safetensors
    if cfg is None:
        cfg = WhisperConfig.from_hf(json.load(open(os.path.join(path, "config.json"))))
        m = WhisperEncoder(cfg)
        m.load_hf_state_dict(load_safetensors(os.path.join(path, "model.safetensors")), strict=False)
        return m.to(device=device, dtype=dtype)
    m = WhisperEncoder(cfg)
    report = m.load_hf_state_dict(load_safetensors(str(path)), strict=strict)
    return m.to(device=device, dtype=dtype), report
