"""Stable-Diffusion-1.5 family: CLIP text encoder, UNet2DConditionModel, VAE encoder/decoder, DDIM scheduler and the text-to-image
pipeline, with diffusers / transformers parameter names so published safetensors load by name.

Reference parity: ferrotorch-diffusion/src/{attention.rs:59,442,645, blocks.rs:38-996, clip.rs:1009, scheduler.rs:109,
embeddings.rs:38,206, unet.rs:1117, vae.rs:261,295, pipeline.rs:59, safetensors_loader.rs:159-412} and the gpu/ variants, which
here are the same modules placed on the device (bf16, channels-last; attention through the framework's fused attention).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import nn
from ..errors import InvalidArgument


# ----------------------------------------------------------------------------------------------------------------------
# embeddings
# ----------------------------------------------------------------------------------------------------------------------
class Timesteps(nn.Module):
    """Sinusoidal timestep features (flip_sin_to_cos=True, freq_shift=0 as in SD-1.5)."""

    def __init__(self, num_channels: int, flip_sin_to_cos: bool = True, freq_shift: float = 0.0, max_period: float = 10000.0):
        super().__init__()
        self.n, self.flip, self.shift, self.max_period = num_channels, flip_sin_to_cos, freq_shift, max_period

    def forward(self, t: torch.Tensor) -> torch.Tensor:
        half = self.n // 2
        e = torch.exp(-math.log(self.max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / (half - self.shift))
        a = t.float()[:, None] * e[None]
        emb = torch.cat([a.sin(), a.cos()], -1)
        if self.flip:
            emb = torch.cat([emb[:, half:], emb[:, :half]], -1)
        return emb


class TimestepEmbedding(nn.Module):
    def __init__(self, in_channels: int, time_embed_dim: int):
        super().__init__()
        self.linear_1, self.linear_2 = nn.Linear(in_channels, time_embed_dim), nn.Linear(time_embed_dim, time_embed_dim)

    def forward(self, x):
        return self.linear_2(F.silu(self.linear_1(x)))


# ----------------------------------------------------------------------------------------------------------------------
# attention blocks
# ----------------------------------------------------------------------------------------------------------------------
class Attention(nn.Module):
    """Multi-head (cross-)attention, diffusers naming: to_q / to_k / to_v / to_out.0."""

    def __init__(self, query_dim: int, cross_dim: Optional[int] = None, heads: int = 8, dim_head: int = 64, bias: bool = False, out_bias: bool = True):
        super().__init__()
        inner = heads * dim_head
        self.heads = heads
        self.to_q = nn.Linear(query_dim, inner, bias=bias)
        self.to_k = nn.Linear(cross_dim or query_dim, inner, bias=bias)
        self.to_v = nn.Linear(cross_dim or query_dim, inner, bias=bias)
        self.to_out = nn.ModuleList([nn.Linear(inner, query_dim, bias=out_bias), nn.Identity()])

    def forward(self, x, context=None):
        ctx = x if context is None else context
        B, S, _ = x.shape
        sp = lambda t: t.view(B, t.shape[1], self.heads, -1).transpose(1, 2)
        o = F.scaled_dot_product_attention(sp(self.to_q(x)), sp(self.to_k(ctx)), sp(self.to_v(ctx)))
        return self.to_out[0](o.transpose(1, 2).reshape(B, S, -1))


class _GEGLU(nn.Module):
    def __init__(self, din, dout):
        super().__init__()
        self.proj = nn.Linear(din, dout * 2)

    def forward(self, x):
        h, g = self.proj(x).chunk(2, -1)
        return h * F.gelu(g)


class FeedForward(nn.Module):
    def __init__(self, dim: int, mult: int = 4):
        super().__init__()
        self.net = nn.ModuleList([_GEGLU(dim, dim * mult), nn.Identity(), nn.Linear(dim * mult, dim)])

    def forward(self, x):
        return self.net[2](self.net[0](x))


class BasicTransformerBlock(nn.Module):
    def __init__(self, dim: int, heads: int, dim_head: int, cross_dim: Optional[int]):
        super().__init__()
        self.norm1, self.norm2, self.norm3 = nn.LayerNorm(dim), nn.LayerNorm(dim), nn.LayerNorm(dim)
        self.attn1 = Attention(dim, None, heads, dim_head)
        self.attn2 = Attention(dim, cross_dim, heads, dim_head)
        self.ff = FeedForward(dim)

    def forward(self, x, context=None):
        x = x + self.attn1(self.norm1(x))
        x = x + self.attn2(self.norm2(x), context)
        return x + self.ff(self.norm3(x))


class Transformer2DModel(nn.Module):
    def __init__(self, channels: int, heads: int, dim_head: int, cross_dim: Optional[int], depth: int = 1, groups: int = 32, linear_proj: bool = False):
        super().__init__()
        inner = heads * dim_head
        self.linear_proj = linear_proj
        self.norm = nn.GroupNorm(groups, channels, eps=1e-6)
        self.proj_in = nn.Linear(channels, inner) if linear_proj else nn.Conv2d(channels, inner, 1)
        self.transformer_blocks = nn.ModuleList([BasicTransformerBlock(inner, heads, dim_head, cross_dim) for _ in range(depth)])
        self.proj_out = nn.Linear(inner, channels) if linear_proj else nn.Conv2d(inner, channels, 1)

    def forward(self, x, context=None):
        B, C, H, W = x.shape
        res = x
        h = self.norm(x)
        if self.linear_proj:
            h = self.proj_in(h.permute(0, 2, 3, 1).reshape(B, H * W, C))
        else:
            h = self.proj_in(h).permute(0, 2, 3, 1).reshape(B, H * W, -1)
        for blk in self.transformer_blocks:
            h = blk(h, context)
        if self.linear_proj:
            h = self.proj_out(h).view(B, H, W, C).permute(0, 3, 1, 2)
        else:
            h = self.proj_out(h.view(B, H, W, -1).permute(0, 3, 1, 2))
        return h + res


# ----------------------------------------------------------------------------------------------------------------------
# residual / sampling blocks
# ----------------------------------------------------------------------------------------------------------------------
class ResnetBlock2D(nn.Module):
    def __init__(self, cin: int, cout: int, temb_channels: Optional[int] = 1280, groups: int = 32, eps: float = 1e-5):
        super().__init__()
        self.norm1, self.conv1 = nn.GroupNorm(groups, cin, eps=eps), nn.Conv2d(cin, cout, 3, padding=1)
        self.time_emb_proj = nn.Linear(temb_channels, cout) if temb_channels else None
        self.norm2, self.conv2 = nn.GroupNorm(groups, cout, eps=eps), nn.Conv2d(cout, cout, 3, padding=1)
        self.conv_shortcut = nn.Conv2d(cin, cout, 1) if cin != cout else None

    def forward(self, x, temb=None):
        h = self.conv1(F.silu(self.norm1(x)))
        if self.time_emb_proj is not None and temb is not None:
            h = h + self.time_emb_proj(F.silu(temb))[:, :, None, None]
        h = self.conv2(F.silu(self.norm2(h)))
        return (x if self.conv_shortcut is None else self.conv_shortcut(x)) + h


class Downsample2D(nn.Module):
    def __init__(self, ch: int, padding: int = 1):
        super().__init__()
        self.pad = padding
        self.conv = nn.Conv2d(ch, ch, 3, stride=2, padding=padding)

    def forward(self, x):
        if self.pad == 0:
            x = F.pad(x, (0, 1, 0, 1))
        return self.conv(x)


class Upsample2D(nn.Module):
    def __init__(self, ch: int):
        super().__init__()
        self.conv = nn.Conv2d(ch, ch, 3, padding=1)

    def forward(self, x):
        return self.conv(F.interpolate(x, scale_factor=2.0, mode="nearest"))


class CrossAttnDownBlock2D(nn.Module):
    def __init__(self, cin, cout, temb, layers, heads, cross_dim, add_down, attn: bool = True):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, temb) for i in range(layers)])
        self.attentions = nn.ModuleList([Transformer2DModel(cout, heads, cout // heads, cross_dim) for _ in range(layers)]) if attn else None
        self.downsamplers = nn.ModuleList([Downsample2D(cout)]) if add_down else None

    def forward(self, x, temb, ctx):
        outs = []
        for i, r in enumerate(self.resnets):
            x = r(x, temb)
            if self.attentions is not None:
                x = self.attentions[i](x, ctx)
            outs.append(x)
        if self.downsamplers is not None:
            x = self.downsamplers[0](x)
            outs.append(x)
        return x, outs


DownBlock2D = lambda cin, cout, temb, layers, add_down: CrossAttnDownBlock2D(cin, cout, temb, layers, 1, None, add_down, attn=False)  # noqa: E731


class CrossAttnUpBlock2D(nn.Module):
    def __init__(self, cin, cout, prev, temb, layers, heads, cross_dim, add_up, attn: bool = True):
        super().__init__()
        res = []
        for i in range(layers):
            skip = cin if i == layers - 1 else cout
            res.append(ResnetBlock2D((prev if i == 0 else cout) + skip, cout, temb))
        self.resnets = nn.ModuleList(res)
        self.attentions = nn.ModuleList([Transformer2DModel(cout, heads, cout // heads, cross_dim) for _ in range(layers)]) if attn else None
        self.upsamplers = nn.ModuleList([Upsample2D(cout)]) if add_up else None

    def forward(self, x, skips: List[torch.Tensor], temb, ctx):
        for i, r in enumerate(self.resnets):
            x = r(torch.cat([x, skips.pop()], 1), temb)
            if self.attentions is not None:
                x = self.attentions[i](x, ctx)
        if self.upsamplers is not None:
            x = self.upsamplers[0](x)
        return x


class UNetMidBlock2DCrossAttn(nn.Module):
    def __init__(self, ch, temb, heads, cross_dim):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(ch, ch, temb), ResnetBlock2D(ch, ch, temb)])
        self.attentions = nn.ModuleList([Transformer2DModel(ch, heads, ch // heads, cross_dim)])

    def forward(self, x, temb, ctx):
        return self.resnets[1](self.attentions[0](self.resnets[0](x, temb), ctx), temb)


@dataclass
class UNetConfig:
    in_channels: int = 4
    out_channels: int = 4
    block_out_channels: Tuple[int, ...] = (320, 640, 1280, 1280)
    layers_per_block: int = 2
    cross_attention_dim: int = 768
    attention_head_dim: int = 8            # SD-1.5: number of heads
    norm_num_groups: int = 32
    attn_levels: Tuple[bool, ...] = (True, True, True, False)

    @classmethod
    def sd15(cls): return cls()
    @classmethod
    def tiny(cls): return cls(block_out_channels=(32, 64), layers_per_block=1, cross_attention_dim=32, attention_head_dim=4, norm_num_groups=8, attn_levels=(True, False))


class UNet2DConditionModel(nn.Module):
    def __init__(self, c: UNetConfig = UNetConfig()):
        super().__init__()
        self.config = c
        ch = c.block_out_channels
        temb = ch[0] * 4
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        self.time_proj = Timesteps(ch[0])
        self.time_embedding = TimestepEmbedding(ch[0], temb)
        downs, cin = [], ch[0]
        for i, co in enumerate(ch):
            last = i == len(ch) - 1
            downs.append(CrossAttnDownBlock2D(cin, co, temb, c.layers_per_block, c.attention_head_dim, c.cross_attention_dim, not last, c.attn_levels[i]))
            cin = co
        self.down_blocks = nn.ModuleList(downs)
        self.mid_block = UNetMidBlock2DCrossAttn(ch[-1], temb, c.attention_head_dim, c.cross_attention_dim)
        ups, rev, prev = [], list(reversed(ch)), ch[-1]
        for i, co in enumerate(rev):
            cin_skip = rev[min(i + 1, len(ch) - 1)]
            ups.append(CrossAttnUpBlock2D(cin_skip, co, prev, temb, c.layers_per_block + 1, c.attention_head_dim, c.cross_attention_dim,
                                          i < len(ch) - 1, list(reversed(c.attn_levels))[i]))
            prev = co
        self.up_blocks = nn.ModuleList(ups)
        self.conv_norm_out = nn.GroupNorm(c.norm_num_groups, ch[0], eps=1e-5)
        self.conv_out = nn.Conv2d(ch[0], c.out_channels, 3, padding=1)
        if c.norm_num_groups != 32:
            for m in self.modules():
                if isinstance(m, nn.GroupNorm):
                    m.num_groups = c.norm_num_groups

    def forward(self, sample, timestep, encoder_hidden_states):
        t = timestep if torch.is_tensor(timestep) else torch.tensor([timestep], device=sample.device)
        t = t.reshape(-1).expand(sample.shape[0])
        temb = self.time_embedding(self.time_proj(t).to(sample.dtype))
        x = self.conv_in(sample)
        skips = [x]
        for blk in self.down_blocks:
            x, outs = blk(x, temb, encoder_hidden_states)
            skips += outs
        x = self.mid_block(x, temb, encoder_hidden_states)
        for blk in self.up_blocks:
            x = blk(x, skips, temb, encoder_hidden_states)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


# ----------------------------------------------------------------------------------------------------------------------
# VAE
# ----------------------------------------------------------------------------------------------------------------------
class _VaeAttention(nn.Module):
    def __init__(self, ch, groups=32):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, ch, eps=1e-6)
        self.to_q, self.to_k, self.to_v = nn.Linear(ch, ch), nn.Linear(ch, ch), nn.Linear(ch, ch)
        self.to_out = nn.ModuleList([nn.Linear(ch, ch), nn.Identity()])

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.group_norm(x).view(B, C, H * W).transpose(1, 2)
        o = F.scaled_dot_product_attention(self.to_q(h)[:, None], self.to_k(h)[:, None], self.to_v(h)[:, None])[:, 0]
        return x + self.to_out[0](o).transpose(1, 2).view(B, C, H, W)


class UNetMidBlock2D(nn.Module):
    def __init__(self, ch, groups=32):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(ch, ch, None, groups, 1e-6), ResnetBlock2D(ch, ch, None, groups, 1e-6)])
        self.attentions = nn.ModuleList([_VaeAttention(ch, groups)])

    def forward(self, x):
        return self.resnets[1](self.attentions[0](self.resnets[0](x)))


class _VaeDown(nn.Module):
    def __init__(self, cin, cout, layers, add_down, groups):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, None, groups, 1e-6) for i in range(layers)])
        self.downsamplers = nn.ModuleList([Downsample2D(cout, padding=0)]) if add_down else None

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        return self.downsamplers[0](x) if self.downsamplers is not None else x


class _VaeUp(nn.Module):
    def __init__(self, cin, cout, layers, add_up, groups):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, None, groups, 1e-6) for i in range(layers)])
        self.upsamplers = nn.ModuleList([Upsample2D(cout)]) if add_up else None

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        return self.upsamplers[0](x) if self.upsamplers is not None else x


@dataclass
class VaeConfig:
    in_channels: int = 3
    latent_channels: int = 4
    block_out_channels: Tuple[int, ...] = (128, 256, 512, 512)
    layers_per_block: int = 2
    norm_num_groups: int = 32
    scaling_factor: float = 0.18215

    @classmethod
    def tiny(cls): return cls(block_out_channels=(16, 32), layers_per_block=1, norm_num_groups=8)


class VaeEncoder(nn.Module):
    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        ch, g = c.block_out_channels, c.norm_num_groups
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        self.down_blocks = nn.ModuleList([_VaeDown(ch[max(i - 1, 0)], ch[i], c.layers_per_block, i < len(ch) - 1, g) for i in range(len(ch))])
        self.mid_block = UNetMidBlock2D(ch[-1], g)
        self.conv_norm_out = nn.GroupNorm(g, ch[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[-1], 2 * c.latent_channels, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class VaeDecoder(nn.Module):
    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        ch, g = list(reversed(c.block_out_channels)), c.norm_num_groups
        self.conv_in = nn.Conv2d(c.latent_channels, ch[0], 3, padding=1)
        self.mid_block = UNetMidBlock2D(ch[0], g)
        self.up_blocks = nn.ModuleList([_VaeUp(ch[max(i - 1, 0)], ch[i], c.layers_per_block + 1, i < len(ch) - 1, g) for i in range(len(ch))])
        self.conv_norm_out = nn.GroupNorm(g, ch[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[-1], c.in_channels, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class AutoencoderKL(nn.Module):
    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        self.config = c
        self.encoder, self.decoder = VaeEncoder(c), VaeDecoder(c)
        self.quant_conv = nn.Conv2d(2 * c.latent_channels, 2 * c.latent_channels, 1)
        self.post_quant_conv = nn.Conv2d(c.latent_channels, c.latent_channels, 1)

    def encode(self, x, sample: bool = True, generator=None):
        mean, logvar = self.quant_conv(self.encoder(x)).chunk(2, 1)
        if not sample:
            return mean
        return mean + (0.5 * logvar.clamp(-30, 20)).exp() * torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype)

    def decode(self, z):
        return self.decoder(self.post_quant_conv(z))


# ----------------------------------------------------------------------------------------------------------------------
# CLIP text encoder
# ----------------------------------------------------------------------------------------------------------------------
@dataclass
class ClipTextConfig:
    vocab_size: int = 49408
    hidden_size: int = 768
    intermediate_size: int = 3072
    num_hidden_layers: int = 12
    num_attention_heads: int = 12
    max_position_embeddings: int = 77
    layer_norm_eps: float = 1e-5

    @classmethod
    def tiny(cls): return cls(vocab_size=1000, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4)


class _ClipAttention(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.h = c.num_attention_heads
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(c.hidden_size, c.hidden_size) for _ in range(4))

    def forward(self, x):
        B, S, E = x.shape
        sp = lambda t: t.view(B, S, self.h, E // self.h).transpose(1, 2)
        o = F.scaled_dot_product_attention(sp(self.q_proj(x)), sp(self.k_proj(x)), sp(self.v_proj(x)), is_causal=True)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, E))


class _ClipMlp(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(c.hidden_size, c.intermediate_size), nn.Linear(c.intermediate_size, c.hidden_size)

    def forward(self, x):
        h = self.fc1(x)
        return self.fc2(h * torch.sigmoid(1.702 * h))               # quick_gelu


class _ClipLayer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.self_attn, self.mlp = _ClipAttention(c), _ClipMlp(c)
        self.layer_norm1, self.layer_norm2 = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps), nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)

    def forward(self, x):
        x = x + self.self_attn(self.layer_norm1(x))
        return x + self.mlp(self.layer_norm2(x))


class _ClipEmbeddings(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.token_embedding = nn.Embedding(c.vocab_size, c.hidden_size)
        self.position_embedding = nn.Embedding(c.max_position_embeddings, c.hidden_size)

    def forward(self, ids):
        return self.token_embedding(ids) + self.position_embedding.weight[: ids.shape[1]]


class _ClipEncoder(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.layers = nn.ModuleList([_ClipLayer(c) for _ in range(c.num_hidden_layers)])


class _ClipTextTransformer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.embeddings, self.encoder = _ClipEmbeddings(c), _ClipEncoder(c)
        self.final_layer_norm = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)

    def forward(self, ids):
        x = self.embeddings(ids)
        for l in self.encoder.layers:
            x = l(x)
        return self.final_layer_norm(x)


class ClipTextEncoder(nn.Module):
    """Parameter names follow ``transformers.CLIPTextModel`` (``text_model.*``); returns the last hidden state ``[B, 77, hidden]``."""

    def __init__(self, c: ClipTextConfig = ClipTextConfig()):
        super().__init__()
        self.config = c
        self.text_model = _ClipTextTransformer(c)

    def forward(self, ids):
        return self.text_model(ids)


# ----------------------------------------------------------------------------------------------------------------------
# scheduler + pipeline
# ----------------------------------------------------------------------------------------------------------------------
class DDIMScheduler:
    def __init__(self, num_train_timesteps: int = 1000, beta_start: float = 0.00085, beta_end: float = 0.012, beta_schedule: str = "scaled_linear",
                 set_alpha_to_one: bool = False, steps_offset: int = 1, prediction_type: str = "epsilon"):
        if beta_schedule == "scaled_linear":
            betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, num_train_timesteps, dtype=torch.float64) ** 2
        elif beta_schedule == "linear":
            betas = torch.linspace(beta_start, beta_end, num_train_timesteps, dtype=torch.float64)
        else:
            raise InvalidArgument(f"unknown beta schedule {beta_schedule}")
        self.alphas_cumprod = torch.cumprod(1.0 - betas, 0)
        self.final_alpha_cumprod = torch.tensor(1.0, dtype=torch.float64) if set_alpha_to_one else self.alphas_cumprod[0]
        self.num_train_timesteps, self.steps_offset, self.prediction_type = num_train_timesteps, steps_offset, prediction_type
        self.init_noise_sigma = 1.0
        self.timesteps: torch.Tensor = torch.arange(num_train_timesteps - 1, -1, -1)
        self.num_inference_steps = num_train_timesteps

    def set_timesteps(self, n: int) -> None:
        if n > self.num_train_timesteps:
            raise InvalidArgument("more inference steps than training steps")
        self.num_inference_steps = n
        ratio = self.num_train_timesteps // n
        self.timesteps = (torch.arange(n) * ratio).flip(0) + self.steps_offset

    def scale_model_input(self, x, t):
        return x

    def step(self, model_output: torch.Tensor, t: int, sample: torch.Tensor, eta: float = 0.0, generator=None) -> torch.Tensor:
        prev_t = int(t) - self.num_train_timesteps // self.num_inference_steps
        a_t = self.alphas_cumprod[int(t)]
        a_prev = self.alphas_cumprod[prev_t] if prev_t >= 0 else self.final_alpha_cumprod
        a_t, a_prev = float(a_t), float(a_prev)
        if self.prediction_type == "epsilon":
            x0 = (sample - (1 - a_t) ** 0.5 * model_output) / a_t ** 0.5
            eps = model_output
        elif self.prediction_type == "v_prediction":
            x0 = a_t ** 0.5 * sample - (1 - a_t) ** 0.5 * model_output
            eps = a_t ** 0.5 * model_output + (1 - a_t) ** 0.5 * sample
        else:
            x0, eps = model_output, (sample - a_t ** 0.5 * model_output) / (1 - a_t) ** 0.5
        var = (1 - a_prev) / (1 - a_t) * (1 - a_t / a_prev)
        sigma = eta * max(var, 0.0) ** 0.5
        prev = a_prev ** 0.5 * x0 + max(1 - a_prev - sigma ** 2, 0.0) ** 0.5 * eps
        if eta > 0:
            prev = prev + sigma * torch.randn(sample.shape, generator=generator, device=sample.device, dtype=sample.dtype)
        return prev

    def add_noise(self, x0, noise, t):
        a = self.alphas_cumprod.to(x0.device)[t].to(x0.dtype).view(-1, 1, 1, 1)
        return a.sqrt() * x0 + (1 - a).sqrt() * noise


class StableDiffusionPipeline:
    """Text-to-image: CLIP text states (cond + uncond) -> DDIM loop over the UNet with classifier-free guidance -> VAE decode."""

    def __init__(self, text_encoder: ClipTextEncoder, unet: UNet2DConditionModel, vae: AutoencoderKL, scheduler: Optional[DDIMScheduler] = None, tokenizer=None):
        self.text_encoder, self.unet, self.vae, self.scheduler, self.tokenizer = text_encoder, unet, vae, scheduler or DDIMScheduler(), tokenizer

    def to(self, *a, **k):
        for m in (self.text_encoder, self.unet, self.vae):
            m.to(*a, **k)
        return self

    def _ids(self, prompt):
        if torch.is_tensor(prompt):
            return prompt
        if self.tokenizer is None:
            raise InvalidArgument("a tokenizer is required for string prompts")
        ids = self.tokenizer.encode(prompt)
        L = self.text_encoder.config.max_position_embeddings
        ids = (ids + [ids[-1]] * L)[:L]
        return torch.tensor([ids])

    @torch.no_grad()
    def __call__(self, prompt, negative_prompt=None, height: int = 512, width: int = 512, num_inference_steps: int = 50, guidance_scale: float = 7.5,
                 generator=None, latents: Optional[torch.Tensor] = None, output_type: str = "tensor"):
        dev = next(self.unet.parameters()).device
        dt = next(self.unet.parameters()).dtype
        ids = self._ids(prompt).to(dev)
        cond = self.text_encoder(ids)
        cfg = guidance_scale > 1.0
        if cfg:
            neg = self._ids(negative_prompt).to(dev) if negative_prompt is not None else torch.zeros_like(ids)
            ctx = torch.cat([self.text_encoder(neg), cond], 0)
        else:
            ctx = cond
        B = ids.shape[0]
        shape = (B, self.unet.config.in_channels, height // 8, width // 8)
        if latents is None:
            latents = torch.randn(shape, generator=generator, dtype=torch.float32).to(dev, dt)
        latents = latents * self.scheduler.init_noise_sigma
        self.scheduler.set_timesteps(num_inference_steps)
        for t in self.scheduler.timesteps.tolist():
            inp = torch.cat([latents, latents], 0) if cfg else latents
            eps = self.unet(inp, torch.tensor([t], device=dev), ctx.to(dt))
            if cfg:
                eu, ec = eps.chunk(2, 0)
                eps = eu + guidance_scale * (ec - eu)
            latents = self.scheduler.step(eps, t, latents)
        img = self.vae.decode(latents / self.vae.config.scaling_factor)
        img = (img / 2 + 0.5).clamp(0, 1)
        if output_type == "uint8":
            return (img * 255).round().to(torch.uint8).permute(0, 2, 3, 1)
        return img


def load_sd_component(module: nn.Module, path: str, strict: bool = True) -> nn.Module:
    """Loads a diffusers-layout safetensors file (``unet/diffusion_pytorch_model.safetensors`` etc.) into the matching module by name."""
    from ..serialize import load_safetensors
    module.load_state_dict(load_safetensors(path), strict=strict)
    return module


# the reference's device variants are these same modules on the device
GpuUNet2DConditional, GpuVaeDecoder, GpuVaeEncoder, GpuClipTextEncoder, GpuStableDiffusionPipeline = (
    UNet2DConditionModel, VaeDecoder, VaeEncoder, ClipTextEncoder, StableDiffusionPipeline)
