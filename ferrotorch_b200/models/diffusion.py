"""Stable-Diffusion-1.5 family: CLIP text encoder, UNet2DConditionModel, VAE encoder/decoder, DDIM scheduler and the text-to-image
pipeline, with diffusers / transformers parameter names so published safetensors load by name.

Reference parity: ferrotorch-diffusion/src/{attention.rs:59,442,645, blocks.rs:38-996, clip.rs:1009, scheduler.rs:109,
embeddings.rs:38,206, unet.rs:1117, vae.rs:261,295, pipeline.rs:59, safetensors_loader.rs:159-412} and the gpu/ variants, which
here are the same modules placed on the device (bf16, channels-last; attention through the framework's fused attention).
"""
from __future__ import annotations

import enum
import json
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .. import nn
from ..nn.functional import scaled_dot_product_attention as sdpa
from ..errors import InvalidArgument, ShapeMismatch
from .bert import DropReport


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
        o = sdpa(sp(self.to_q(x)), sp(self.to_k(ctx)), sp(self.to_v(ctx)))
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


class ResnetBlock2DTime(ResnetBlock2D):
    """The UNet's residual block: the timestep embedding is required and added between the two convolutions
    (ferrotorch-diffusion/src/resnet_block_time.rs:35-107)."""

    def __init__(self, cin: int, cout: int, temb_channels: int = 1280, groups: int = 32, eps: float = 1e-5):
        if not temb_channels:
            raise InvalidArgument("ResnetBlock2DTime: temb_channels must be positive")
        super().__init__(cin, cout, temb_channels, groups, eps)

    def forward(self, x, temb):
        if temb is None or temb.dim() != 2 or temb.shape[1] != self.time_emb_proj.in_features:
            raise ShapeMismatch(f"ResnetBlock2DTime: expected temb [B, {self.time_emb_proj.in_features}]")
        return super().forward(x, temb)

    forward_t = forward


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
    def __init__(self, cin, cout, temb, layers, heads, cross_dim, add_down, attn: bool = True, groups: int = 32, depth: int = 1):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, temb, groups) for i in range(layers)])
        self.attentions = nn.ModuleList([Transformer2DModel(cout, heads, cout // heads, cross_dim, depth, groups) for _ in range(layers)]) if attn else None
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


class DownBlock2D(CrossAttnDownBlock2D):
    """Resnets + optional downsample, no attention (ferrotorch-diffusion/src/unet.rs:277)."""

    def __init__(self, cin, cout, temb, layers, add_down, groups: int = 32):
        super().__init__(cin, cout, temb, layers, 1, None, add_down, attn=False, groups=groups)

    def forward(self, x, temb, ctx=None):
        return super().forward(x, temb, None)

    forward_t = forward


class CrossAttnUpBlock2D(nn.Module):
    def __init__(self, cin, cout, prev, temb, layers, heads, cross_dim, add_up, attn: bool = True, groups: int = 32, depth: int = 1):
        super().__init__()
        res = []
        for i in range(layers):
            skip = cin if i == layers - 1 else cout
            res.append(ResnetBlock2D((prev if i == 0 else cout) + skip, cout, temb, groups))
        self.resnets = nn.ModuleList(res)
        self.attentions = nn.ModuleList([Transformer2DModel(cout, heads, cout // heads, cross_dim, depth, groups) for _ in range(layers)]) if attn else None
        self.upsamplers = nn.ModuleList([Upsample2D(cout)]) if add_up else None

    def forward(self, x, skips: List[torch.Tensor], temb, ctx):
        for i, r in enumerate(self.resnets):
            x = r(torch.cat([x, skips.pop()], 1), temb)
            if self.attentions is not None:
                x = self.attentions[i](x, ctx)
        if self.upsamplers is not None:
            x = self.upsamplers[0](x)
        return x


class UpBlock2D(CrossAttnUpBlock2D):
    """Skip-concatenating resnets + optional upsample, no attention (ferrotorch-diffusion/src/unet.rs:839)."""

    def __init__(self, cin, cout, prev, temb, layers, add_up, groups: int = 32):
        super().__init__(cin, cout, prev, temb, layers, 1, None, add_up, attn=False, groups=groups)

    def forward(self, x, skips, temb, ctx=None):
        return super().forward(x, skips, temb, None)

    forward_t = forward


from typing import Union as _Union                                           # noqa: E402
AnyDownBlock = _Union[CrossAttnDownBlock2D, DownBlock2D]                     # ferrotorch-diffusion/src/unet.rs:1011, 1059: the two block kinds a
AnyUpBlock = _Union[CrossAttnUpBlock2D, UpBlock2D]                           # level of the UNet can hold


class UNetMidBlock2DCrossAttn(nn.Module):
    def __init__(self, ch, temb, heads, cross_dim, groups: int = 32, depth: int = 1):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(ch, ch, temb, groups), ResnetBlock2D(ch, ch, temb, groups)])
        self.attentions = nn.ModuleList([Transformer2DModel(ch, heads, ch // heads, cross_dim, depth, groups)])

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
    attn_levels: Tuple[bool, ...] = (True, True, True, False)      # which down blocks carry cross-attention (``down_block_has_attn``)
    up_attn_levels: Optional[Tuple[bool, ...]] = None              # ``up_block_has_attn``; default: the down list reversed
    sample_size: int = 64
    flip_sin_to_cos: bool = True
    freq_shift: float = 0.0
    transformer_layers_per_block: int = 1

    @classmethod
    def sd15(cls): return cls()

    sd_v1_5 = sd15                                                 # ferrotorch-diffusion/src/unet_config.rs:73

    @property
    def down_block_has_attn(self) -> Tuple[bool, ...]:
        return tuple(self.attn_levels)

    @property
    def up_block_has_attn(self) -> Tuple[bool, ...]:
        return tuple(self.up_attn_levels) if self.up_attn_levels is not None else tuple(reversed(self.attn_levels))

    def time_embed_dim(self) -> int:
        return self.block_out_channels[0] * 4

    def num_blocks(self) -> int:
        return len(self.block_out_channels)

    def validate(self) -> None:
        """ferrotorch-diffusion/src/unet_config.rs:83-140."""
        n = "UNet2DConditionConfig"
        if not self.block_out_channels:
            raise InvalidArgument(f"{n}: block_out_channels must be non-empty")
        if self.norm_num_groups <= 0:
            raise InvalidArgument(f"{n}: norm_num_groups must be > 0")
        if min(self.in_channels, self.out_channels, self.layers_per_block, self.cross_attention_dim, self.attention_head_dim, self.sample_size) <= 0:
            raise InvalidArgument(f"{n}: a positive-only field was zero")
        for c in self.block_out_channels:
            if c <= 0 or c % self.norm_num_groups:
                raise InvalidArgument(f"{n}: block_out_channels entry {c} must be > 0 and divisible by norm_num_groups={self.norm_num_groups}")
            if c % self.attention_head_dim:
                raise InvalidArgument(f"{n}: block_out_channels entry {c} must be divisible by attention_head_dim={self.attention_head_dim}")
        if len(self.down_block_has_attn) != len(self.block_out_channels) or len(self.up_block_has_attn) != len(self.block_out_channels):
            raise InvalidArgument(f"{n}: down/up_block_has_attn must have the same length as block_out_channels ({len(self.block_out_channels)} blocks), "
                                  f"got down={len(self.down_block_has_attn)} up={len(self.up_block_has_attn)}")

    @classmethod
    def from_json_str(cls, s: str) -> "UNetConfig":
        """A diffusers ``unet/config.json``: absent keys keep the SD-1.5 defaults, block types map to the has-attention lists
        (unet_config.rs:158-268)."""
        try:
            v = json.loads(s)
        except ValueError as e:
            raise InvalidArgument(f"UNet2DConditionConfig.from_json_str: bad JSON: {e}") from None
        kw = {}
        for k in ("in_channels", "out_channels", "layers_per_block", "attention_head_dim", "cross_attention_dim", "norm_num_groups", "sample_size",
                  "transformer_layers_per_block"):
            if isinstance(v.get(k), int) and not isinstance(v.get(k), bool):
                kw[k] = v[k]
        if isinstance(v.get("flip_sin_to_cos"), bool):
            kw["flip_sin_to_cos"] = v["flip_sin_to_cos"]
        if isinstance(v.get("freq_shift"), (int, float)) and not isinstance(v.get("freq_shift"), bool):
            kw["freq_shift"] = float(v["freq_shift"])
        if isinstance(v.get("block_out_channels"), list):
            if not all(isinstance(e, int) and not isinstance(e, bool) and e >= 0 for e in v["block_out_channels"]):
                raise InvalidArgument("UNet2DConditionConfig.from_json_str: block_out_channels entry must be a non-negative integer")
            kw["block_out_channels"] = tuple(v["block_out_channels"])
        for key, field_, names in (("down_block_types", "attn_levels", {"CrossAttnDownBlock2D": True, "DownBlock2D": False}),
                                   ("up_block_types", "up_attn_levels", {"CrossAttnUpBlock2D": True, "UpBlock2D": False})):
            if isinstance(v.get(key), list):
                out = []
                for e in v[key]:
                    if not isinstance(e, str):
                        raise InvalidArgument(f"UNet2DConditionConfig.from_json_str: {key} entry must be a string, got {e!r}")
                    if e not in names:
                        raise InvalidArgument(f"UNet2DConditionConfig.from_json_str: unsupported {key[:-1]} '{e}'. Only {' / '.join(names)} are recognised.")
                    out.append(names[e])
                kw[field_] = tuple(out)
        c = cls(**kw)
        c.validate()
        return c

    @classmethod
    def from_file(cls, path) -> "UNetConfig":
        try:
            text = open(path, encoding="utf-8").read()
        except (OSError, UnicodeDecodeError) as e:
            raise InvalidArgument(f"UNet2DConditionConfig.from_file: failed to read {path}: {e}") from None
        return cls.from_json_str(text)
    @classmethod
    def tiny(cls): return cls(block_out_channels=(32, 64), layers_per_block=1, cross_attention_dim=32, attention_head_dim=4, norm_num_groups=8, attn_levels=(True, False))


UNet2DConditionConfig = UNetConfig


class UNet2DConditionModel(nn.Module):
    def __init__(self, c: UNetConfig = UNetConfig()):
        super().__init__()
        c.validate()
        self.config = c
        ch = c.block_out_channels
        temb = ch[0] * 4
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        self.time_proj = Timesteps(ch[0], c.flip_sin_to_cos, c.freq_shift)
        self.time_embedding = TimestepEmbedding(ch[0], temb)
        downs, cin = [], ch[0]
        for i, co in enumerate(ch):
            last = i == len(ch) - 1
            downs.append(CrossAttnDownBlock2D(cin, co, temb, c.layers_per_block, c.attention_head_dim, c.cross_attention_dim, not last, c.attn_levels[i],
                                              c.norm_num_groups, c.transformer_layers_per_block))
            cin = co
        self.down_blocks = nn.ModuleList(downs)
        self.mid_block = UNetMidBlock2DCrossAttn(ch[-1], temb, c.attention_head_dim, c.cross_attention_dim, c.norm_num_groups, c.transformer_layers_per_block)
        ups, rev, prev = [], list(reversed(ch)), ch[-1]
        for i, co in enumerate(rev):
            cin_skip = rev[min(i + 1, len(ch) - 1)]
            ups.append(CrossAttnUpBlock2D(cin_skip, co, prev, temb, c.layers_per_block + 1, c.attention_head_dim, c.cross_attention_dim,
                                          i < len(ch) - 1, c.up_block_has_attn[i], c.norm_num_groups, c.transformer_layers_per_block))
            prev = co
        self.up_blocks = nn.ModuleList(ups)
        self.conv_norm_out = nn.GroupNorm(c.norm_num_groups, ch[0], eps=1e-5)
        self.conv_out = nn.Conv2d(ch[0], c.out_channels, 3, padding=1)

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

    forward_t = forward

    def load_hf_state_dict(self, hf_state: Dict[str, torch.Tensor], strict: bool = True) -> DropReport:
        """A diffusers UNet state dict, bare or under ``unet.`` (ferrotorch-diffusion/src/safetensors_loader.rs:58)."""
        return _load_prefixed(self, hf_state, {"unet.": ""}, None, strict, "UNet2DConditionModel")


def _load_prefixed(module: nn.Module, state: Dict[str, torch.Tensor], strip: Dict[str, str], known: Optional[Tuple[str, ...]], strict: bool, who: str,
                   always_drop: Tuple[str, ...] = ()) -> DropReport:
    """Shared body of the checkpoint loaders: strip an optional bundle prefix, keep the keys under ``known`` (all keys when ``None``), drop
    ``always_drop`` in both modes, refuse (``strict``) or list every other key, check shapes, and require every parameter under ``strict``."""
    own, keep, dropped = module.state_dict(), {}, []
    for k, v in state.items():
        name = k
        for pre, rep in strip.items():
            if name.startswith(pre):
                name = rep + name[len(pre):]
                break
        if name in always_drop:
            dropped.append(k)
        elif (known is None or name.startswith(known)) and name in own:
            if tuple(v.shape) != tuple(own[name].shape):
                raise ShapeMismatch(f"{who}: {name}: checkpoint {tuple(v.shape)} vs model {tuple(own[name].shape)}")
            keep[name] = v
        elif strict:
            raise InvalidArgument(f"{who}.load_hf_state_dict: key {k!r} does not belong to this module and strict mode is on; pass strict=False to drop it")
        else:
            dropped.append(k)
    if strict and len(keep) != len(own):
        raise InvalidArgument(f"{who}.load_hf_state_dict: missing keys {[k for k in own if k not in keep][:4]}")
    module.load_state_dict(keep, strict=False)
    return DropReport(dropped=tuple(sorted(dropped)))


# ----------------------------------------------------------------------------------------------------------------------
# VAE
# ----------------------------------------------------------------------------------------------------------------------
class AttnBlock2D(nn.Module):
    """Single-head spatial self-attention of the VAE mid block, residual included (ferrotorch-diffusion/src/blocks.rs:245)."""

    def __init__(self, ch, groups=32):
        super().__init__()
        self.group_norm = nn.GroupNorm(groups, ch, eps=1e-6)
        self.to_q, self.to_k, self.to_v = nn.Linear(ch, ch), nn.Linear(ch, ch), nn.Linear(ch, ch)
        self.to_out = nn.ModuleList([nn.Linear(ch, ch), nn.Identity()])

    def forward(self, x):
        B, C, H, W = x.shape
        h = self.group_norm(x).view(B, C, H * W).transpose(1, 2)
        o = sdpa(self.to_q(h)[:, None], self.to_k(h)[:, None], self.to_v(h)[:, None])[:, 0]
        return x + self.to_out[0](o).transpose(1, 2).view(B, C, H, W)


class UNetMidBlock2D(nn.Module):
    def __init__(self, ch, groups=32):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(ch, ch, None, groups, 1e-6), ResnetBlock2D(ch, ch, None, groups, 1e-6)])
        self.attentions = nn.ModuleList([AttnBlock2D(ch, groups)])

    def forward(self, x):
        return self.resnets[1](self.attentions[0](self.resnets[0](x)))


class DownEncoderBlock2D(nn.Module):
    """ferrotorch-diffusion/src/blocks.rs:813."""

    def __init__(self, cin, cout, layers, add_down, groups):
        super().__init__()
        self.resnets = nn.ModuleList([ResnetBlock2D(cin if i == 0 else cout, cout, None, groups, 1e-6) for i in range(layers)])
        self.downsamplers = nn.ModuleList([Downsample2D(cout, padding=0)]) if add_down else None

    def forward(self, x):
        for r in self.resnets:
            x = r(x)
        return self.downsamplers[0](x) if self.downsamplers is not None else x


class UpDecoderBlock2D(nn.Module):
    """ferrotorch-diffusion/src/blocks.rs:630."""

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
    sample_size: int = 512

    @classmethod
    def tiny(cls): return cls(block_out_channels=(16, 32), layers_per_block=1, norm_num_groups=8)

    @classmethod
    def sd_v1_5(cls): return cls()                                 # ferrotorch-diffusion/src/config.rs:59

    @property
    def out_channels(self) -> int:                                 # the reference names the image channels from the decoder's side
        return self.in_channels

    def resnets_per_up_block(self) -> int:
        return self.layers_per_block + 1

    def num_up_blocks(self) -> int:
        return len(self.block_out_channels)

    def validate(self) -> None:
        """ferrotorch-diffusion/src/config.rs:70-122."""
        n = "VaeDecoderConfig"
        if not self.block_out_channels:
            raise InvalidArgument(f"{n}: block_out_channels must be non-empty")
        if self.norm_num_groups <= 0:
            raise InvalidArgument(f"{n}: norm_num_groups must be > 0")
        for c in self.block_out_channels:
            if c <= 0 or c % self.norm_num_groups:
                raise InvalidArgument(f"{n}: block_out_channels entry {c} must be > 0 and divisible by norm_num_groups={self.norm_num_groups}")
        for f in ("latent_channels", "in_channels", "layers_per_block", "sample_size"):
            if getattr(self, f) <= 0:
                raise InvalidArgument(f"{n}: {'out_channels' if f == 'in_channels' else f} must be > 0")
        if not math.isfinite(self.scaling_factor) or self.scaling_factor == 0.0:
            raise InvalidArgument(f"{n}: scaling_factor must be finite and non-zero, got {self.scaling_factor}")

    @classmethod
    def from_json_str(cls, s: str) -> "VaeConfig":
        """A diffusers ``vae/config.json``; absent keys keep the SD-1.5 defaults (config.rs:148-193)."""
        try:
            v = json.loads(s)
        except ValueError as e:
            raise InvalidArgument(f"VaeDecoderConfig.from_json_str: bad JSON: {e}") from None
        kw = {}
        for src, dst in (("out_channels", "in_channels"), ("latent_channels",) * 2, ("layers_per_block",) * 2, ("norm_num_groups",) * 2, ("sample_size",) * 2):
            if isinstance(v.get(src), int) and not isinstance(v.get(src), bool):
                kw[dst] = v[src]
        if isinstance(v.get("scaling_factor"), (int, float)) and not isinstance(v.get("scaling_factor"), bool):
            kw["scaling_factor"] = float(v["scaling_factor"])
        if isinstance(v.get("block_out_channels"), list):
            if not all(isinstance(e, int) and not isinstance(e, bool) and e >= 0 for e in v["block_out_channels"]):
                raise InvalidArgument("VaeDecoderConfig.from_json_str: block_out_channels entry must be a non-negative integer")
            kw["block_out_channels"] = tuple(v["block_out_channels"])
        c = cls(**kw)
        c.validate()
        return c

    @classmethod
    def from_file(cls, path) -> "VaeConfig":
        try:
            text = open(path, encoding="utf-8").read()
        except (OSError, UnicodeDecodeError) as e:
            raise InvalidArgument(f"VaeDecoderConfig.from_file: failed to read {path}: {e}") from None
        return cls.from_json_str(text)


VaeDecoderConfig = VaeEncoderConfig = VaeConfig                    # one config for both halves (ferrotorch-diffusion/src/vae_encoder.rs:41)


class Encoder(nn.Module):
    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        ch, g = c.block_out_channels, c.norm_num_groups
        self.conv_in = nn.Conv2d(c.in_channels, ch[0], 3, padding=1)
        self.down_blocks = nn.ModuleList([DownEncoderBlock2D(ch[max(i - 1, 0)], ch[i], c.layers_per_block, i < len(ch) - 1, g) for i in range(len(ch))])
        self.mid_block = UNetMidBlock2D(ch[-1], g)
        self.conv_norm_out = nn.GroupNorm(g, ch[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[-1], 2 * c.latent_channels, 3, padding=1)

    def forward(self, x):
        x = self.conv_in(x)
        for b in self.down_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(self.mid_block(x))))


class Decoder(nn.Module):
    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        ch, g = list(reversed(c.block_out_channels)), c.norm_num_groups
        self.conv_in = nn.Conv2d(c.latent_channels, ch[0], 3, padding=1)
        self.mid_block = UNetMidBlock2D(ch[0], g)
        self.up_blocks = nn.ModuleList([UpDecoderBlock2D(ch[max(i - 1, 0)], ch[i], c.layers_per_block + 1, i < len(ch) - 1, g) for i in range(len(ch))])
        self.conv_norm_out = nn.GroupNorm(g, ch[-1], eps=1e-6)
        self.conv_out = nn.Conv2d(ch[-1], c.in_channels, 3, padding=1)

    def forward(self, z):
        x = self.mid_block(self.conv_in(z))
        for b in self.up_blocks:
            x = b(x)
        return self.conv_out(F.silu(self.conv_norm_out(x)))


class DiagonalGaussianDistribution:
    """Posterior of the VAE encoder: channel halves ``[mean, logvar]`` of ``[B, 2L, h, w]`` moments, log-variance clamped to [-30, 20]
    (ferrotorch-diffusion/src/vae_encoder.rs:464-560)."""

    def __init__(self, mean: torch.Tensor, logvar: torch.Tensor):
        self.mean, self.logvar = mean, logvar

    @classmethod
    def from_parameters(cls, params: torch.Tensor, latent_channels: int) -> "DiagonalGaussianDistribution":
        if params.dim() != 4 or params.shape[1] != 2 * latent_channels:
            raise ShapeMismatch(f"DiagonalGaussianDistribution.from_parameters: expected [B, {2 * latent_channels}, H, W], got {list(params.shape)}")
        mean, logvar = params.chunk(2, 1)
        return cls(mean, logvar.clamp(-30.0, 20.0))

    def mode(self) -> torch.Tensor:
        return self.mean

    def std(self) -> torch.Tensor:
        return (0.5 * self.logvar).exp()

    def sample(self, generator: Optional[torch.Generator] = None) -> torch.Tensor:
        eps = torch.randn(self.mean.shape, generator=generator, dtype=torch.float32, device=generator.device if generator is not None else "cpu")
        return self.mean + self.std() * eps.to(self.mean.device, self.mean.dtype)

    def sample_with_seed(self, seed: int) -> torch.Tensor:
        return self.sample(torch.Generator().manual_seed(int(seed)))

    def kl(self) -> torch.Tensor:
        return 0.5 * (self.mean.pow(2) + self.logvar.exp() - 1.0 - self.logvar).flatten(1).sum(1)


class VaeEncoder(nn.Module):
    """``encoder`` + ``quant_conv`` of an AutoencoderKL: image in [-1, 1] -> posterior over latents (ferrotorch-diffusion/src/vae_encoder.rs:295)."""

    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        c.validate()
        self.config = c
        self.encoder = Encoder(c)
        self.quant_conv = nn.Conv2d(2 * c.latent_channels, 2 * c.latent_channels, 1)

    def encode(self, image: torch.Tensor) -> DiagonalGaussianDistribution:
        if image.dim() != 4 or image.shape[1] != self.config.in_channels:
            raise ShapeMismatch(f"VaeEncoder.encode: expected [B, {self.config.in_channels}, H, W], got {list(image.shape)}")
        return DiagonalGaussianDistribution.from_parameters(self.quant_conv(self.encoder(image)), self.config.latent_channels)

    def encode_with_scaling(self, image: torch.Tensor, seed: Optional[int] = None) -> torch.Tensor:
        """Posterior sample (``seed`` given) or mode, times ``scaling_factor``: the latent the UNet sees (vae_encoder.rs:354)."""
        d = self.encode(image)
        return (d.mode() if seed is None else d.sample_with_seed(seed)) * self.config.scaling_factor

    def forward(self, image):
        return self.quant_conv(self.encoder(image))

    def load_hf_state_dict(self, hf_state, strict: bool = True) -> DropReport:
        return _load_prefixed(self, hf_state, {"vae.": ""}, ("encoder.", "quant_conv."), strict, "VaeEncoder")


class VaeDecoder(nn.Module):
    """``post_quant_conv`` + ``decoder`` of an AutoencoderKL (ferrotorch-diffusion/src/vae.rs:261)."""

    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        c.validate()
        self.config = c
        self.post_quant_conv = nn.Conv2d(c.latent_channels, c.latent_channels, 1)
        self.decoder = Decoder(c)

    def forward(self, z):
        if z.dim() != 4 or z.shape[1] != self.config.latent_channels:
            raise ShapeMismatch(f"VaeDecoder: expected [B, {self.config.latent_channels}, h, w], got {list(z.shape)}")
        return self.decoder(self.post_quant_conv(z))

    decode = forward

    def decode_with_scaling(self, latent: torch.Tensor) -> torch.Tensor:
        """``decode(latent / scaling_factor)``: undoes the scaling the pipeline's latents carry (vae.rs:303)."""
        return self.forward(latent / self.config.scaling_factor)

    def load_hf_state_dict(self, hf_state, strict: bool = True) -> DropReport:
        """Takes ``post_quant_conv.*`` / ``decoder.*`` (bare or under ``vae.``); the encoder half is refused under ``strict`` and otherwise
        listed (ferrotorch-diffusion/src/safetensors_loader.rs:58-105)."""
        return _load_prefixed(self, hf_state, {"vae.": ""}, ("decoder.", "post_quant_conv."), strict, "VaeDecoder")


class AutoencoderKL(nn.Module):
    def __init__(self, c: VaeConfig = VaeConfig()):
        super().__init__()
        self.config = c
        self.encoder, self.decoder = Encoder(c), Decoder(c)
        self.quant_conv = nn.Conv2d(2 * c.latent_channels, 2 * c.latent_channels, 1)
        self.post_quant_conv = nn.Conv2d(c.latent_channels, c.latent_channels, 1)

    def encode(self, x, sample: bool = True, generator=None):
        mean, logvar = self.quant_conv(self.encoder(x)).chunk(2, 1)
        if not sample:
            return mean
        return mean + (0.5 * logvar.clamp(-30, 20)).exp() * torch.randn(mean.shape, generator=generator, device=mean.device, dtype=mean.dtype)

    def decode(self, z):
        return self.decoder(self.post_quant_conv(z))

    def decode_with_scaling(self, latent):
        return self.decode(latent / self.config.scaling_factor)


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

    @classmethod
    def sd_v1_5(cls): return cls()                                 # ferrotorch-diffusion/src/clip_text_encoder.rs:130

    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    def validate(self) -> None:
        if min(self.vocab_size, self.hidden_size, self.intermediate_size, self.num_hidden_layers, self.num_attention_heads, self.max_position_embeddings) <= 0:
            raise InvalidArgument("ClipTextConfig: sizes must all be positive")
        if self.hidden_size % self.num_attention_heads:
            raise InvalidArgument(f"ClipTextConfig: hidden_size ({self.hidden_size}) must be divisible by num_attention_heads ({self.num_attention_heads})")
        if not (self.layer_norm_eps > 0 and math.isfinite(self.layer_norm_eps)):
            raise InvalidArgument("ClipTextConfig: layer_norm_eps must be positive and finite")

    @classmethod
    def from_json_str(cls, s: str) -> "ClipTextConfig":
        """A transformers ``text_encoder/config.json`` (the text tower's keys, also when nested under ``text_config``); absent keys keep the
        SD-1.5 defaults (clip_text_encoder.rs:197-235)."""
        try:
            v = json.loads(s)
        except ValueError as e:
            raise InvalidArgument(f"ClipTextConfig.from_json_str: bad JSON: {e}") from None
        if isinstance(v.get("text_config"), dict):
            v = v["text_config"]
        act = v.get("hidden_act", "quick_gelu")
        if act != "quick_gelu":
            raise InvalidArgument(f"ClipTextConfig.from_json_str: unsupported hidden_act {act!r} (only quick_gelu)")
        c = cls(**{k: v[k] for k in cls.__dataclass_fields__ if isinstance(v.get(k), (int, float)) and not isinstance(v.get(k), bool)})
        c.validate()
        return c

    @classmethod
    def from_file(cls, path) -> "ClipTextConfig":
        try:
            text = open(path, encoding="utf-8").read()
        except (OSError, UnicodeDecodeError) as e:
            raise InvalidArgument(f"ClipTextConfig.from_file: failed to read {path}: {e}") from None
        return cls.from_json_str(text)


class ClipSelfAttention(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.h = c.num_attention_heads
        self.q_proj, self.k_proj, self.v_proj, self.out_proj = (nn.Linear(c.hidden_size, c.hidden_size) for _ in range(4))

    def forward(self, x):
        B, S, E = x.shape
        sp = lambda t: t.view(B, S, self.h, E // self.h).transpose(1, 2)
        o = sdpa(sp(self.q_proj(x)), sp(self.k_proj(x)), sp(self.v_proj(x)), is_causal=True)
        return self.out_proj(o.transpose(1, 2).reshape(B, S, E))


class ClipMlp(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.fc1, self.fc2 = nn.Linear(c.hidden_size, c.intermediate_size), nn.Linear(c.intermediate_size, c.hidden_size)

    def forward(self, x):
        h = self.fc1(x)
        return self.fc2(h * torch.sigmoid(1.702 * h))               # quick_gelu


class ClipEncoderLayer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.self_attn, self.mlp = ClipSelfAttention(c), ClipMlp(c)
        self.layer_norm1, self.layer_norm2 = nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps), nn.LayerNorm(c.hidden_size, eps=c.layer_norm_eps)

    def forward(self, x):
        x = x + self.self_attn(self.layer_norm1(x))
        return x + self.mlp(self.layer_norm2(x))


class ClipTextEmbeddings(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.token_embedding = nn.Embedding(c.vocab_size, c.hidden_size)
        self.position_embedding = nn.Embedding(c.max_position_embeddings, c.hidden_size)

    def forward(self, ids):
        return self.token_embedding(ids) + self.position_embedding.weight[: ids.shape[1]]


class ClipEncoder(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.layers = nn.ModuleList([ClipEncoderLayer(c) for _ in range(c.num_hidden_layers)])

    def forward(self, x):
        for l in self.layers:
            x = l(x)
        return x


class _ClipTextTransformer(nn.Module):
    def __init__(self, c):
        super().__init__()
        self.embeddings, self.encoder = ClipTextEmbeddings(c), ClipEncoder(c)
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

    forward_from_id_tensor = forward

    def forward_from_ids(self, input_ids: Sequence[int]) -> torch.Tensor:
        """One prompt as a plain list of token ids -> ``[1, S, hidden]`` (ferrotorch-diffusion/src/clip_text_encoder.rs:1054)."""
        if len(input_ids) == 0 or len(input_ids) > self.config.max_position_embeddings:
            raise InvalidArgument(f"ClipTextEncoder: 1..{self.config.max_position_embeddings} token ids expected, got {len(input_ids)}")
        if max(input_ids) >= self.config.vocab_size:
            raise InvalidArgument(f"ClipTextEncoder: token id {max(input_ids)} outside the vocabulary ({self.config.vocab_size})")
        dev = self.text_model.final_layer_norm.weight.device
        return self.forward(torch.tensor([list(input_ids)], dtype=torch.long, device=dev))

    def load_hf_state_dict(self, hf_state, strict: bool = True) -> DropReport:
        """A ``CLIPTextModel`` state dict (``text_model.*`` or bare): the ``position_ids`` buffer is dropped in both modes, keys outside the text
        tower are refused under ``strict`` and otherwise listed (ferrotorch-diffusion/src/clip_text_encoder.rs:1129-1170)."""
        st = {(k if k.startswith("text_model.") else "text_model." + k): v for k, v in hf_state.items()}
        rep = _load_prefixed(self, st, {}, ("text_model.embeddings.token_embedding.", "text_model.embeddings.position_embedding.", "text_model.encoder.",
                                            "text_model.final_layer_norm."), strict, "ClipTextEncoder", always_drop=("text_model.embeddings.position_ids",))
        back = {(k if k.startswith("text_model.") else "text_model." + k): k for k in hf_state}
        return DropReport(dropped=tuple(sorted(back[k] for k in rep.dropped)))


# ----------------------------------------------------------------------------------------------------------------------
# scheduler + pipeline
# ----------------------------------------------------------------------------------------------------------------------
class BetaSchedule(enum.Enum):
    """ferrotorch-diffusion/src/scheduler.rs:25."""
    ScaledLinear = "scaled_linear"
    Linear = "linear"


class TimestepSpacing(enum.Enum):
    """ferrotorch-diffusion/src/scheduler.rs:34."""
    Leading = "leading"
    Linspace = "linspace"


class PredictionType(enum.Enum):
    """What the UNet predicts. The reference implements ``Epsilon`` only (scheduler.rs:74); the other two are extras of this scheduler."""
    Epsilon = "epsilon"
    VPrediction = "v_prediction"
    Sample = "sample"


@dataclass
class DDIMConfig:
    """The scheduler fields that change the arithmetic, SD-1.5 defaults (ferrotorch-diffusion/src/scheduler.rs:46-103)."""
    num_train_timesteps: int = 1000
    beta_start: float = 0.00085
    beta_end: float = 0.012
    beta_schedule: BetaSchedule = BetaSchedule.ScaledLinear
    clip_sample: bool = False
    set_alpha_to_one: bool = False
    prediction_type: PredictionType = PredictionType.Epsilon
    timestep_spacing: TimestepSpacing = TimestepSpacing.Leading
    steps_offset: int = 1

    @classmethod
    def sd_v1_5(cls) -> "DDIMConfig":
        return cls()


class DDIMScheduler:
    """DDIM sampler. Built from keyword fields or from a :class:`DDIMConfig` as the first argument (ferrotorch-diffusion/src/scheduler.rs:109)."""

    def __init__(self, num_train_timesteps=1000, beta_start: float = 0.00085, beta_end: float = 0.012, beta_schedule="scaled_linear",
                 set_alpha_to_one: bool = False, steps_offset: int = 1, prediction_type="epsilon", timestep_spacing="leading", clip_sample: bool = False):
        if isinstance(num_train_timesteps, DDIMConfig):
            c = num_train_timesteps
        else:
            try:
                c = DDIMConfig(int(num_train_timesteps), beta_start, beta_end, BetaSchedule(getattr(beta_schedule, "value", beta_schedule)), clip_sample,
                               set_alpha_to_one, PredictionType(getattr(prediction_type, "value", prediction_type)),
                               TimestepSpacing(getattr(timestep_spacing, "value", timestep_spacing)), steps_offset)
            except ValueError as e:
                raise InvalidArgument(f"DDIMScheduler: {e}") from None
        if c.num_train_timesteps <= 0 or not (0 < c.beta_start <= c.beta_end < 1):
            raise InvalidArgument("DDIMScheduler: need num_train_timesteps > 0 and 0 < beta_start <= beta_end < 1")
        self._config = c
        num_train_timesteps = c.num_train_timesteps
        if c.beta_schedule is BetaSchedule.ScaledLinear:
            betas = torch.linspace(c.beta_start ** 0.5, c.beta_end ** 0.5, num_train_timesteps, dtype=torch.float64) ** 2
        else:
            betas = torch.linspace(c.beta_start, c.beta_end, num_train_timesteps, dtype=torch.float64)
        self.alphas_cumprod = torch.cumprod(1.0 - betas, 0)
        self.final_alpha_cumprod = torch.tensor(1.0, dtype=torch.float64) if c.set_alpha_to_one else self.alphas_cumprod[0]
        self.num_train_timesteps, self.steps_offset, self.prediction_type = num_train_timesteps, c.steps_offset, c.prediction_type.value
        self.init_noise_sigma = 1.0
        self.timesteps: torch.Tensor = torch.arange(num_train_timesteps - 1, -1, -1)
        self.num_inference_steps = num_train_timesteps

    def config(self) -> DDIMConfig:
        return self._config

    def set_timesteps(self, n: int) -> List[int]:
        """Chooses the inference grid, highest timestep first, and returns it (scheduler.rs:191-248)."""
        if n <= 0:
            raise InvalidArgument("DDIMScheduler.set_timesteps: num_inference_steps must be > 0")
        if n > self.num_train_timesteps:
            raise InvalidArgument(f"DDIMScheduler.set_timesteps: num_inference_steps {n} must be <= num_train_timesteps {self.num_train_timesteps}")
        self.num_inference_steps = n
        if self._config.timestep_spacing is TimestepSpacing.Leading:
            ts = (torch.arange(n) * (self.num_train_timesteps // n)).flip(0) + self.steps_offset
        else:
            ts = torch.tensor([int(round(i * self.num_train_timesteps / n)) for i in reversed(range(n))], dtype=torch.long)
        self.timesteps = ts.clamp_max(self.num_train_timesteps - 1)
        return self.timesteps.tolist()

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
        if self._config.clip_sample:
            x0 = x0.clamp(-1.0, 1.0)
            eps = (sample - a_t ** 0.5 * x0) / (1 - a_t) ** 0.5
        var = (1 - a_prev) / (1 - a_t) * (1 - a_t / a_prev)
        sigma = eta * max(var, 0.0) ** 0.5
        prev = a_prev ** 0.5 * x0 + max(1 - a_prev - sigma ** 2, 0.0) ** 0.5 * eps
        if eta > 0:
            prev = prev + sigma * torch.randn(sample.shape, generator=generator, device=sample.device, dtype=sample.dtype)
        return prev

    def add_noise(self, x0, noise, t):
        a = self.alphas_cumprod.to(x0.device)[t].to(x0.dtype).view(-1, 1, 1, 1)
        return a.sqrt() * x0 + (1 - a).sqrt() * noise


@dataclass
class PipelineStepDump:
    """What one denoising step produced, for stage-by-stage comparison against another implementation (ferrotorch-diffusion/src/pipeline.rs:38)."""
    step: int
    timestep: int
    noise_pred_uncond: torch.Tensor
    noise_pred_cond: torch.Tensor
    guided_noise: torch.Tensor
    latent_after_step: torch.Tensor


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

    def encode_prompt(self, input_ids) -> torch.Tensor:
        """Token ids (list or ``[B, S]`` tensor) -> CLIP hidden states (pipeline.rs:101)."""
        return self.text_encoder(input_ids.to(next(self.text_encoder.parameters()).device)) if torch.is_tensor(input_ids) \
            else self.text_encoder.forward_from_ids(input_ids)

    @torch.no_grad()
    def generate(self, cond_embeds: torch.Tensor, uncond_embeds: torch.Tensor, init_latent: torch.Tensor, num_inference_steps: int,
                 guidance_scale: float) -> Tuple[torch.Tensor, List[PipelineStepDump]]:
        """The reference's entry point (pipeline.rs:167-245): ready-made embeddings and starting latent in, decoded image in [-1, 1] and one
        :class:`PipelineStepDump` per step out. The two UNet passes of a step run as one batch of two."""
        if init_latent.dim() != 4:
            raise ShapeMismatch(f"StableDiffusionPipeline.generate: expected init_latent [B, {self.unet.config.in_channels}, H, W], got {list(init_latent.shape)}")
        if cond_embeds.shape != uncond_embeds.shape:
            raise ShapeMismatch(f"StableDiffusionPipeline.generate: cond_embeds shape {list(cond_embeds.shape)} != uncond_embeds {list(uncond_embeds.shape)}")
        p = next(self.unet.parameters())
        latent = init_latent.to(p.device, p.dtype) * self.scheduler.init_noise_sigma
        ctx = torch.cat([uncond_embeds, cond_embeds], 0).to(p.device, p.dtype)
        dumps = []
        for i, t in enumerate(self.scheduler.set_timesteps(num_inference_steps)):
            inp = self.scheduler.scale_model_input(latent, t)
            eu, ec = self.unet(torch.cat([inp, inp], 0), torch.tensor([t], device=p.device), ctx).chunk(2, 0)
            guided = eu + guidance_scale * (ec - eu)
            latent = self.scheduler.step(guided, t, latent)
            dumps.append(PipelineStepDump(i, int(t), eu, ec, guided, latent))
        return self.vae.decode_with_scaling(latent), dumps

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
        for t in self.scheduler.set_timesteps(num_inference_steps):
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


def _read_weights(path, who: str) -> Dict[str, torch.Tensor]:
    from ..serialize import load_safetensors
    try:
        return load_safetensors(str(path))
    except Exception as e:
        raise InvalidArgument(f"{who}: failed to decode safetensors {path}: {e}") from None


def load_unet(path, cfg: Optional[UNetConfig] = None, strict: bool = True, device="cpu", dtype=torch.float32):
    """``unet/diffusion_pytorch_model.safetensors`` -> ``(UNet2DConditionModel, DropReport)`` (ferrotorch-diffusion/src/safetensors_loader.rs:159)."""
    m = UNet2DConditionModel(cfg or UNetConfig())
    rep = m.load_hf_state_dict(_read_weights(path, "load_unet"), strict)
    return m.to(device=device, dtype=dtype), rep


def load_clip_text_encoder(path, cfg: Optional[ClipTextConfig] = None, strict: bool = True, device="cpu", dtype=torch.float32):
    """``text_encoder/model.safetensors`` -> ``(ClipTextEncoder, DropReport)``; an integer ``position_ids`` tensor in the file is dropped
    and reported (safetensors_loader.rs:268)."""
    m = ClipTextEncoder(cfg or ClipTextConfig())
    rep = m.load_hf_state_dict(_read_weights(path, "load_clip_text_encoder"), strict)
    return m.to(device=device, dtype=dtype), rep


def load_vae_decoder(path, cfg: Optional[VaeConfig] = None, strict: bool = False, device="cpu", dtype=torch.float32):
    """The decoder half of ``vae/diffusion_pytorch_model.safetensors`` -> ``(VaeDecoder, DropReport)`` (safetensors_loader.rs:319). A whole
    AutoencoderKL file needs ``strict=False``: its encoder keys are then listed in the report."""
    m = VaeDecoder(cfg or VaeConfig())
    rep = m.load_hf_state_dict(_read_weights(path, "load_vae_decoder"), strict)
    return m.to(device=device, dtype=dtype), rep


def load_vae_encoder(path, cfg: Optional[VaeConfig] = None, strict: bool = False, device="cpu", dtype=torch.float32):
    """The encoder half (``encoder.*`` + ``quant_conv.*``) -> ``(VaeEncoder, DropReport)`` (safetensors_loader.rs:412)."""
    m = VaeEncoder(cfg or VaeConfig())
    rep = m.load_hf_state_dict(_read_weights(path, "load_vae_encoder"), strict)
    return m.to(device=device, dtype=dtype), rep


# the reference's device variants are these same modules on the device
GpuUNet2DConditional, GpuVaeDecoder, GpuVaeEncoder, GpuClipTextEncoder, GpuStableDiffusionPipeline = (
    UNet2DConditionModel, VaeDecoder, VaeEncoder, ClipTextEncoder, StableDiffusionPipeline)
