"""Decoder half of the Qwen-Image VAE (16-channel latents, 8x spatial upsampling) for single images.

The reference reaches this network through ``diffusers.QwenImagePipeline``
(python/cornserve/task_executors/geri/models/qwen_image.py:49,100-106).  The checkpoint is a causal *3-D*
convolutional decoder; for one frame every causal 3x3x3 convolution only sees its last temporal tap, so the
image decoder is a 2-D network built from that tap.  Activations are channels-last ``[pixels, C]`` bf16:

* 3x3 convolution = tap-gather kernel (SiLU of the preceding activation and the nearest 2x upsampling are
  applied while gathering) + tcgen05 GEMM with bias and residual in the epilogue;
* channel RMS norm = row RMSNorm kernel;
* the single-head middle attention = two GEMMs around a row soft-max kernel;
* output = clamp to [-1, 1] and uint8 conversion kernel.

Checkpoint tensor names are those of the diffusers autoencoder (``decoder.up_blocks.N.resnets.M.conv1`` ...).
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Iterable

import torch
from torch import nn

from .. import ops
from .layers import _param


@dataclass
class QwenImageVAEConfig:
    base_dim: int = 96
    z_dim: int = 16
    dim_mult: tuple[int, ...] = (1, 2, 4, 4)
    num_res_blocks: int = 2
    latents_mean: tuple[float, ...] = (-0.7571, -0.7089, -0.9113, 0.1075, -0.1745, 0.9653, -0.1517, 1.5508,
                                       0.4134, -0.0715, 0.5517, -0.3632, -0.1922, -0.9497, 0.2503, -0.2921)
    latents_std: tuple[float, ...] = (2.8184, 1.4541, 2.3275, 2.6558, 1.2196, 1.7708, 2.6052, 2.0743,
                                      3.2687, 2.1526, 2.8652, 1.5579, 1.6382, 1.1253, 2.8251, 1.9160)

    @classmethod
    def from_hf(cls, cfg: dict) -> "QwenImageVAEConfig":
        kw = {k: (tuple(cfg[k]) if isinstance(cfg[k], list) else cfg[k]) for k in cls.__dataclass_fields__ if k in cfg}
        return cls(**kw)


def conv_weight_2d(w: torch.Tensor) -> torch.Tensor:
    """Checkpoint conv weight (``[Co, Ci, kt, kh, kw]`` causal 3-D, or ``[Co, Ci, kh, kw]``) -> GEMM operand
    ``[Co, kh*kw*Ci]`` in (ky, kx, ci) order; a 3-D kernel contributes its last temporal tap."""
    if w.dim() == 5:
        w = w[:, :, -1]
    return w.permute(0, 2, 3, 1).reshape(w.shape[0], -1).contiguous()


class Conv(nn.Module):
    """3x3 (padding 1) or 1x1 convolution on channels-last pixels, as a GEMM."""

    def __init__(self, cin: int, cout: int, k: int, device, pad_out: int | None = None):
        super().__init__()
        self.cin, self.cout, self.k = cin, cout, k
        self.cout_padded = pad_out or cout
        self.weight = _param(self.cout_padded, k * k * cin, device=device, dtype=torch.bfloat16,
                             std=1.0 / math.sqrt(k * k * cin))
        self.bias = _param(self.cout_padded, device=device, dtype=torch.bfloat16, std=None)
        if self.cout_padded != cout:
            self.weight.data[cout:].zero_()

    def forward(self, x, B, H, W, *, silu=False, up=1, residual=None):
        if self.k == 1:
            assert not silu and up == 1
            return ops.linear(x, self.weight, self.bias, residual=residual)
        return ops.conv3x3(x, self.weight, self.bias, B, H, W, up=up, silu=silu, residual=residual)

    def load(self, weight=None, bias=None):
        if weight is not None:
            self.weight.data[: self.cout].copy_(conv_weight_2d(weight))
        if bias is not None:
            self.bias.data[: self.cout].copy_(bias)


class ChannelNorm(nn.Module):
    """``x / rms(x over channels) * gamma`` (the checkpoint's L2-normalise-and-scale norm)."""

    def __init__(self, dim: int, device):
        super().__init__()
        self.gamma = _param(dim, device=device, dtype=torch.bfloat16, std=1.0)

    def forward(self, x):
        return ops.rms_norm(x, self.gamma, 1e-12)

    def load(self, gamma):
        self.gamma.data.copy_(gamma.reshape(-1))


class ResBlock(nn.Module):
    def __init__(self, cin: int, cout: int, device):
        super().__init__()
        self.norm1, self.conv1 = ChannelNorm(cin, device), Conv(cin, cout, 3, device)
        self.norm2, self.conv2 = ChannelNorm(cout, device), Conv(cout, cout, 3, device)
        self.shortcut = Conv(cin, cout, 1, device) if cin != cout else None

    def forward(self, x, B, H, W):
        h = self.shortcut(x, B, H, W) if self.shortcut is not None else x
        y = self.conv1(self.norm1(x), B, H, W, silu=True)
        return self.conv2(self.norm2(y), B, H, W, silu=True, residual=h)


class MidAttention(nn.Module):
    """Single-head self-attention over the pixels of one image."""

    def __init__(self, dim: int, device):
        super().__init__()
        self.dim = dim
        self.norm = ChannelNorm(dim, device)
        self.to_qkv = Conv(dim, 3 * dim, 1, device)
        self.proj = Conv(dim, dim, 1, device)

    def forward(self, x, B, H, W):
        C, n = self.dim, H * W
        qkv = self.to_qkv(self.norm(x), B, H, W)
        out = torch.empty_like(x)
        for b in range(B):
            r = slice(b * n, (b + 1) * n)
            q, k, v = qkv[r, :C], qkv[r, C:2 * C], qkv[r, 2 * C:]
            s = ops.linear(q.contiguous(), k.contiguous())              # [n, n] scores
            p = ops.softmax_rows(s, 1.0 / math.sqrt(C))
            out[r] = ops.linear(p, v.t().contiguous())                   # [n, C]
        return self.proj(out, B, H, W, residual=x)


class QwenImageVAEDecoder(nn.Module):
    def __init__(self, cfg: QwenImageVAEConfig | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg = cfg or QwenImageVAEConfig()
        mult = list(cfg.dim_mult)
        dims = [cfg.base_dim * u for u in [mult[-1]] + mult[::-1]]
        self.post_quant = Conv(cfg.z_dim, cfg.z_dim, 1, device)
        self.conv_in = Conv(cfg.z_dim, dims[0], 3, device)
        self.mid_res = nn.ModuleList([ResBlock(dims[0], dims[0], device), ResBlock(dims[0], dims[0], device)])
        self.mid_attn = MidAttention(dims[0], device)
        self.up_res = nn.ModuleList()
        self.up_conv = nn.ModuleList()   # the 3x3 conv that follows the nearest 2x upsampling (None at the end)
        self.has_up: list[bool] = []
        for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
            if i > 0:
                cin //= 2
            blocks = [ResBlock(cin if j == 0 else cout, cout, device) for j in range(cfg.num_res_blocks + 1)]
            self.up_res.append(nn.ModuleList(blocks))
            up = i != len(mult) - 1
            self.has_up.append(up)
            self.up_conv.append(Conv(cout, cout // 2, 3, device) if up else nn.Identity())
        self.norm_out = ChannelNorm(dims[-1], device)
        self.conv_out = Conv(dims[-1], 3, 3, device, pad_out=8)
        self.register_buffer("lat_mean", torch.tensor(cfg.latents_mean, dtype=torch.float32, device=device), persistent=False)
        self.register_buffer("lat_std", torch.tensor(cfg.latents_std, dtype=torch.float32, device=device), persistent=False)

    @property
    def device(self) -> torch.device:
        return self.conv_in.weight.device

    @torch.inference_mode()
    def decode(self, latents: torch.Tensor) -> tuple[torch.Tensor, int, int, int]:
        """Normalised latents ``[B, 16, h, w]`` -> channels-last image rows ``[B*8h*8w, 8]`` (RGB in the first three
        columns, range about [-1, 1]) and ``(B, H, W)``."""
        B, C, H, W = latents.shape
        z = latents.float() * self.lat_std.view(1, -1, 1, 1) + self.lat_mean.view(1, -1, 1, 1)
        x = z.permute(0, 2, 3, 1).reshape(B * H * W, C).to(torch.bfloat16).contiguous()
        x = self.post_quant(x, B, H, W)
        x = self.conv_in(x, B, H, W)
        x = self.mid_res[0](x, B, H, W)
        x = self.mid_attn(x, B, H, W)
        x = self.mid_res[1](x, B, H, W)
        for blocks, up, has_up in zip(self.up_res, self.up_conv, self.has_up):
            for blk in blocks:
                x = blk(x, B, H, W)
            if has_up:
                x = up(x, B, H, W, up=2)
                H, W = 2 * H, 2 * W
        x = self.conv_out(self.norm_out(x), B, H, W, silu=True)
        return x, B, H, W

    def decode_to_rgb8(self, latents: torch.Tensor) -> torch.Tensor:
        x, B, H, W = self.decode(latents)
        return ops.to_rgb8(x).view(B, H, W, 3)

    # -- checkpoint loading (diffusers names) ----------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded: set[str] = set()
        for name, t in weights:
            tgt = self._target(name)
            if tgt is None:
                continue
            mod, leaf = tgt
            if isinstance(mod, ChannelNorm):
                mod.load(t)
            else:
                mod.load(**{leaf: t})
            loaded.add(name)
        return loaded

    def _target(self, name: str):
        p = name.split(".")
        leaf = p[-1]
        if p[0] == "post_quant_conv":
            return self.post_quant, leaf
        if p[0] != "decoder":
            return None
        p = p[1:]

        def res(blk: ResBlock, rest: list[str]):
            m = {"norm1": blk.norm1, "conv1": blk.conv1, "norm2": blk.norm2, "conv2": blk.conv2,
                 "conv_shortcut": blk.shortcut}.get(rest[0])
            return (m, leaf) if m is not None else None

        if p[0] == "conv_in":
            return self.conv_in, leaf
        if p[0] == "conv_out":
            return self.conv_out, leaf
        if p[0] == "norm_out":
            return self.norm_out, leaf
        if p[0] == "mid_block":
            if p[1] == "resnets":
                return res(self.mid_res[int(p[2])], p[3:])
            if p[1] == "attentions":
                m = {"norm": self.mid_attn.norm, "to_qkv": self.mid_attn.to_qkv, "proj": self.mid_attn.proj}.get(p[3])
                return (m, leaf) if m is not None else None
        if p[0] == "up_blocks":
            i = int(p[1])
            if p[2] == "resnets":
                return res(self.up_res[i][int(p[3])], p[4:])
            if p[2] == "upsamplers" and p[4] == "resample":
                return self.up_conv[i], leaf
            # upsamplers.0.time_conv only acts between frames of a video: unused for single images
        return None
