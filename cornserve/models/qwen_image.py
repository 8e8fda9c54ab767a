"""Qwen-Image text-to-image generator: MMDiT denoiser, flow-matching sampler and the pipeline around them.

The reference wraps ``diffusers.QwenImagePipeline`` with its text encoder removed
(python/cornserve/task_executors/geri/models/qwen_image.py:23-141): prompt embeddings arrive from the LLM
executor, the pipeline pads and masks them, runs ``num_inference_steps`` denoising steps and returns PNGs.
Here the denoiser, the sampler and the VAE decoder are this repository's own modules on its own kernels:

* 60 dual-stream blocks (image and text streams with separate weights, one joint attention): AdaLN
  modulation inside the LayerNorm kernel, fused q|k|v GEMM per stream written straight into the joint
  sequence, per-head RMSNorm + rotary in one in-place kernel, var-len tcgen05 attention over [text; image],
  output / MLP GEMMs with the gate and the residual in their epilogues;
* checkpoint tensor names are those of the diffusers transformer (``transformer_blocks.N.attn.to_q`` ...);
  the rotary embedding of the checkpoint is interleaved-pair complex multiplication, which is turned into
  the rotate-half form by permuting the rows of the q/k projections and q/k norms once at load time;
* Ulysses sequence parallelism: tokens are sharded over the group outside attention and heads inside it.
* true classifier-free guidance with norm rescaling is part of the Euler-step kernel.
"""

from __future__ import annotations

import base64
import io
import math
from dataclasses import dataclass, field
from typing import Iterable

import numpy as np
import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group
from .layers import LayerNorm, Linear, RMSNorm
from .qwen_image_vae import QwenImageVAEConfig, QwenImageVAEDecoder


@dataclass
class QwenImageDiTConfig:
    patch_size: int = 2
    in_channels: int = 64
    out_channels: int = 16
    num_layers: int = 60
    attention_head_dim: int = 128
    num_attention_heads: int = 24
    joint_attention_dim: int = 3584
    axes_dims_rope: tuple[int, int, int] = (16, 56, 56)
    rope_theta: float = 10000.0

    @property
    def inner_dim(self) -> int:
        return self.num_attention_heads * self.attention_head_dim

    @classmethod
    def from_hf(cls, cfg: dict) -> "QwenImageDiTConfig":
        kw = {k: cfg[k] for k in cls.__dataclass_fields__ if k in cfg}
        if "axes_dims_rope" in kw:
            kw["axes_dims_rope"] = tuple(kw["axes_dims_rope"])
        return cls(**kw)


@dataclass
class FlowMatchConfig:
    """Flow-matching Euler schedule with resolution-dependent exponential time shift."""

    base_image_seq_len: int = 256
    max_image_seq_len: int = 8192
    base_shift: float = 0.5
    max_shift: float = 0.9
    shift_terminal: float | None = 0.02
    num_train_timesteps: int = 1000


def flow_match_sigmas(num_steps: int, image_seq_len: int, cfg: FlowMatchConfig | None = None) -> np.ndarray:
    """``num_steps + 1`` noise levels from 1 towards 0 (the last entry is exactly 0)."""
    cfg = cfg or FlowMatchConfig()
    sig = np.linspace(1.0, 1.0 / num_steps, num_steps, dtype=np.float64)
    m = (cfg.max_shift - cfg.base_shift) / (cfg.max_image_seq_len - cfg.base_image_seq_len)
    mu = image_seq_len * m + (cfg.base_shift - m * cfg.base_image_seq_len)
    sig = math.exp(mu) / (math.exp(mu) + (1.0 / sig - 1.0))
    if cfg.shift_terminal is not None:
        one_minus = 1.0 - sig
        sig = 1.0 - one_minus / (one_minus[-1] / (1.0 - cfg.shift_terminal))
    return np.concatenate([sig, [0.0]]).astype(np.float32)


def interleaved_to_half_perm(head_dim: int) -> torch.Tensor:
    """Row order that maps channel pairs ``(2i, 2i+1)`` of a head to ``(i, i + d/2)``."""
    return torch.cat([torch.arange(0, head_dim, 2), torch.arange(1, head_dim, 2)])


def timestep_embedding(t: torch.Tensor, dim: int = 256, scale: float = 1000.0, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal features ``[cos | sin]`` of ``scale * t`` (``t`` in [0, 1])."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    ang = (t.float() * scale)[:, None] * freqs[None, :]
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


class RopeTable:
    """cos/sin tables ``[tokens, 2, d/2]`` for image tokens (frame, row, column axes with centred row/column
    indices) and text tokens (one index on all three axes, starting after the largest image index)."""

    def __init__(self, cfg: QwenImageDiTConfig):
        self.axes = cfg.axes_dims_rope
        self.theta = cfg.rope_theta

    def _freqs(self, pos: np.ndarray, dim: int) -> np.ndarray:
        inv = 1.0 / (self.theta ** (np.arange(0, dim, 2, dtype=np.float64) / dim))
        return pos.astype(np.float64)[:, None] * inv[None, :]

    def image(self, frames: int, h: int, w: int) -> np.ndarray:
        a0, a1, a2 = self.axes
        f = np.arange(frames)
        hh = np.concatenate([np.arange(-(h - h // 2), 0), np.arange(0, h // 2)])
        ww = np.concatenate([np.arange(-(w - w // 2), 0), np.arange(0, w // 2)])
        F = np.broadcast_to(self._freqs(f, a0)[:, None, None, :], (frames, h, w, a0 // 2))
        Hh = np.broadcast_to(self._freqs(hh, a1)[None, :, None, :], (frames, h, w, a1 // 2))
        Ww = np.broadcast_to(self._freqs(ww, a2)[None, None, :, :], (frames, h, w, a2 // 2))
        ang = np.concatenate([F, Hh, Ww], axis=-1).reshape(frames * h * w, -1)
        return np.stack([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)

    def text(self, length: int, h: int, w: int) -> np.ndarray:
        start = max(h // 2, w // 2)
        pos = np.arange(start, start + length)
        ang = np.concatenate([self._freqs(pos, a) for a in self.axes], axis=-1)
        return np.stack([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)


class StreamParams(nn.Module):
    """Weights of one stream (image or text) of a dual-stream block."""

    def __init__(self, dim: int, head_dim: int, device):
        super().__init__()
        self.mod = Linear(dim, 6 * dim, device=device)
        self.qkv = Linear(dim, 3 * dim, device=device)
        self.norm_q = RMSNorm(head_dim, 1e-6, device=device)
        self.norm_k = RMSNorm(head_dim, 1e-6, device=device)
        self.out = Linear(dim, dim, device=device)
        self.fc1 = Linear(dim, 4 * dim, device=device)
        self.fc2 = Linear(4 * dim, dim, device=device)


class DualStreamBlock(nn.Module):
    def __init__(self, cfg: QwenImageDiTConfig, group: ParallelGroup, device):
        super().__init__()
        self.cfg, self.group = cfg, group
        D, d = cfg.inner_dim, cfg.attention_head_dim
        self.img = StreamParams(D, d, device)
        self.txt = StreamParams(D, d, device)
        self.norm = LayerNorm(D, 1e-6, affine=False, device=device)

    def forward(self, img: torch.Tensor, txt: torch.Tensor, temb_act: torch.Tensor, lay: "JointLayout"):
        """``img`` ``[B*n_img, D]``, ``txt`` ``[B*n_txt, D]`` (this rank's token shards), ``temb_act`` =
        ``silu(time embedding)`` ``[B, D]``.  Returns the updated streams."""
        cfg = self.cfg
        D, H, d = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
        B = lay.batch
        mod_i = self.img.mod(temb_act)  # [B, 6D] = shift1 | scale1 | gate1 | shift2 | scale2 | gate2
        mod_t = self.txt.mod(temb_act)
        # ---- joint attention ------------------------------------------------------------------------
        xi = self.norm(img, scale=mod_i[:, D:2 * D], shift=mod_i[:, :D], rows_per_batch=lay.n_img)
        xt = self.norm(txt, scale=mod_t[:, D:2 * D], shift=mod_t[:, :D], rows_per_batch=lay.n_txt)
        if lay.fused is not None:
            attn = self._fused_sp_attention(xi, xt, lay)
        else:
            qkv = torch.empty((lay.rows, 3 * D), device=img.device, dtype=img.dtype)
            for b in range(B):
                ops.linear(xt[b * lay.n_txt:(b + 1) * lay.n_txt], self.txt.qkv.weight, self.txt.qkv.bias,
                           out=qkv[lay.txt_rows(b)])
                ops.linear(xi[b * lay.n_img:(b + 1) * lay.n_img], self.img.qkv.weight, self.img.qkv.bias,
                           out=qkv[lay.img_rows(b)])
            ops.qk_norm_rope_(qkv, H, d, D, self.txt.norm_q.weight, self.txt.norm_k.weight, 1e-6, lay.cs_rows,
                              wq2=self.img.norm_q.weight, wk2=self.img.norm_k.weight, seg=lay.per_sample, n_first=lay.n_txt)
            attn = lay.attention(qkv, H, d, self.group)  # [rows, D]
        for b in range(B):
            g_i, g_t = mod_i[b:b + 1, 2 * D:3 * D], mod_t[b:b + 1, 2 * D:3 * D]
            si, st = slice(b * lay.n_img, (b + 1) * lay.n_img), slice(b * lay.n_txt, (b + 1) * lay.n_txt)
            ops.linear(attn[lay.img_rows(b)], self.img.out.weight, self.img.out.bias, gate=g_i,
                       gate_rows_per_batch=lay.n_img, residual=img[si], out=img[si])
            ops.linear(attn[lay.txt_rows(b)], self.txt.out.weight, self.txt.out.bias, gate=g_t,
                       gate_rows_per_batch=lay.n_txt, residual=txt[st], out=txt[st])
        # ---- MLPs -----------------------------------------------------------------------------------
        for x, sp, mod, n in ((img, self.img, mod_i, lay.n_img), (txt, self.txt, mod_t, lay.n_txt)):
            h = self.norm(x, scale=mod[:, 4 * D:5 * D], shift=mod[:, 3 * D:4 * D], rows_per_batch=n)
            h = sp.fc1(h, act="gelu_tanh")
            ops.linear(h, sp.fc2.weight, sp.fc2.bias, gate=mod[:, 5 * D:6 * D], gate_rows_per_batch=n, residual=x, out=x)
        return img, txt

    def _fused_sp_attention(self, xi: torch.Tensor, xt: torch.Tensor, lay: "JointLayout") -> torch.Tensor:
        """Sequence-parallel joint attention whose exchanges ride in the kernels: the q|k|v projections store each
        head tile into the owning rank's buffer, the per-head norm and rotation run there on every token of the
        rank's heads, and the attention output returns to the token owners by one peer-store kernel."""
        cfg, fu = self.cfg, lay.fused
        d = cfg.attention_head_dim
        P, per = lay.sp, lay.per_sample
        Hl, own = fu.Hl, fu.own
        fu.qkv_scatter(xt, self.txt.qkv.weight, self.txt.qkv.bias, 0, lay.n_txt, per, per)
        fu.qkv_scatter(xi, self.img.qkv.weight, self.img.qkv.bias, lay.n_txt, lay.n_img, per, per)
        R = P * lay.rows
        full = fu.gathered_qkv(R)  # [R, 3 * own], rows = (sample, rank, that rank's [text; image] tokens)
        ops.qk_norm_rope_(full, Hl, d, own, self.txt.norm_q.weight, self.txt.norm_k.weight, 1e-6, lay.cs_full,
                          wq2=self.img.norm_q.weight, wk2=self.img.norm_k.weight, seg=per, n_first=lay.n_txt)
        packed = full if lay.gather_idx is None else ops.gather_rows(full, lay.gather_idx)
        T = packed.shape[0]
        q, k, v = (packed[:, i * own:(i + 1) * own].view(T, Hl, d) for i in range(3))
        o = ops.attention_varlen(q, k, v, lay.cu, lay.cu, lay.max_len).view(T, own)
        if lay.gather_idx is not None:
            o = ops.scatter_rows_(lay.o_full, lay.gather_idx, o)
        return fu.push_heads(o, per)


@dataclass
class JointLayout:
    """Row bookkeeping of the joint ``[text; image]`` sequence of every sample on this rank.

    Rows of sample ``b`` are ``[b*(n_txt+n_img), ...)``: first its ``n_txt`` text tokens, then its ``n_img`` image
    tokens (token shards when sequence parallel).  ``txt_len[b]`` counts the valid (unpadded) text tokens."""

    batch: int
    n_txt: int
    n_img: int
    txt_len: list[int]
    cs_txt: torch.Tensor
    cs_img: torch.Tensor
    sp: int = 1
    sp_rank: int = 0
    cu: torch.Tensor | None = None
    max_len: int = 0
    gather_idx: torch.Tensor | None = None
    fused: object | None = None         # FusedUlysses context when the exchanges are done by the kernels
    cs_full: torch.Tensor | None = None  # rotary table of every token of every rank, in gathered row order
    cs_rows: torch.Tensor | None = None  # rotary table of this rank's rows ([text; image] per sample)
    o_full: torch.Tensor | None = None   # zeroed [sp * rows, own] scratch for the scattered attention output

    @property
    def per_sample(self) -> int:
        return self.n_txt + self.n_img

    @property
    def rows(self) -> int:
        return self.batch * self.per_sample

    def txt_rows(self, b: int) -> slice:
        lo = b * self.per_sample
        return slice(lo, lo + self.n_txt)

    def img_rows(self, b: int) -> slice:
        lo = b * self.per_sample + self.n_txt
        return slice(lo, lo + self.n_img)

    def attention(self, qkv: torch.Tensor, H: int, d: int, group: ParallelGroup) -> torch.Tensor:
        """Joint attention over every sample's valid tokens; ``qkv`` is ``[rows, 3*H*d]``."""
        D = H * d
        if self.sp > 1:
            return ulysses_attention(qkv, H, d, self, group)
        src = qkv if self.gather_idx is None else ops.gather_rows(qkv, self.gather_idx)
        T = src.shape[0]
        q, k, v = (src[:, i * D:(i + 1) * D].view(T, H, d) for i in range(3))
        o = ops.attention_varlen(q, k, v, self.cu, self.cu, self.max_len).view(T, D)
        if self.gather_idx is None:
            return o
        out = torch.zeros((self.rows, D), device=qkv.device, dtype=qkv.dtype)
        return ops.scatter_rows_(out, self.gather_idx, o)


def ulysses_attention(qkv: torch.Tensor, H: int, d: int, lay: JointLayout, group: ParallelGroup) -> torch.Tensor:
    """Sequence-parallel joint attention with library collectives: all-to-all from token shards to head
    shards, attention over the full sequence on ``H / sp`` heads, all-to-all back."""
    P, R = lay.sp, lay.rows
    Hl = H // P
    # [R, 3, P, Hl*d] -> [P, R, 3*Hl*d]: block p goes to rank p
    send = qkv.view(R, 3, P, Hl * d).permute(2, 0, 1, 3).contiguous()
    recv = group.all_to_all(send.view(P * R, 3 * Hl * d)).view(P, lay.batch, lay.per_sample, 3 * Hl * d)
    # sample-major full sequences: [B, P, per_sample, ...]; padded text rows sit at known places and are masked
    # out by gathering only valid rows
    full = recv.permute(1, 0, 2, 3).reshape(lay.batch * P * lay.per_sample, 3 * Hl * d)
    packed = full if lay.gather_idx is None else ops.gather_rows(full, lay.gather_idx)
    T = packed.shape[0]
    q, k, v = (packed[:, i * Hl * d:(i + 1) * Hl * d].view(T, Hl, d) for i in range(3))
    o_full = ops.attention_varlen(q, k, v, lay.cu, lay.cu, lay.max_len).view(T, Hl * d)
    if lay.gather_idx is not None:
        o_full = ops.scatter_rows_(torch.zeros((lay.batch * P * lay.per_sample, Hl * d), device=qkv.device, dtype=qkv.dtype),
                                   lay.gather_idx, o_full)
    back = o_full.view(lay.batch, P, lay.per_sample, Hl * d).permute(1, 0, 2, 3).contiguous()
    out = group.all_to_all(back.view(P * R, Hl * d)).view(P, R, Hl * d)
    return out.permute(1, 0, 2).reshape(R, H * d)


class QwenImageDiT(nn.Module):
    """MMDiT denoiser.  ``forward`` takes packed latents ``[B, n_img, 64]`` and returns the velocity."""

    def __init__(self, cfg: QwenImageDiTConfig | None = None, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg = cfg or QwenImageDiTConfig()
        self.group = group or single_group(device)
        D = cfg.inner_dim
        if cfg.num_attention_heads % self.group.size != 0:
            raise ValueError("attention heads must divide over the sequence-parallel group")
        self.time_in1 = Linear(256, D, device=device)
        self.time_in2 = Linear(D, D, device=device)
        self.txt_norm = RMSNorm(cfg.joint_attention_dim, 1e-6, device=device)
        self.img_in = Linear(cfg.in_channels, D, device=device)
        self.txt_in = Linear(cfg.joint_attention_dim, D, device=device)
        self.blocks = nn.ModuleList([DualStreamBlock(cfg, self.group, device) for _ in range(cfg.num_layers)])
        self.norm_out = LayerNorm(D, 1e-6, affine=False, device=device)
        self.norm_out_mod = Linear(D, 2 * D, device=device)
        self.proj_out = Linear(D, cfg.patch_size * cfg.patch_size * cfg.out_channels, device=device)
        self.rope = RopeTable(cfg)
        self.fused_exchange = True  # sequence parallel: let the kernels do the exchanges when peer memory is there
        self._fused = None

    @property
    def device(self) -> torch.device:
        return self.img_in.weight.device

    @property
    def dtype(self) -> torch.dtype:
        return self.img_in.weight.dtype

    def make_layout(self, batch: int, txt_len: list[int], n_txt_pad: int, grid_hw: tuple[int, int]) -> JointLayout:
        """Precompute rotary tables, attention boundaries and (sequence parallel) gather indices."""
        dev, cfg = self.device, self.cfg
        h, w = grid_hw
        P, r = self.group.size, self.group.rank
        n_img_full = h * w
        if n_img_full % P or n_txt_pad % P:
            raise ValueError("token counts must divide over the sequence-parallel group")
        n_img, n_txt = n_img_full // P, n_txt_pad // P
        cs_img = self.rope.image(1, h, w)[r * n_img:(r + 1) * n_img]
        cs_txt = self.rope.text(n_txt_pad, h, w)[r * n_txt:(r + 1) * n_txt]
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
        lay = JointLayout(batch, n_txt, n_img, list(txt_len), t(cs_txt), t(cs_img), P, r)
        lay.cs_rows = t(np.tile(np.concatenate([cs_txt, cs_img]), (batch, 1, 1)))
        per = n_txt + n_img
        if all(n == n_txt_pad for n in txt_len):
            # no padding: a sample's rows are contiguous whatever the rank order inside (attention is not causal)
            lay.cu = t(np.arange(batch + 1, dtype=np.int32) * per * P)
            lay.max_len = per * P
        else:
            idx, cu = [], [0]
            for b in range(batch):
                n_valid = 0
                for p in range(P):
                    base = (b * P + p) * per
                    lo = p * n_txt
                    valid_txt = int(np.clip(txt_len[b] - lo, 0, n_txt))
                    idx.extend(range(base, base + valid_txt))
                    idx.extend(range(base + n_txt, base + per))
                    n_valid += valid_txt + n_img
                cu.append(cu[-1] + n_valid)
            lay.gather_idx = t(np.asarray(idx, dtype=np.int32))
            lay.cu = t(np.asarray(cu, dtype=np.int32))
            lay.max_len = int(np.diff(cu).max())
        own = (cfg.num_attention_heads // P) * cfg.attention_head_dim
        if P > 1 and self.fused_exchange and self.group.fabric is not None and dev.type == "cuda" and own % 128 == 0:
            from ..parallel.fused import FusedUlysses

            if self._fused is None or self._fused.cap < lay.rows:
                self._fused = FusedUlysses(self.group, cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim, lay.rows)
            lay.fused = self._fused
            full_txt, full_img = self.rope.text(n_txt_pad, h, w), self.rope.image(1, h, w)
            seg = np.concatenate([np.concatenate([full_txt[p * n_txt:(p + 1) * n_txt], full_img[p * n_img:(p + 1) * n_img]])
                                  for p in range(P)])
            lay.cs_full = t(np.tile(seg, (batch, 1, 1)))
            if lay.gather_idx is not None:
                lay.o_full = torch.zeros((P * lay.rows, own), device=dev, dtype=self.dtype)
        return lay

    @torch.inference_mode()
    def forward(self, latents: torch.Tensor, prompt: torch.Tensor, timestep: torch.Tensor, lay: JointLayout) -> torch.Tensor:
        """``latents`` ``[B*n_img, in_channels]`` and ``prompt`` ``[B*n_txt, joint_dim]`` are this rank's token
        shards; ``timestep`` ``[B]`` in [0, 1].  Returns the velocity ``[B*n_img, patch^2 * out_channels]``."""
        cfg = self.cfg
        D = cfg.inner_dim
        temb = timestep_embedding(timestep, 256).to(self.dtype)
        temb = self.time_in2(self.time_in1(temb, act="silu"))
        temb_act = ops.act_mul(torch.cat([temb, torch.ones_like(temb)], dim=-1), "silu")  # silu(temb)
        img = self.img_in(latents)
        txt = self.txt_in(self.txt_norm(prompt))
        if lay.fused is not None:
            lay.fused.begin_pass()
        for blk in self.blocks:
            img, txt = blk(img, txt, temb_act, lay)
        mod = self.norm_out_mod(temb_act)  # [B, 2D] = scale | shift
        x = self.norm_out(img, scale=mod[:, :D], shift=mod[:, D:], rows_per_batch=lay.n_img)
        return self.proj_out(x)

    # -- checkpoint loading (diffusers names) ----------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        cfg = self.cfg
        D, H, d = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
        perm = interleaved_to_half_perm(d)
        head_perm = (torch.arange(H)[:, None] * d + perm[None, :]).reshape(-1)
        loaded: set[str] = set()
        simple = {
            "time_text_embed.timestep_embedder.linear_1": self.time_in1,
            "time_text_embed.timestep_embedder.linear_2": self.time_in2,
            "img_in": self.img_in, "txt_in": self.txt_in, "norm_out.linear": self.norm_out_mod,
            "proj_out": self.proj_out,
        }
        for name, t in weights:
            mod_name, _, leaf = name.rpartition(".")
            if name == "txt_norm.weight":
                self.txt_norm.weight.data.copy_(t)
            elif mod_name in simple:
                simple[mod_name].load(**{leaf: t})
            elif name.startswith("transformer_blocks."):
                parts = name.split(".")
                blk: DualStreamBlock = self.blocks[int(parts[1])]
                sub = ".".join(parts[2:-1])
                tgt = self._block_target(blk, sub)
                if tgt is None:
                    continue
                layer, row_lo, permute = tgt
                if isinstance(layer, RMSNorm):
                    layer.weight.data.copy_(t[perm])
                elif row_lo is None:
                    layer.load(**{leaf: t})
                else:
                    src = t[head_perm] if permute else t
                    dst = layer.weight if leaf == "weight" else layer.bias
                    dst.data[row_lo:row_lo + D].copy_(src)
            else:
                continue
            loaded.add(name)
        return loaded

    @staticmethod
    def _block_target(blk: DualStreamBlock, sub: str):
        i, t = blk.img, blk.txt
        D = blk.cfg.inner_dim
        table = {
            "img_mod.1": (i.mod, None, False), "txt_mod.1": (t.mod, None, False),
            "attn.to_q": (i.qkv, 0, True), "attn.to_k": (i.qkv, D, True), "attn.to_v": (i.qkv, 2 * D, False),
            "attn.add_q_proj": (t.qkv, 0, True), "attn.add_k_proj": (t.qkv, D, True),
            "attn.add_v_proj": (t.qkv, 2 * D, False),
            "attn.norm_q": (i.norm_q, None, True), "attn.norm_k": (i.norm_k, None, True),
            "attn.norm_added_q": (t.norm_q, None, True), "attn.norm_added_k": (t.norm_k, None, True),
            "attn.to_out.0": (i.out, None, False), "attn.to_add_out": (t.out, None, False),
            "img_mlp.net.0.proj": (i.fc1, None, False), "img_mlp.net.2": (i.fc2, None, False),
            "txt_mlp.net.0.proj": (t.fc1, None, False), "txt_mlp.net.2": (t.fc2, None, False),
        }
        return table.get(sub)


def pack_latents(lat: torch.Tensor, patch: int = 2) -> torch.Tensor:
    """``[B, C, H, W]`` -> ``[B, (H/p)(W/p), C*p*p]`` (channel-major inside a patch)."""
    B, C, Hh, Ww = lat.shape
    x = lat.view(B, C, Hh // patch, patch, Ww // patch, patch).permute(0, 2, 4, 1, 3, 5)
    return x.reshape(B, (Hh // patch) * (Ww // patch), C * patch * patch)


def unpack_latents(x: torch.Tensor, h: int, w: int, patch: int = 2) -> torch.Tensor:
    """Inverse of :func:`pack_latents`: ``[B, h*w, C*p*p]`` -> ``[B, C, h*p, w*p]``."""
    B, _, cpp = x.shape
    C = cpp // (patch * patch)
    return x.view(B, h, w, C, patch, patch).permute(0, 3, 1, 4, 2, 5).reshape(B, C, h * patch, w * patch)


def encode_png(rgb: np.ndarray) -> bytes:
    """uint8 ``[H, W, 3]`` -> PNG bytes (PIL when present, else a minimal zlib writer)."""
    try:
        from PIL import Image

        buf = io.BytesIO()
        Image.fromarray(rgb).save(buf, format="PNG")
        return buf.getvalue()
    except ImportError:
        import struct
        import zlib

        h, w, _ = rgb.shape
        raw = b"".join(b"\x00" + rgb[y].tobytes() for y in range(h))

        def chunk(tag: bytes, data: bytes) -> bytes:
            return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xffffffff)

        return (b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
                + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


@dataclass
class QwenImagePipelineConfig:
    dit: QwenImageDiTConfig = field(default_factory=QwenImageDiTConfig)
    vae: QwenImageVAEConfig = field(default_factory=QwenImageVAEConfig)
    sched: FlowMatchConfig = field(default_factory=FlowMatchConfig)
    vae_scale_factor: int = 8


class QwenImageModel:
    """Batch generator with the interface of the reference's ``BatchGeriModel``
    (python/cornserve/task_executors/geri/models/base.py:62-90): ``generate(prompt_embeds, height, width,
    num_inference_steps) -> list[base64 PNG]``; extra keyword arguments add classifier-free guidance."""

    def __init__(self, cfg: QwenImagePipelineConfig | None = None, group: ParallelGroup | None = None, device="cpu",
                 seed: int = 0):
        self.cfg = cfg or QwenImagePipelineConfig()
        self.group = group or single_group(device)
        self.dit = QwenImageDiT(self.cfg.dit, self.group, device)
        self.vae = QwenImageVAEDecoder(self.cfg.vae, device)
        self.seed = seed

    @property
    def dtype(self) -> torch.dtype:
        return self.dit.dtype

    @property
    def device(self) -> torch.device:
        return self.dit.device

    @property
    def embedding_dim(self) -> int:
        return self.cfg.dit.joint_attention_dim

    def _shard(self, x: torch.Tensor, n_local: int) -> torch.Tensor:
        """``[B, n, C]`` -> this rank's token shard ``[B*n_local, C]``."""
        r = self.group.rank
        return x[:, r * n_local:(r + 1) * n_local].reshape(-1, x.shape[-1]).contiguous()

    @torch.inference_mode()
    def denoise(self, prompt_embeds: list[torch.Tensor], height: int, width: int, num_inference_steps: int,
                negative_embeds: list[torch.Tensor] | None = None, true_cfg_scale: float = 4.0,
                latents: torch.Tensor | None = None, batch_cfg: bool = True) -> torch.Tensor:
        """Run the sampler; returns clean latents ``[B, 16, height/8, width/8]`` (fp32).

        With a negative prompt, ``batch_cfg`` runs the conditional and the unconditional samples as one batch of
        ``2B`` per step (the reference pipeline calls the denoiser twice): the text-stream GEMMs and the modulation
        projections read their weights once instead of twice, and every launch carries twice the rows."""
        cfg, dev, P = self.cfg, self.device, self.group.size
        B = len(prompt_embeds)
        vs, patch = cfg.vae_scale_factor, cfg.dit.patch_size
        lh, lw = height // vs, width // vs
        gh, gw = lh // patch, lw // patch
        C = cfg.dit.out_channels
        if latents is None:
            g = torch.Generator(device="cpu").manual_seed(self.seed)
            latents = torch.randn((B, C, lh, lw), generator=g, dtype=torch.float32)
        x_full = pack_latents(latents.to(dev, torch.float32), patch)  # [B, n_img, 64]
        n_img = gh * gw // P
        x = self._shard(x_full, n_img)  # fp32 [B*n_img, 64]

        def prep(embeds: list[torch.Tensor]):
            lens = [int(e.shape[0]) for e in embeds]
            n_pad = -(-max(lens) // P) * P
            buf = torch.zeros((len(embeds), n_pad, self.embedding_dim), device=dev, dtype=self.dtype)
            for b, e in enumerate(embeds):
                buf[b, : lens[b]] = e.to(dev, self.dtype)
            lay = self.dit.make_layout(len(embeds), lens, n_pad, (gh, gw))
            return self._shard(buf, n_pad // P), lay

        both = unc = None
        if negative_embeds is not None and batch_cfg:
            both = prep(list(prompt_embeds) + list(negative_embeds))
        else:
            cond, lay_c = prep(prompt_embeds)
            unc = prep(negative_embeds) if negative_embeds is not None else None
        sig = flow_match_sigmas(num_inference_steps, gh * gw, cfg.sched)
        rows = B * n_img
        for i in range(num_inference_steps):
            xin = x.to(self.dtype)
            if both is not None:
                t = torch.full((2 * B,), float(sig[i]), device=dev, dtype=torch.float32)
                v = self.dit(torch.cat([xin, xin]), both[0], t, both[1])
                v_c, v_u = v[:rows], v[rows:]
            else:
                t = torch.full((B,), float(sig[i]), device=dev, dtype=torch.float32)
                v_c = self.dit(xin, cond, t, lay_c)
                v_u = self.dit(xin, unc[0], t, unc[1]) if unc is not None else None
            ops.flow_step_(x, v_c.contiguous(), None if v_u is None else v_u.contiguous(), true_cfg_scale,
                           float(sig[i + 1] - sig[i]), norm_rescale=True)
        x = x.view(B, n_img, -1)
        if P > 1:
            x = self.group.all_gather(x, dim=1)
        return unpack_latents(x, gh, gw, patch)

    @torch.inference_mode()
    def generate_rgb(self, prompt_embeds, height, width, num_inference_steps=50, **kw) -> torch.Tensor:
        """uint8 images ``[B, height, width, 3]`` on the device."""
        lat = self.denoise(prompt_embeds, height, width, num_inference_steps, **kw)
        return self.vae.decode_to_rgb8(lat)

    def generate(self, prompt_embeds: list[torch.Tensor], height: int, width: int, num_inference_steps: int = 50,
                 **kw) -> list[str]:
        rgb = self.generate_rgb(prompt_embeds, height, width, num_inference_steps, **kw).cpu().numpy()
        return [base64.b64encode(encode_png(img)).decode("ascii") for img in rgb]

    def load_weights(self, transformer: Iterable[tuple[str, torch.Tensor]], vae: Iterable[tuple[str, torch.Tensor]]):
        return self.dit.load_weights(transformer), self.vae.load_weights(vae)
