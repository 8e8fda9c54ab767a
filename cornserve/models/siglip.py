"""SigLIP vision tower and the two encoders built on it: Gemma-3 (average-pool + Gemma RMSNorm + projection,
one projector "adapter" per LLM size so that several Gemma models share one tower) and LLaVA-OneVision (MLP
projector, any-resolution tile packing with un-padding and row-end "newline" embeddings).  Reference:
python/cornserve/task_executors/eric/models/layers/siglip.py:22-404, gemma3.py:19-156, llava_onevision.py:24-318.

The tower runs on the shared encoder block: patch embedding as one GEMM over unfolded pixels with the learned
position table in the residual operand, LayerNorm blocks with GELU-tanh MLPs, dense attention inside every tile.
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Iterable

import numpy as np
import torch
import torch.nn.functional as F
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group
from .layers import LayerNorm, Linear, RMSNorm, _param
from .vit import HF_ACT, BlockSpec, EncoderBlock, fused_tp_blocks, fused_tp_context


@dataclass
class SiglipConfig:
    hidden_size: int = 1152
    intermediate_size: int = 4304
    num_hidden_layers: int = 27
    num_attention_heads: int = 16
    num_channels: int = 3
    image_size: int = 896
    patch_size: int = 14
    hidden_act: str = "gelu_pytorch_tanh"
    layer_norm_eps: float = 1e-6

    @classmethod
    def from_hf(cls, v: dict) -> "SiglipConfig":
        return cls(**{k: v[k] for k in cls.__dataclass_fields__ if k in v})

    @property
    def num_patches(self) -> int:
        return (self.image_size // self.patch_size) ** 2


class SiglipVisionTower(nn.Module):
    """``forward(pixel_values [B, 3, S, S]) -> [B, N, hidden]``; ``num_layers`` truncates the stack (feature taps),
    ``post_norm`` applies the final LayerNorm."""

    def __init__(self, cfg: SiglipConfig, group: ParallelGroup, device, num_layers: int | None = None, post_norm: bool = True):
        super().__init__()
        self.cfg = cfg
        H, p = cfg.hidden_size, cfg.patch_size
        self.k_raw = cfg.num_channels * p * p
        self.k_pad = (-self.k_raw) % 8   # TMA rows must be multiples of 16 bytes: 3*14*14 = 588 -> 592 zero-padded columns
        self.patch_embed = Linear(self.k_raw + self.k_pad, H, bias=True, device=device)
        self.patch_embed.weight.data[:, self.k_raw:].zero_()
        self.pos_embed = _param(cfg.num_patches, H, device=device, dtype=torch.bfloat16)
        spec = BlockSpec(H, cfg.num_attention_heads, cfg.intermediate_size, norm="layer", eps=cfg.layer_norm_eps,
                         act=HF_ACT[cfg.hidden_act])
        n = cfg.num_hidden_layers if num_layers is None else num_layers
        self.layers = nn.ModuleList([EncoderBlock(spec, group, device) for _ in range(n)])
        self.post_layernorm = LayerNorm(H, cfg.layer_norm_eps, device=device) if post_norm else None

    def forward(self, pixel_values: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, C, S, _ = pixel_values.shape
        p, g = cfg.patch_size, S // cfg.patch_size
        N = g * g
        x = pixel_values.to(self.patch_embed.weight.dtype).view(B, C, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B * N, C * p * p)
        pos = self.pos_embed.unsqueeze(0).expand(B, N, -1).reshape(B * N, -1)
        if self.k_pad:
            x = F.pad(x, (0, self.k_pad))
        x = self.patch_embed(x.contiguous(), residual=pos.contiguous())
        cu = torch.arange(B + 1, device=x.device, dtype=torch.int32) * N
        tp = fused_tp_context(self, self.layers[0].group, cfg.hidden_size, x.shape[0], self.layers[0].spec) if len(self.layers) else None
        if tp is not None:
            x = fused_tp_blocks(tp, list(self.layers), x, None, [(cu, N)] * len(self.layers))
        else:
            for layer in self.layers:
                x = layer(x, None, cu, N)
        if self.post_layernorm is not None:
            x = self.post_layernorm(x)
        return x.view(B, N, -1)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """Names below ``vision_model.`` (``embeddings.*``, ``encoder.layers.N.*``, ``post_layernorm.*``)."""
        loaded: set[str] = set()
        for name, t in weights:
            p = name.split(".")
            leaf = p[-1]
            if name.startswith("embeddings.patch_embedding."):
                if leaf == "weight":
                    self.patch_embed.weight.data[:, : self.k_raw].copy_(t.reshape(t.shape[0], -1))
                else:
                    self.patch_embed.load(bias=t)
            elif name == "embeddings.position_embedding.weight":
                self.pos_embed.data.copy_(t)
            elif p[0] == "encoder" and p[1] == "layers":
                i = int(p[2])
                if i >= len(self.layers):
                    loaded.add(name)  # a layer above the feature tap: not needed
                    continue
                blk: EncoderBlock = self.layers[i]
                sub = ".".join(p[3:-1])
                if sub == "layer_norm1":
                    blk.load_norm(1, leaf, t)
                elif sub == "layer_norm2":
                    blk.load_norm(2, leaf, t)
                elif sub in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                    blk.qkv.load(sub[-6], **{leaf: t})
                elif sub == "self_attn.out_proj":
                    blk.proj.load(**{leaf: t})
                elif sub in ("mlp.fc1", "mlp.fc2"):
                    blk.load_mlp(sub[-3:], leaf, t)
                else:
                    continue
            elif p[0] == "post_layernorm":
                if self.post_layernorm is None:
                    loaded.add(name)
                    continue
                getattr(self.post_layernorm, leaf).data.copy_(t)
            else:
                continue  # pooling head etc.
            loaded.add(name)
        return loaded


# ------------------------------------------------------------------------------------------------
# Gemma-3
# ------------------------------------------------------------------------------------------------
@dataclass
class Gemma3VisionConfig:
    vision: SiglipConfig = field(default_factory=SiglipConfig)
    text_hidden_size: int = 2560
    mm_tokens_per_image: int = 256

    @classmethod
    def from_hf(cls, cfg: dict) -> "Gemma3VisionConfig":
        return cls(SiglipConfig.from_hf(cfg.get("vision_config", {})), int(cfg.get("text_config", {}).get("hidden_size", 2560)),
                   int(cfg.get("mm_tokens_per_image", 256)))


class Gemma3Projector(nn.Module):
    """Average-pool the patch grid to ``mm_tokens_per_image`` tokens, Gemma RMSNorm, project to the LLM width."""

    def __init__(self, cfg: Gemma3VisionConfig, device):
        super().__init__()
        v = cfg.vision
        self.side = v.image_size // v.patch_size
        self.tokens_side = int(cfg.mm_tokens_per_image ** 0.5)
        self.kernel = self.side // self.tokens_side
        self.norm = RMSNorm(v.hidden_size, v.layer_norm_eps, gemma=True, device=device)
        self.proj = Linear(v.hidden_size, cfg.text_hidden_size, bias=False, device=device)

    def forward(self, feats: torch.Tensor) -> torch.Tensor:
        B, N, H = feats.shape
        k, ts = self.kernel, self.tokens_side
        pooled = feats.view(B, ts, k, ts, k, H).float().mean(dim=(2, 4)).to(feats.dtype).reshape(B * ts * ts, H)
        return self.proj(self.norm(pooled)).view(B, ts * ts, -1)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded = set()
        for name, t in weights:
            if name == "mm_input_projection_weight":
                self.proj.load(weight=t.t())
            elif name == "mm_soft_emb_norm.weight":
                self.norm.weight.data.copy_(t)
            else:
                continue
            loaded.add(name)
        return loaded


class Gemma3VisionEncoder(nn.Module):
    """``forward("image", adapter_name, {"pixel_values": [[n_i, 3, S, S]], "num_crops": [...]})``; ``adapter_name`` is
    the model id of the Gemma-3 variant whose projector is applied."""

    modalities = ("image",)

    def __init__(self, cfg: Gemma3VisionConfig, group: ParallelGroup | None = None, device="cpu", model_id: str | None = None):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        self.vision_tower = SiglipVisionTower(cfg.vision, self.group, device)
        self.projectors = nn.ModuleDict()
        self.default_adapter = model_id or "default"
        self.add_adapter(self.default_adapter, cfg)

    @staticmethod
    def _key(name: str) -> str:
        return name.replace(".", "_").replace("/", "__")

    def add_adapter(self, name: str, cfg: Gemma3VisionConfig | dict, weights: Iterable[tuple[str, torch.Tensor]] | None = None):
        if isinstance(cfg, dict):
            cfg = Gemma3VisionConfig.from_hf(cfg)
        proj = Gemma3Projector(cfg, self.device if len(self.projectors) else self.vision_tower.pos_embed.device)
        if self.vision_tower.pos_embed.dtype == torch.float32:
            proj.float()
        if weights is not None:
            proj.load_weights(weights)
        self.projectors[self._key(name)] = proj
        return proj

    @property
    def dtype(self) -> torch.dtype:
        return self.vision_tower.pos_embed.dtype

    @property
    def device(self) -> torch.device:
        return self.vision_tower.pos_embed.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return (1, 256)  # rows are sent in slots of 256 elements; every Gemma-3 width is a multiple of it

    @torch.inference_mode()
    def forward(self, modality: str, adapter_name: str | None, batch: dict[str, list]) -> list[torch.Tensor]:
        if modality != "image":
            raise ValueError(f"unsupported modality {modality}")
        key = self._key(adapter_name or self.default_adapter)
        if key not in self.projectors:
            raise ValueError(f"no projector loaded for {adapter_name}")
        pix = [p.reshape(-1, *p.shape[-3:]) for p in batch["pixel_values"]]
        counts = [p.shape[0] for p in pix]
        feats = self.vision_tower(torch.cat(pix).to(self.device))
        emb = self.projectors[key](feats)
        return [e.flatten(0, 1) for e in emb.split(counts)]

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        tower, proj = [], []
        for full, t in weights:
            name = full[len("model."):] if full.startswith("model.") else full
            if name.startswith("vision_tower.vision_model."):
                tower.append((full, name[len("vision_tower.vision_model."):], t))
            elif name.startswith("multi_modal_projector."):
                proj.append((full, name[len("multi_modal_projector."):], t))
        ok_t = self.vision_tower.load_weights((n, t) for _, n, t in tower)
        ok_p = self.projectors[self._key(self.default_adapter)].load_weights((n, t) for _, n, t in proj)
        return {f for f, n, _ in tower if n in ok_t} | {f for f, n, _ in proj if n in ok_p}


# ------------------------------------------------------------------------------------------------
# LLaVA-OneVision
# ------------------------------------------------------------------------------------------------
@dataclass
class LlavaOnevisionVisionConfig:
    vision: SiglipConfig = field(default_factory=lambda: SiglipConfig(image_size=384, num_hidden_layers=26))
    text_hidden_size: int = 3584
    image_grid_pinpoints: list[list[int]] = field(default_factory=lambda: [[384 * a, 384 * b] for a in range(1, 7) for b in range(1, 7)])
    vision_feature_layer: int = -1
    vision_aspect_ratio: str = "anyres_max_9"
    projector_hidden_act: str = "gelu"

    @classmethod
    def from_hf(cls, cfg: dict) -> "LlavaOnevisionVisionConfig":
        kw = {k: cfg[k] for k in ("image_grid_pinpoints", "vision_feature_layer", "vision_aspect_ratio", "projector_hidden_act") if k in cfg}
        return cls(SiglipConfig.from_hf(cfg.get("vision_config", {})), int(cfg.get("text_config", {}).get("hidden_size", 3584)), **kw)


def select_best_resolution(original_size: tuple[int, int], resolutions: list[list[int]]) -> tuple[int, int]:
    """The tiling ``(height, width)`` that keeps most of the image's pixels while wasting the least area."""
    oh, ow = original_size
    best, best_eff, best_waste = None, 0, float("inf")
    for h, w in resolutions:
        scale = min(w / ow, h / oh)
        dw, dh = int(ow * scale), int(oh * scale)
        eff = min(dw * dh, ow * oh)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (h, w), eff, waste
    return best


def unpad_features(x: torch.Tensor, original_size: tuple[int, int]) -> torch.Tensor:
    """``x`` [C, H, W] covers a letter-boxed image: cut the rows or columns that are only padding."""
    oh, ow = original_size
    ch, cw = x.shape[1:]
    if ow / oh > cw / ch:
        new_h = int(round(oh * (cw / ow), 7))
        pad = (ch - new_h) // 2
        return x[:, pad: ch - pad, :]
    new_w = int(round(ow * (ch / oh), 7))
    pad = (cw - new_w) // 2
    return x[:, :, pad: cw - pad]


class LlavaOnevisionEncoder(nn.Module):
    modalities = ("image", "video")

    def __init__(self, cfg: LlavaOnevisionVisionConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        v = cfg.vision
        layer = cfg.vision_feature_layer
        n_layers = v.num_hidden_layers + layer + 1 if layer < 0 else layer
        self.vision_tower = SiglipVisionTower(v, self.group, device, num_layers=n_layers, post_norm=False)
        self.linear_1 = Linear(v.hidden_size, cfg.text_hidden_size, device=device)
        self.linear_2 = Linear(cfg.text_hidden_size, cfg.text_hidden_size, device=device)
        self.image_newline = _param(cfg.text_hidden_size, device=device, dtype=torch.bfloat16)

    @property
    def dtype(self) -> torch.dtype:
        return self.image_newline.dtype

    @property
    def device(self) -> torch.device:
        return self.image_newline.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return (1, self.cfg.text_hidden_size)

    def _project(self, pixel_values: torch.Tensor) -> torch.Tensor:
        f = self.vision_tower(pixel_values.to(self.device))
        B, N, H = f.shape
        y = self.linear_2(self.linear_1(f.view(B * N, H), act=HF_ACT[self.cfg.projector_hidden_act]))
        return y.view(B, N, -1)

    def pack_image(self, feats: torch.Tensor, image_size: tuple[int, int]) -> torch.Tensor:
        """``feats`` [tiles, N, D] (tile 0 = the whole image resized) -> packed rows with a newline per grid row."""
        cfg = self.cfg
        side = cfg.vision.image_size // cfg.vision.patch_size
        nl = self.image_newline.to(feats.dtype)
        if feats.shape[0] == 1:
            return torch.cat([feats[0], nl[None]], dim=0)
        base, tiles = feats[0], feats[1:]
        bh, bw = select_best_resolution(image_size, cfg.image_grid_pinpoints)
        gh, gw = bh // cfg.vision.image_size, bw // cfg.vision.image_size
        x = tiles.view(gh, gw, side, side, -1).permute(4, 0, 2, 1, 3).contiguous().flatten(1, 2).flatten(2, 3)
        x = unpad_features(x, image_size)
        max_tiles = int(cfg.vision_aspect_ratio.replace("anyres_max_", ""))
        _, h, w = x.shape
        ratio = math.sqrt(h * w / (max_tiles * side ** 2))
        if ratio > 1.1:
            x = F.interpolate(x[None].float(), [int(h // ratio), int(w // ratio)], mode="bilinear")[0].to(feats.dtype)
        x = torch.cat([x, nl[:, None, None].expand(-1, x.shape[1], 1)], dim=-1)
        return torch.cat([base, x.flatten(1, 2).transpose(0, 1)], dim=0)

    @torch.inference_mode()
    def forward(self, modality: str, adapter_name: str | None, batch: dict[str, list]) -> list[torch.Tensor]:
        if modality == "image":
            pix = [p.reshape(-1, *p.shape[-3:]) for p in batch["pixel_values"]]
            sizes = [tuple(int(v) for v in torch.as_tensor(s).reshape(-1)[:2].tolist()) for s in batch["image_sizes"]]
            feats = self._project(torch.cat(pix)).split([p.shape[0] for p in pix])
            return [self.pack_image(f, s) for f, s in zip(feats, sizes)]
        if modality == "video":
            outs = []
            side = self.cfg.vision.image_size // self.cfg.vision.patch_size
            for frames in batch["pixel_values_videos"]:
                frames = frames.reshape(-1, *frames.shape[-3:])
                f = self._project(frames)  # [T, N, D]
                T, _, D = f.shape
                g = f.view(T, side, side, D).permute(0, 3, 1, 2).float()
                g = F.interpolate(g, size=[math.ceil(side / 2)] * 2, mode="bilinear").permute(0, 2, 3, 1).reshape(-1, D)
                outs.append(torch.cat([g.to(f.dtype), self.image_newline.to(f.dtype)[None]], dim=0))
            return outs
        raise ValueError(f"unsupported modality {modality}")

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded: set[str] = set()
        tower = []
        for name, t in weights:
            n = name[len("model."):] if name.startswith("model.") else name
            if n.startswith("vision_tower.vision_model."):
                tower.append((name, n[len("vision_tower.vision_model."):], t))
            elif n.startswith("multi_modal_projector.linear_"):
                getattr(self, n.split(".")[1]).load(**{n.split(".")[-1]: t})
                loaded.add(name)
            elif n == "image_newline":
                self.image_newline.data.copy_(t)
                loaded.add(name)
        ok = self.vision_tower.load_weights((n, t) for _, n, t in tower)
        loaded |= {full for full, n, _ in tower if n in ok}
        return loaded
