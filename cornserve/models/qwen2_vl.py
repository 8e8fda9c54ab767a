"""Qwen2-VL vision tower (reference: python/cornserve/task_executors/eric/models/qwen2_vl.py:24-466): Conv3d patch
embedding applied to pre-flattened patches (one GEMM), 2-D rotary embedding, LayerNorm blocks with full attention
inside every frame and a QuickGELU MLP, and the 2x2 patch merger (LayerNorm -> Linear -> GELU -> Linear)."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

import numpy as np
import torch
from torch import nn

from ..parallel.state import ParallelGroup, single_group
from .layers import ColumnParallelLinear, LayerNorm, Linear, RowParallelLinear
from .vit import HF_ACT, BlockSpec, EncoderBlock, frame_cu_seqlens, fused_tp_blocks, fused_tp_context, rotary_table_2d


@dataclass
class Qwen2VisionConfig:
    depth: int = 32
    embed_dim: int = 1280
    num_heads: int = 16
    mlp_ratio: float = 4.0
    hidden_size: int = 3584          # width of the LLM the merger projects to
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    hidden_act: str = "quick_gelu"

    @classmethod
    def from_hf(cls, cfg: dict) -> "Qwen2VisionConfig":
        v = cfg.get("vision_config", cfg)
        kw = {k: v[k] for k in cls.__dataclass_fields__ if k in v}
        if "in_chans" in v:
            kw["in_channels"] = v["in_chans"]
        if "spatial_patch_size" in v:
            kw["patch_size"] = v["spatial_patch_size"]
        return cls(**kw)

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2


class PatchMerger(nn.Module):
    """``norm`` over the patch width (or, with ``postshuffle``, over the merged 2x2 width) -> fc1 -> GELU -> fc2."""

    def __init__(self, hidden: int, out: int, merge: int, group: ParallelGroup, device, eps: float = 1e-6,
                 postshuffle: bool = False):
        super().__init__()
        self.inner = hidden * merge * merge
        self.postshuffle = postshuffle
        self.norm = LayerNorm(self.inner if postshuffle else hidden, eps, device=device)
        self.fc1 = ColumnParallelLinear(self.inner, self.inner, group=group, device=device)
        self.fc2 = RowParallelLinear(self.inner, out, group=group, in_padded=self.fc1.out_padded, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.norm(x.view(-1, self.inner)) if self.postshuffle else self.norm(x).view(-1, self.inner)
        return self.fc2(self.fc1(x, act="gelu"))

    def load(self, part: str, leaf: str, t: torch.Tensor) -> None:
        if part == "norm":
            getattr(self.norm, leaf).data.copy_(t)
        else:
            (self.fc1 if part == "fc1" else self.fc2).load(**{leaf: t})


class Qwen2VisionTransformer(nn.Module):
    modalities = ("image", "video")

    def __init__(self, cfg: Qwen2VisionConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        H = cfg.embed_dim
        self.patch_embed = Linear(cfg.patch_dim, H, bias=False, device=device)
        spec = BlockSpec(H, cfg.num_heads, int(H * cfg.mlp_ratio), norm="layer", eps=1e-6, act=HF_ACT[cfg.hidden_act])
        self.blocks = nn.ModuleList([EncoderBlock(spec, self.group, device) for _ in range(cfg.depth)])
        self.merger = PatchMerger(H, cfg.hidden_size, cfg.spatial_merge_size, self.group, device)

    @property
    def dtype(self) -> torch.dtype:
        return self.patch_embed.weight.dtype

    @property
    def device(self) -> torch.device:
        return self.patch_embed.weight.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return (1, self.cfg.hidden_size)

    def forward(self, modality: str, adapter_name: str | None, batch: dict[str, list]) -> list[torch.Tensor]:
        key = {"image": ("pixel_values", "image_grid_thw"), "video": ("pixel_values_videos", "video_grid_thw")}.get(modality)
        if key is None:
            raise ValueError(f"unsupported modality {modality}")
        pixels, grids = batch[key[0]], batch[key[1]]
        grid = np.concatenate([np.asarray(g, dtype=np.int64).reshape(-1, 3) for g in grids], axis=0)
        per_item = [int(np.prod(np.asarray(g, dtype=np.int64).reshape(-1, 3), axis=1).sum()) for g in grids]
        x = torch.cat([p.reshape(-1, self.cfg.patch_dim) for p in pixels], dim=0)
        out = self.encode(x, grid)
        unit = self.cfg.spatial_merge_size ** 2
        return list(out.split([n // unit for n in per_item], dim=0))

    @torch.inference_mode()
    def encode(self, pixel_patches: torch.Tensor, grid_thw: np.ndarray) -> torch.Tensor:
        cfg, dev = self.cfg, self.device
        x = pixel_patches.to(device=dev, dtype=self.dtype, non_blocking=True)
        cs = torch.from_numpy(rotary_table_2d(grid_thw, cfg.spatial_merge_size, cfg.embed_dim // cfg.num_heads)).to(dev)
        cu, max_len = frame_cu_seqlens(grid_thw)
        cu = torch.from_numpy(cu).to(dev)
        x = self.patch_embed(x)
        tp = fused_tp_context(self, self.group, cfg.embed_dim, x.shape[0], self.blocks[0].spec)
        if tp is not None:
            x = fused_tp_blocks(tp, list(self.blocks), x, cs, [(cu, max_len)] * len(self.blocks))
        else:
            for blk in self.blocks:
                x = blk(x, cs, cu, max_len)
        return self.merger(x)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded: set[str] = set()
        for name, t in weights:
            p = name.split(".")
            leaf = p[-1]
            if name == "patch_embed.proj.weight":
                self.patch_embed.load(t.reshape(self.cfg.embed_dim, -1))
            elif p[0] == "blocks":
                blk: EncoderBlock = self.blocks[int(p[1])]
                sub = ".".join(p[2:-1])
                if sub in ("norm1", "norm2"):
                    blk.load_norm(int(sub[-1]), leaf, t)
                elif sub == "attn.qkv":
                    blk.qkv.load_fused(**{leaf: t})
                elif sub == "attn.proj":
                    blk.proj.load(**{leaf: t})
                elif sub in ("mlp.fc1", "mlp.fc2"):
                    blk.load_mlp(sub[-3:], leaf, t)
                else:
                    continue
            elif p[0] == "merger":
                part = {"ln_q": "norm", "mlp.0": "fc1", "mlp.2": "fc2"}.get(".".join(p[1:-1]))
                if part is None:
                    continue
                self.merger.load(part, leaf, t)
            else:
                continue
            loaded.add(name)
        return loaded
