"""Qwen3-VL vision tower, also the vision half of Qwen3-VL-MoE and Qwen3-Omni (reference:
python/cornserve/task_executors/eric/models/qwen3_vl.py:25-461 and qwen3_omni_moe.py:429-495): patch embedding with
bias, a learned position table interpolated bilinearly onto the patch grid (one kernel: gather the four neighbours,
weight, add), 2-D rotary LayerNorm blocks with a GELU-tanh MLP, the 2x2 merger, and "deep-stack" mergers that tap
intermediate layers.  The output rows are ``[merger | deep-stack 0 | deep-stack 1 | ...]`` along the channel
dimension, which is how the language model consumes them."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable

import numpy as np
import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group
from .layers import Linear, _param
from .qwen2_vl import PatchMerger
from .vit import HF_ACT, BlockSpec, EncoderBlock, bilinear_pos_indices, frame_cu_seqlens, rotary_table_2d


@dataclass
class Qwen3VisionConfig:
    depth: int = 27
    hidden_size: int = 1152
    num_heads: int = 16
    intermediate_size: int = 4304
    in_channels: int = 3
    patch_size: int = 16
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    out_hidden_size: int = 3584
    num_position_embeddings: int = 2304
    deepstack_visual_indexes: list[int] = field(default_factory=lambda: [8, 16, 24])
    hidden_act: str = "gelu_pytorch_tanh"

    @classmethod
    def from_hf(cls, cfg: dict) -> "Qwen3VisionConfig":
        v = cfg.get("vision_config") or (cfg.get("thinker_config") or {}).get("vision_config") or cfg
        return cls(**{k: v[k] for k in cls.__dataclass_fields__ if k in v})

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size ** 2


class Qwen3VisionTransformer(nn.Module):
    modalities = ("image", "video")

    def __init__(self, cfg: Qwen3VisionConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        H = cfg.hidden_size
        self.patch_embed = Linear(cfg.patch_dim, H, bias=True, device=device)
        self.pos_embed = _param(cfg.num_position_embeddings, H, device=device, dtype=torch.bfloat16)
        self.side = int(cfg.num_position_embeddings ** 0.5)
        spec = BlockSpec(H, cfg.num_heads, cfg.intermediate_size, norm="layer", eps=1e-6, act=HF_ACT[cfg.hidden_act])
        self.blocks = nn.ModuleList([EncoderBlock(spec, self.group, device) for _ in range(cfg.depth)])
        self.merger = PatchMerger(H, cfg.out_hidden_size, cfg.spatial_merge_size, self.group, device)
        self.deepstack = nn.ModuleList([PatchMerger(H, cfg.out_hidden_size, cfg.spatial_merge_size, self.group, device,
                                                    postshuffle=True) for _ in cfg.deepstack_visual_indexes])

    @property
    def dtype(self) -> torch.dtype:
        return self.patch_embed.weight.dtype

    @property
    def device(self) -> torch.device:
        return self.patch_embed.weight.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return (1, self.cfg.out_hidden_size * (1 + len(self.cfg.deepstack_visual_indexes)))

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
        idx, wgt = bilinear_pos_indices(grid_thw, self.side, cfg.spatial_merge_size)
        cs = torch.from_numpy(rotary_table_2d(grid_thw, cfg.spatial_merge_size, cfg.hidden_size // cfg.num_heads)).to(dev)
        cu, max_len = frame_cu_seqlens(grid_thw)
        cu = torch.from_numpy(cu).to(dev)
        x = self.patch_embed(x)
        ops.bilinear_embed_add_(x, self.pos_embed, torch.from_numpy(idx).to(dev), torch.from_numpy(wgt).to(dev))
        taps: list[torch.Tensor] = []
        for i, blk in enumerate(self.blocks):
            x = blk(x, cs, cu, max_len)
            if i in cfg.deepstack_visual_indexes:
                taps.append(self.deepstack[cfg.deepstack_visual_indexes.index(i)](x))
        return torch.cat([self.merger(x), *taps], dim=1)

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded: set[str] = set()
        for name, t in weights:
            p = name.split(".")
            leaf = p[-1]
            if name.startswith("patch_embed.proj."):
                self.patch_embed.load(**{leaf: t.reshape(self.cfg.hidden_size, -1) if leaf == "weight" else t})
            elif name == "pos_embed.weight":
                self.pos_embed.data.copy_(t)
            elif p[0] == "blocks":
                blk: EncoderBlock = self.blocks[int(p[1])]
                sub = ".".join(p[2:-1])
                if sub in ("norm1", "norm2"):
                    blk.load_norm(int(sub[-1]), leaf, t)
                elif sub == "attn.qkv":
                    blk.qkv.load_fused(**{leaf: t})
                elif sub == "attn.proj":
                    blk.proj.load(**{leaf: t})
                elif sub in ("mlp.linear_fc1", "mlp.linear_fc2"):
                    blk.load_mlp(sub[-3:], leaf, t)
                else:
                    continue
            elif p[0] in ("merger", "deepstack_merger_list"):
                m = self.merger if p[0] == "merger" else self.deepstack[int(p[1])]
                part = {"norm": "norm", "linear_fc1": "fc1", "linear_fc2": "fc2"}.get(p[-2])
                if part is None:
                    continue
                m.load(part, leaf, t)
            else:
                continue
            loaded.add(name)
        return loaded
