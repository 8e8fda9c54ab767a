"""InternVL vision encoder: InternViT tower + pixel-shuffle + MLP projector (reference:
python/cornserve/task_executors/eric/models/layers/intern_vit.py:26-351 and models/internvl.py:30-604; checkpoint
names are those of the ``internvl_chat`` models: ``vision_model.*`` and ``mlp1.*``).

Every 448x448 tile becomes a class token plus 1024 patch tokens; blocks use LayerNorm or RMSNorm, an optional
RMSNorm of q and k over the full hidden width, learned layer scales (carried in the GEMM epilogue's gate operand)
and a GELU MLP.  The 2x2 pixel shuffle quarters the token count before the projector.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

import torch
from torch import nn

from ..parallel.state import ParallelGroup, single_group
from .layers import LayerNorm, Linear, _param
from .vit import HF_ACT, BlockSpec, EncoderBlock


@dataclass
class InternVLVisionConfig:
    hidden_size: int = 1024
    intermediate_size: int = 4096
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    image_size: int = 448
    patch_size: int = 14
    qkv_bias: bool = True
    qk_normalization: bool = False
    norm_type: str = "layer_norm"
    layer_norm_eps: float = 1e-6
    hidden_act: str = "gelu"
    select_layer: int = -1
    downsample_ratio: float = 0.5
    ps_version: str = "v2"
    llm_hidden_size: int = 4096

    @classmethod
    def from_hf(cls, cfg: dict) -> "InternVLVisionConfig":
        v = cfg.get("vision_config", {})
        kw = {k: v[k] for k in cls.__dataclass_fields__ if k in v}
        for k in ("select_layer", "downsample_ratio", "ps_version"):
            if k in cfg:
                kw[k] = cfg[k]
        llm = cfg.get("llm_config") or cfg.get("text_config") or {}
        if "hidden_size" in llm:
            kw["llm_hidden_size"] = llm["hidden_size"]
        return cls(**kw)


def pixel_shuffle(x: torch.Tensor, scale: float = 0.5, version: str = "v2") -> torch.Tensor:
    """``[n, w, h, c]`` -> ``[n, w*scale, h*scale, c/scale^2]`` (space-to-depth for ``scale`` < 1)."""
    n, w, h, c = x.shape
    x = x.view(n, w, int(h * scale), int(c / scale)).permute(0, 2, 1, 3).contiguous()
    x = x.view(n, int(h * scale), int(w * scale), int(c / (scale * scale)))
    return x if version == "v1" else x.permute(0, 2, 1, 3).contiguous()


class InternVLEncoder(nn.Module):
    modalities = ("image", "video")

    def __init__(self, cfg: InternVLVisionConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        H, p = cfg.hidden_size, cfg.patch_size
        self.side = cfg.image_size // p
        self.k_raw = 3 * p * p
        self.k_pad = (-self.k_raw) % 8   # TMA rows must be multiples of 16 bytes: 588 -> 592 zero-padded columns
        self.patch_embed = Linear(self.k_raw + self.k_pad, H, bias=True, device=device)
        self.patch_embed.weight.data[:, self.k_raw:].zero_()
        self.class_embedding = _param(1, H, device=device, dtype=torch.bfloat16)
        self.position_embedding = _param(self.side ** 2 + 1, H, device=device, dtype=torch.bfloat16)
        heads = cfg.num_attention_heads
        if heads % self.group.size != 0:
            raise ValueError(f"{heads} heads cannot be split over {self.group.size} ranks (InternViT-6B has 25 heads: use 1 or 5)")
        spec = BlockSpec(H, heads, cfg.intermediate_size, norm="rms" if cfg.norm_type == "rms_norm" else "layer",
                         eps=cfg.layer_norm_eps, act=HF_ACT[cfg.hidden_act], qkv_bias=cfg.qkv_bias, layer_scale=True,
                         qk_norm=cfg.qk_normalization)
        n = cfg.num_hidden_layers + cfg.select_layer + 1 if cfg.select_layer < 0 else cfg.select_layer
        self.layers = nn.ModuleList([EncoderBlock(spec, self.group, device) for _ in range(n)])
        inner = int(H / (cfg.downsample_ratio ** 2))
        self.mlp_norm = LayerNorm(inner, 1e-5, device=device)
        self.mlp_fc1 = Linear(inner, cfg.llm_hidden_size, device=device)
        self.mlp_fc2 = Linear(cfg.llm_hidden_size, cfg.llm_hidden_size, device=device)

    @property
    def dtype(self) -> torch.dtype:
        return self.class_embedding.dtype

    @property
    def device(self) -> torch.device:
        return self.class_embedding.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return (1, self.cfg.llm_hidden_size)

    @torch.inference_mode()
    def encode_tiles(self, pixel_values: torch.Tensor) -> torch.Tensor:
        """``[B, 3, S, S]`` tiles -> ``[B, (S/p/2)^2, llm_hidden]``."""
        cfg = self.cfg
        B, C, S, _ = pixel_values.shape
        p, g = cfg.patch_size, self.side
        N = g * g
        H = cfg.hidden_size
        x = pixel_values.to(self.device, self.dtype).view(B, C, g, p, g, p).permute(0, 2, 4, 1, 3, 5).reshape(B * N, C * p * p)
        pos = self.position_embedding[1:].unsqueeze(0).expand(B, N, H).reshape(B * N, H)
        if self.k_pad:
            x = torch.nn.functional.pad(x, (0, self.k_pad))
        patches = self.patch_embed(x.contiguous(), residual=pos.contiguous()).view(B, N, H)
        cls = (self.class_embedding + self.position_embedding[:1]).expand(B, 1, H)
        x = torch.cat([cls, patches], dim=1).reshape(B * (N + 1), H)
        cu = torch.arange(B + 1, device=x.device, dtype=torch.int32) * (N + 1)
        for layer in self.layers:
            x = layer(x, None, cu, N + 1)
        x = x.view(B, N + 1, H)[:, 1:].reshape(B, g, g, H)
        x = pixel_shuffle(x, cfg.downsample_ratio, cfg.ps_version)
        x = x.reshape(-1, x.shape[-1])
        y = self.mlp_fc2(self.mlp_fc1(self.mlp_norm(x), act="gelu"))
        return y.view(B, -1, cfg.llm_hidden_size)

    def forward(self, modality: str, adapter_name: str | None, batch: dict[str, list]) -> list[torch.Tensor]:
        key = "pixel_values" if modality == "image" else "pixel_values_videos"
        if modality not in self.modalities:
            raise ValueError(f"unsupported modality {modality}")
        pix = [p.reshape(-1, *p.shape[-3:]) for p in batch[key]]
        emb = self.encode_tiles(torch.cat(pix))
        return [e.flatten(0, 1) for e in emb.split([p.shape[0] for p in pix])]

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded: set[str] = set()
        for name, t in weights:
            p = name.split(".")
            leaf = p[-1]
            if name.startswith("vision_model.embeddings."):
                if p[2] == "class_embedding":
                    self.class_embedding.data.copy_(t.reshape(1, -1))
                elif p[2] == "position_embedding":
                    self.position_embedding.data.copy_(t.reshape(-1, t.shape[-1]))
                elif p[2] == "patch_embedding":
                    if leaf == "weight":
                        self.patch_embed.weight.data[:, : self.k_raw].copy_(t.reshape(t.shape[0], -1))
                    else:
                        self.patch_embed.load(bias=t)
                else:
                    continue
            elif name.startswith("vision_model.encoder.layers."):
                i = int(p[3])
                if i >= len(self.layers):
                    loaded.add(name)
                    continue
                blk: EncoderBlock = self.layers[i]
                sub = ".".join(p[4:-1]) if len(p) > 5 else p[4]
                if sub in ("norm1", "norm2"):
                    blk.load_norm(int(sub[-1]), leaf, t)
                elif sub == "attn.qkv":
                    blk.qkv.load_fused(**{leaf: t})
                elif sub == "attn.proj":
                    blk.proj.load(**{leaf: t})
                elif sub in ("attn.q_norm", "attn.k_norm"):
                    getattr(blk, sub[-6:]).weight.data.copy_(t)
                elif sub in ("mlp.fc1", "mlp.fc2"):
                    blk.load_mlp(sub[-3:], leaf, t)
                elif p[4] in ("ls1", "ls2"):
                    getattr(blk, p[4]).data.copy_(t.reshape(1, -1))
                else:
                    continue
            elif p[0] == "mlp1":
                m = {"0": self.mlp_norm, "1": self.mlp_fc1, "3": self.mlp_fc2}.get(p[1])
                if m is None:
                    continue
                if p[1] == "0":
                    getattr(m, leaf).data.copy_(t)
                else:
                    m.load(**{leaf: t})
            else:
                continue
            loaded.add(name)
        return loaded
