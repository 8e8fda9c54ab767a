"""Qwen2.5-VL vision tower (encoder side of Qwen2.5-VL-3B/7B/32B/72B).

Same math and checkpoint names as the reference tower
(python/cornserve/task_executors/eric/models/qwen2_5_vl.py:181-483): Conv3d patch embed applied to
pre-flattened patches, 2-D rotary embedding, window attention with periodic full-attention blocks,
RMSNorm + SwiGLU blocks, 2x2 patch merger.  Differences that matter on B200:

* one launch per fused step: qkv GEMM(+bias), in-place rotary on q|k, var-len tcgen05 attention,
  out-proj GEMM with bias+residual epilogue, gate/up GEMM with the SwiGLU product in its epilogue,
  down GEMM with bias+residual epilogue;
* tensor parallelism shards *heads* for attention, so no all-gather of qkv is needed (the reference
  gathers the full qkv and re-slices it because its fused qkv weight is sharded by rows);
* window / rotary index building is vectorised NumPy without device syncs.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable

import numpy as np
import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group
from .layers import (ColumnParallelLinear, Linear, MergedColumnParallelLinear, QKVParallelLinear, RMSNorm,
                     RowParallelLinear)


@dataclass
class Qwen25VisionConfig:
    depth: int = 32
    hidden_size: int = 1280
    num_heads: int = 16
    intermediate_size: int = 3420
    in_channels: int = 3
    patch_size: int = 14
    temporal_patch_size: int = 2
    spatial_merge_size: int = 2
    window_size: int = 112
    fullatt_block_indexes: list[int] = field(default_factory=lambda: [7, 15, 23, 31])
    out_hidden_size: int = 3584
    rms_norm_eps: float = 1e-6
    hidden_act: str = "silu"

    @classmethod
    def from_hf(cls, cfg: dict) -> "Qwen25VisionConfig":
        v = cfg.get("vision_config", cfg)
        keys = cls.__dataclass_fields__.keys()
        return cls(**{k: v[k] for k in keys if k in v})

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads

    @property
    def patch_dim(self) -> int:
        return self.in_channels * self.temporal_patch_size * self.patch_size * self.patch_size


# ------------------------------------------------------------------------------------------------
# host-side index building (no device syncs)
# ------------------------------------------------------------------------------------------------
def rot_pos_ids(grid_thw: np.ndarray, merge: int) -> np.ndarray:
    """(h, w) position of every patch in merge-block order: ``[L, 2]``."""
    out = []
    for t, h, w in grid_thw.tolist():
        hp = np.broadcast_to(np.arange(h)[:, None], (h, w))
        wp = np.broadcast_to(np.arange(w)[None, :], (h, w))

        def blk(a):
            return a.reshape(h // merge, merge, w // merge, merge).transpose(0, 2, 1, 3).reshape(-1)

        ids = np.stack([blk(hp), blk(wp)], axis=-1)
        out.append(np.tile(ids, (t, 1)))
    return np.concatenate(out, axis=0)


def window_index(grid_thw: np.ndarray, window: int, merge: int, patch: int) -> tuple[np.ndarray, np.ndarray]:
    """Permutation of merged cells into window order and the window boundaries (in patch tokens).

    Returns ``(index [L/merge^2], cu_window_seqlens [num_windows + 1])``.
    """
    cell = window // merge // patch  # merged cells per window side
    unit = merge * merge
    index, cu = [], [0]
    base = 0
    for t, h, w in grid_thw.tolist():
        gh, gw = h // merge, w // merge
        nh, nw = -(-gh // cell), -(-gw // cell)
        ids = np.full((t, nh * cell, nw * cell), -1, dtype=np.int64)
        ids[:, :gh, :gw] = np.arange(t * gh * gw).reshape(t, gh, gw)
        ids = ids.reshape(t, nh, cell, nw, cell).transpose(0, 1, 3, 2, 4).reshape(t * nh * nw, cell * cell)
        valid = ids >= 0
        counts = valid.sum(axis=1)
        index.append(ids[valid] + base)
        ends = np.cumsum(counts[counts > 0]) * unit + cu[-1]
        cu.extend(ends.tolist())
        base += t * gh * gw
    return np.concatenate(index), np.asarray(cu, dtype=np.int32)


def pack_windows(cu_win: np.ndarray, limit: int = 128) -> tuple[np.ndarray, np.ndarray, np.ndarray]:
    """Groups consecutive attention windows (tokens are already in window order) into runs of at most ``limit`` tokens,
    so that short windows share one 128-row attention tile.  Returns ``(cu_groups, lo [L], hi [L])``: the group
    boundaries and, for every token, the key range of its own window."""
    sizes = np.diff(cu_win)
    cu = [0]
    run = 0
    for n in sizes.tolist():
        if run and run + n > limit:
            cu.append(cu[-1] + run)
            run = 0
        run += n
    cu.append(cu[-1] + run)
    lo = np.repeat(cu_win[:-1], sizes).astype(np.int32)
    hi = np.repeat(cu_win[1:], sizes).astype(np.int32)
    return np.asarray(cu, dtype=np.int32), lo, hi


class VisionBlock(nn.Module):
    def __init__(self, cfg: Qwen25VisionConfig, group: ParallelGroup, device):
        super().__init__()
        H, d = cfg.hidden_size, cfg.head_dim
        self.cfg, self.group = cfg, group
        self.norm1 = RMSNorm(H, cfg.rms_norm_eps, device=device)
        self.norm2 = RMSNorm(H, cfg.rms_norm_eps, device=device)
        self.qkv = QKVParallelLinear(H, d, cfg.num_heads, cfg.num_heads, bias=True, group=group, device=device)
        self.proj = RowParallelLinear(H, H, bias=True, group=group, device=device)
        self.gate_up = MergedColumnParallelLinear(H, cfg.intermediate_size, bias=True, group=group, device=device)
        self.down = RowParallelLinear(cfg.intermediate_size, H, bias=True, group=group,
                                      in_padded=self.gate_up.inter_padded, device=device)
        self.heads_local = self.qkv.heads_local

    def forward(self, x: torch.Tensor, cs: torch.Tensor, cu: torch.Tensor, max_len: int, bounds=None) -> torch.Tensor:
        T = x.shape[0]
        hl, d = self.heads_local, self.cfg.head_dim
        qkv = self.qkv(self.norm1(x))  # [T, 3 * hl * d] = q heads | k heads | v heads
        qk = qkv[:, : 2 * hl * d].view(T, 2 * hl, d)
        ops.rope_(qk, cs)
        q = qkv[:, : hl * d].view(T, hl, d)
        k = qkv[:, hl * d: 2 * hl * d].view(T, hl, d)
        v = qkv[:, 2 * hl * d:].view(T, hl, d)
        a = ops.attention_varlen(q, k, v, cu, cu, max_len, row_bounds=bounds)
        x = self.proj(a.view(T, hl * d), residual=x)
        h = self.gate_up(self.norm2(x), act=self.cfg.hidden_act)
        return self.down(h, residual=x)


class PatchMerger(nn.Module):
    def __init__(self, cfg: Qwen25VisionConfig, group: ParallelGroup, device):
        super().__init__()
        self.unit = cfg.spatial_merge_size ** 2
        self.inner = cfg.hidden_size * self.unit
        self.ln_q = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device)
        self.fc1 = ColumnParallelLinear(self.inner, self.inner, bias=True, group=group, device=device)
        self.fc2 = RowParallelLinear(self.inner, cfg.out_hidden_size, bias=True, group=group,
                                     in_padded=self.fc1.out_padded, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x = self.ln_q(x).view(-1, self.inner)
        return self.fc2(self.fc1(x, act="gelu"))


class Qwen25VisionTransformer(nn.Module):
    """``forward(modality, adapter_name, batch)`` returns one ``[tokens, out_hidden]`` tensor per item."""

    modalities = ("image", "video")

    def __init__(self, cfg: Qwen25VisionConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        self.dev = torch.device(device)
        self.patch_embed = Linear(cfg.patch_dim, cfg.hidden_size, bias=False, device=device)
        self.blocks = nn.ModuleList([VisionBlock(cfg, self.group, device) for _ in range(cfg.depth)])
        self.merger = PatchMerger(cfg, self.group, device)
        d = cfg.head_dim
        self.inv_freq = 1.0 / (10000.0 ** (np.arange(0, d // 2, 2, dtype=np.float64) / (d // 2)))

    # -- interface used by the Eric worker -------------------------------------------------------
    @property
    def dtype(self) -> torch.dtype:
        return self.patch_embed.weight.dtype

    @property
    def device(self) -> torch.device:
        return self.patch_embed.weight.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return (1, self.cfg.out_hidden_size)

    def rotary_table(self, grid_thw: np.ndarray) -> np.ndarray:
        pos = rot_pos_ids(grid_thw, self.cfg.spatial_merge_size)  # [L, 2]
        ang = pos[:, :, None].astype(np.float64) * self.inv_freq[None, None, :]  # [L, 2, d/4]
        ang = ang.reshape(pos.shape[0], -1)  # [L, d/2] = h freqs then w freqs
        return np.stack([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)  # [L, 2, d/2]

    def forward(self, modality: str, adapter_name: str | None, batch: dict[str, list[torch.Tensor]]) -> list[torch.Tensor]:
        if modality == "image":
            pixels, grids = batch["pixel_values"], batch["image_grid_thw"]
        elif modality == "video":
            pixels, grids = batch["pixel_values_videos"], batch["video_grid_thw"]
        else:
            raise ValueError(f"unsupported modality {modality}")
        grid = np.concatenate([np.asarray(g, dtype=np.int64).reshape(-1, 3) for g in grids], axis=0)
        per_item = [int(np.prod(np.asarray(g, dtype=np.int64).reshape(-1, 3), axis=1).sum()) for g in grids]
        x = torch.cat([p.reshape(-1, self.cfg.patch_dim) for p in pixels], dim=0)
        out = self.encode(x, grid)
        unit = self.cfg.spatial_merge_size ** 2
        return list(out.split([n // unit for n in per_item], dim=0))

    def encode(self, pixel_patches: torch.Tensor, grid_thw: np.ndarray) -> torch.Tensor:
        cfg = self.cfg
        dev = self.device
        unit = cfg.spatial_merge_size ** 2
        x = pixel_patches.to(device=dev, dtype=self.dtype, non_blocking=True)
        L = x.shape[0]
        widx_d, cs_d, cu_win_d, cu_full_d, max_win, max_full, win_bounds = self._index_tables(grid_thw, L)

        x = self.patch_embed(x)
        x = ops.gather_rows(x.view(L // unit, unit * cfg.hidden_size), widx_d).view(L, cfg.hidden_size)
        att = [(cu_full_d, max_full, None) if i in cfg.fullatt_block_indexes else (cu_win_d, max_win, win_bounds)
               for i in range(len(self.blocks))]
        tp = self._fused_tp(L)
        if tp is not None:
            y = self._blocks_fused(tp, x, cs_d, att)
        else:
            for blk, (cu, mx, bounds) in zip(self.blocks, att):
                x = blk(x, cs_d, cu, mx, bounds)
            y = self.merger(x)  # [L/unit, out] in window order
        out = torch.empty_like(y)
        ops.scatter_rows_(out, widx_d, y)  # undo the window permutation
        return out

    def _index_tables(self, grid_thw: np.ndarray, L: int):
        """Window permutation, rotary table and attention boundaries of a batch, on the device.  Built on the host
        with NumPy (no device synchronisation) and kept per grid signature: serving traffic repeats a few shapes."""
        cfg, dev = self.cfg, self.device
        key = (str(dev), grid_thw.astype(np.int64).tobytes())
        cache = self.__dict__.setdefault("_tables", {})
        hit = cache.get(key)
        if hit is not None:
            return hit
        unit = cfg.spatial_merge_size ** 2
        widx, cu_win = window_index(grid_thw, cfg.window_size, cfg.spatial_merge_size, cfg.patch_size)
        cs = self.rotary_table(grid_thw).reshape(L // unit, unit, 2, -1)[widx].reshape(L, 2, -1)
        frames = np.repeat(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
        cu_full = np.concatenate([[0], np.cumsum(frames)]).astype(np.int32)
        to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev, non_blocking=True)  # noqa: E731
        bounds = None
        if dev.type == "cuda" and int(np.diff(cu_win).max()) <= 64:
            # windows of at most 64 tokens: two or more fit into one 128-row attention tile
            cu_pack, lo, hi = pack_windows(cu_win)
            cu_win, bounds = cu_pack, (to_dev(lo), to_dev(hi))
        out = (to_dev(widx.astype(np.int32)), to_dev(cs), to_dev(cu_win), to_dev(cu_full), int(np.diff(cu_win).max()),
               int(frames.max()), bounds)
        if len(cache) >= 64:
            cache.pop(next(iter(cache)))
        cache[key] = out
        return out

    # -- tensor-parallel path without library collectives ------------------------------------------------
    def _fused_tp(self, rows: int):
        """The peer-memory context for ``rows`` patch tokens, or ``None`` when the plain path applies (one GPU, no
        fabric, or too few rows to give every rank a 128-row block)."""
        g = self.group
        if g.size == 1 or g.fabric is None or self.device.type != "cuda" or rows < 128 * g.size or rows % 4:
            return None
        from ..parallel.fused import FusedEncoderTP

        tp = getattr(self, "_tp_ctx", None)
        if tp is None or tp.S_cap < rows:
            # sized by the first batch that needs it (collective: all ranks run the same batches)
            tp = self._tp_ctx = FusedEncoderTP(g, self.cfg.hidden_size, max(rows, 40960))
        return tp

    def _blocks_fused(self, tp, x: torch.Tensor, cs: torch.Tensor, att: list) -> torch.Tensor:
        """All blocks and the merger with row-sharded activations between GEMMs.  ``x`` is the full (replicated)
        patch-embedding output; every rank keeps only its rows of the residual stream from here on."""
        cfg = self.cfg
        T = x.shape[0]
        tp.begin(T)
        lo, hi = tp.row_range
        xs = x[lo:hi].contiguous()
        eps = cfg.rms_norm_eps
        blocks = list(self.blocks)
        tp.reduce_norm_push(bias=None, residual=xs, norm_w=blocks[0].norm1.weight, eps=eps, dst=0, reduce=False)
        for i, (blk, (cu, mx, bounds)) in enumerate(zip(blocks, att)):
            hl, d = blk.heads_local, cfg.head_dim
            qkv = tp.gemm_gathered(0, blk.qkv.weight, blk.qkv.bias)
            ops.rope_(qkv[:, : 2 * hl * d].view(T, 2 * hl, d), cs)
            q, k, v = (qkv[:, j * hl * d:(j + 1) * hl * d].view(T, hl, d) for j in range(3))
            a = ops.attention_varlen(q, k, v, cu, cu, mx, row_bounds=bounds)
            tp.gemm_push(a.view(T, hl * d), blk.proj.weight)
            xs = tp.reduce_norm_push(bias=blk.proj.bias, residual=xs, norm_w=blk.norm2.weight, eps=eps, dst=1)
            h = tp.gemm_gathered(1, blk.gate_up.weight, blk.gate_up.bias, act=cfg.hidden_act, swiglu=True)
            tp.gemm_push(h, blk.down.weight)
            last = i + 1 == len(blocks)
            nxt = self.merger.ln_q.weight if last else blocks[i + 1].norm1.weight
            xs = tp.reduce_norm_push(bias=blk.down.bias, residual=xs, norm_w=nxt, eps=eps, dst=2 if last else 0,
                                     gather_chunk=128 * self.merger.unit if last else 128)
        m = self.merger
        h = tp.gemm_gathered(2, m.fc1.weight, m.fc1.bias, act="gelu", a_rpr=m.unit)
        return m.fc2(h)  # small: [T/4, out] partial sums reduced by the library collective

    # -- checkpoint loading (HF names, prefix "visual." already stripped) ---------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded: set[str] = set()
        for name, t in weights:
            parts = name.split(".")
            try:
                if name == "patch_embed.proj.weight":
                    self.patch_embed.load(t.reshape(self.cfg.hidden_size, -1))
                elif parts[0] == "blocks":
                    blk: VisionBlock = self.blocks[int(parts[1])]
                    sub, leaf = ".".join(parts[2:-1]), parts[-1]
                    kw = {leaf: t}
                    if sub == "norm1":
                        blk.norm1.weight.data.copy_(t)
                    elif sub == "norm2":
                        blk.norm2.weight.data.copy_(t)
                    elif sub == "attn.qkv":
                        blk.qkv.load_fused(**kw)
                    elif sub in ("attn.q", "attn.k", "attn.v"):  # Qwen2.5-Omni stores the projections separately
                        blk.qkv.load(sub[-1], **kw)
                    elif sub == "attn.proj":
                        blk.proj.load(**kw)
                    elif sub == "mlp.gate_proj":
                        blk.gate_up.load("gate", **kw)
                    elif sub == "mlp.up_proj":
                        blk.gate_up.load("up", **kw)
                    elif sub == "mlp.down_proj":
                        blk.down.load(**kw)
                    else:
                        continue
                elif name == "merger.ln_q.weight":
                    self.merger.ln_q.weight.data.copy_(t)
                elif parts[0] == "merger" and parts[1] == "mlp":
                    layer = self.merger.fc1 if parts[2] == "0" else self.merger.fc2
                    layer.load(**{parts[-1]: t})
                else:
                    continue
            except Exception as e:  # pragma: no cover - surfaces shape mismatches with the tensor name
                raise RuntimeError(f"failed to load {name}: {e}") from e
            loaded.add(name)
        return loaded
