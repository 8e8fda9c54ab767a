"""Building blocks shared by the encoder towers (vision and audio) of the model registry.

One pre-norm transformer block covers every tower the reference ships
(python/cornserve/task_executors/eric/models/{qwen2_vl,qwen3_vl,qwen2_5_omni,qwen3_omni_moe}.py and
.../layers/{siglip,intern_vit}.py): LayerNorm or RMSNorm, plain or gated MLP, optional rotary embedding,
optional learned layer scale, optional q/k normalisation over the full hidden width, packed var-len attention.
Per block: norm kernel -> fused qkv GEMM (+bias) -> in-place rotary -> tcgen05 var-len attention -> output GEMM
with bias + residual (+ layer scale) in the epilogue -> norm -> MLP GEMM(s) with the activation (and gate
product) in the epilogue -> GEMM with bias + residual.  Tensor parallelism shards heads and MLP columns.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup
from .layers import (ColumnParallelLinear, LayerNorm, MergedColumnParallelLinear, QKVParallelLinear, RMSNorm,
                     RowParallelLinear, _param)

HF_ACT = {"gelu": "gelu", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "gelu_fast": "gelu_tanh",
          "quick_gelu": "quick_gelu", "silu": "silu", "swish": "silu", "relu": "relu"}


@dataclass
class BlockSpec:
    hidden: int
    heads: int
    intermediate: int
    norm: str = "layer"            # "layer" | "rms"
    eps: float = 1e-6
    act: str = "gelu"
    gated: bool = False
    qkv_bias: bool = True
    proj_bias: bool = True
    mlp_bias: bool = True
    layer_scale: bool = False
    qk_norm: bool = False          # RMSNorm of q and k over the whole hidden width (InternViT)

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads


def make_norm(kind: str, dim: int, eps: float, device):
    return RMSNorm(dim, eps, device=device) if kind == "rms" else LayerNorm(dim, eps, device=device)


class EncoderBlock(nn.Module):
    def __init__(self, spec: BlockSpec, group: ParallelGroup, device):
        super().__init__()
        self.spec, self.group = spec, group
        H, d = spec.hidden, spec.head_dim
        self.norm1 = make_norm(spec.norm, H, spec.eps, device)
        self.norm2 = make_norm(spec.norm, H, spec.eps, device)
        self.qkv = QKVParallelLinear(H, d, spec.heads, spec.heads, bias=spec.qkv_bias, group=group, device=device)
        self.proj = RowParallelLinear(H, H, bias=spec.proj_bias, group=group, device=device)
        if spec.gated:
            self.fc1 = MergedColumnParallelLinear(H, spec.intermediate, bias=spec.mlp_bias, group=group, device=device)
            inner = self.fc1.inter_padded
        else:
            self.fc1 = ColumnParallelLinear(H, spec.intermediate, bias=spec.mlp_bias, group=group, device=device)
            inner = self.fc1.out_padded
        self.fc2 = RowParallelLinear(spec.intermediate, H, bias=spec.mlp_bias, group=group, in_padded=inner, device=device)
        self.heads_local = self.qkv.heads_local
        if spec.layer_scale:
            self.ls1 = _param(1, H, device=device, dtype=torch.bfloat16, std=1.0)
            self.ls2 = _param(1, H, device=device, dtype=torch.bfloat16, std=1.0)
        if spec.qk_norm:
            self.q_norm = RMSNorm(H, spec.eps, device=device)
            self.k_norm = RMSNorm(H, spec.eps, device=device)

    def _row_parallel(self, layer: RowParallelLinear, x, residual, scale):
        """``residual + scale * layer(x)``; the scale rides in the GEMM epilogue when there is nothing to reduce."""
        if scale is None:
            return layer(x, residual=residual)
        if self.group.size == 1:
            return ops.linear(x, layer.weight, layer.bias, gate=scale, gate_rows_per_batch=x.shape[0], residual=residual)
        y = layer(x)
        return torch.addcmul(residual, y, scale.to(y.dtype))

    def _qk_norm_full(self, qkv: torch.Tensor, T: int) -> None:
        """RMSNorm of q and of k over all heads (in place).  Under tensor parallelism the sum of squares is
        reduced over the group so that every rank normalises by the statistics of the full width."""
        n = self.heads_local * self.spec.head_dim
        H = self.spec.hidden
        for i, norm in enumerate((self.q_norm, self.k_norm)):
            part = qkv[:, i * n:(i + 1) * n]
            if self.group.size == 1:
                part.copy_(norm(part.contiguous()))
                continue
            ss = part.float().pow(2).sum(-1, keepdim=True)
            ss = self.group.all_reduce(ss)
            lo = self.group.rank * n
            w = norm.weight[lo: lo + n].float()
            part.copy_((part.float() * torch.rsqrt(ss / H + norm.eps) * w).to(part.dtype))

    def forward(self, x: torch.Tensor, cs: torch.Tensor | None, cu: torch.Tensor, max_len: int) -> torch.Tensor:
        spec = self.spec
        T = x.shape[0]
        hl, d = self.heads_local, spec.head_dim
        qkv = self.qkv(self.norm1(x))
        if spec.qk_norm:
            self._qk_norm_full(qkv, T)
        if cs is not None:
            ops.rope_(qkv[:, : 2 * hl * d].view(T, 2 * hl, d), cs)
        q = qkv[:, : hl * d].view(T, hl, d)
        k = qkv[:, hl * d: 2 * hl * d].view(T, hl, d)
        v = qkv[:, 2 * hl * d:].view(T, hl, d)
        a = ops.attention_varlen(q, k, v, cu, cu, max_len)
        x = self._row_parallel(self.proj, a.view(T, hl * d), x, self.ls1 if spec.layer_scale else None)
        h = self.norm2(x)
        h = self.fc1(h, act=spec.act)
        return self._row_parallel(self.fc2, h, x, self.ls2 if spec.layer_scale else None)

    # -- checkpoint helpers ------------------------------------------------------------------------------
    def load_norm(self, which: int, leaf: str, t: torch.Tensor) -> None:
        n = self.norm1 if which == 1 else self.norm2
        getattr(n, leaf).data.copy_(t)

    def load_mlp(self, name: str, leaf: str, t: torch.Tensor) -> None:
        """``name`` in {"fc1", "fc2", "gate", "up"}."""
        kw = {leaf: t}
        if name == "fc2":
            self.fc2.load(**kw)
        elif name == "fc1":
            self.fc1.load(**kw)
        else:
            self.fc1.load(name, **kw)


def fused_tp_context(owner: nn.Module, group: ParallelGroup, hidden: int, rows: int, spec: BlockSpec):
    """The peer-memory context that runs a tower's blocks without library collectives, or ``None`` when the plain path
    applies: one GPU, no fabric, too few rows to give every rank a 128-row block, or a block variant that the
    reduction kernel does not cover (learned layer scale, q/k norm over all heads)."""
    if (not getattr(owner, "fused_tp", True) or group.size == 1 or group.fabric is None or rows < 128 * group.size or hidden > 2048 or spec.layer_scale or spec.qk_norm
            or next(owner.parameters()).device.type != "cuda"):
        return None
    from ..parallel.fused import FusedEncoderTP

    tp = getattr(owner, "_tp_ctx", None)
    if tp is None or tp.S_cap < rows:
        tp = owner._tp_ctx = FusedEncoderTP(group, hidden, max(rows, 16384))   # collective: all ranks see the same batches
    return tp


def fused_tp_blocks(tp, blocks: list["EncoderBlock"], x: torch.Tensor, cs: torch.Tensor | None, att: list[tuple[torch.Tensor, int]]) -> torch.Tensor:
    """Runs ``blocks`` on the full (replicated) rows ``x`` with row-sharded activations between the GEMMs: every
    row-parallel GEMM pushes its partial tiles to the owner of the rows, a reduce + residual + norm kernel pushes the
    normalised rows into every rank's next operand, and the following GEMM consumes them chunk by chunk.  Returns the
    full rows again (one library all-gather at the end of the tower)."""
    T = x.shape[0]
    tp.begin(T)
    lo, hi = tp.row_range
    xs = x[lo:hi].contiguous()

    def norm_args(n):
        ln = isinstance(n, LayerNorm)
        return dict(norm_w=n.weight, eps=n.eps, norm_b=getattr(n, "bias", None) if ln else None, layer_norm=ln)

    tp.reduce_norm_push(bias=None, residual=xs, dst=0, reduce=False, **norm_args(blocks[0].norm1))
    for i, (blk, (cu, mx)) in enumerate(zip(blocks, att)):
        spec, hl, d = blk.spec, blk.heads_local, blk.spec.head_dim
        qkv = tp.gemm_gathered(0, blk.qkv.weight, blk.qkv.bias)
        if cs is not None:
            ops.rope_(qkv[:, : 2 * hl * d].view(T, 2 * hl, d), cs)
        q, k, v = (qkv[:, j * hl * d:(j + 1) * hl * d].view(T, hl, d) for j in range(3))
        a = ops.attention_varlen(q, k, v, cu, cu, mx)
        tp.gemm_push(a.view(T, hl * d), blk.proj.weight)
        xs = tp.reduce_norm_push(bias=blk.proj.bias, residual=xs, dst=1, **norm_args(blk.norm2))
        h = tp.gemm_gathered(1, blk.fc1.weight, blk.fc1.bias, act=spec.act, swiglu=spec.gated)
        tp.gemm_push(h, blk.fc2.weight)
        if i + 1 < len(blocks):
            xs = tp.reduce_norm_push(bias=blk.fc2.bias, residual=xs, dst=0, **norm_args(blocks[i + 1].norm1))
        else:
            xs = tp.reduce_norm_push(bias=blk.fc2.bias, residual=xs, norm_w=None, eps=0.0, dst=None)
    # rows of the residual stream back on every rank: owners hold R rows each (the last one fewer)
    full = torch.zeros((tp.group.size * tp.R, x.shape[1]), device=x.device, dtype=x.dtype)
    mine = full[lo: lo + tp.R]
    mine[: xs.shape[0]] = xs
    import torch.distributed as dist

    dist.all_gather_into_tensor(full, mine.clone(), group=tp.group.group)
    return full[:T]


def rot_pos_ids(grid_thw: np.ndarray, merge: int) -> np.ndarray:
    """(row, column) of every patch in merge-block order: ``[L, 2]``."""
    out = []
    for t, h, w in grid_thw.tolist():
        hp = np.broadcast_to(np.arange(h)[:, None], (h, w))
        wp = np.broadcast_to(np.arange(w)[None, :], (h, w))

        def blk(a):
            return a.reshape(h // merge, merge, w // merge, merge).transpose(0, 2, 1, 3).reshape(-1)

        out.append(np.tile(np.stack([blk(hp), blk(wp)], axis=-1), (t, 1)))
    return np.concatenate(out, axis=0)


def rotary_table_2d(grid_thw: np.ndarray, merge: int, head_dim: int, theta: float = 10000.0) -> np.ndarray:
    """cos/sin ``[L, 2, head_dim/2]``: the first quarter of the head rotates with the row index, the second with
    the column index (the 2-D rotary embedding of the Qwen vision towers)."""
    inv = 1.0 / (theta ** (np.arange(0, head_dim // 2, 2, dtype=np.float64) / (head_dim // 2)))
    pos = rot_pos_ids(grid_thw, merge)
    ang = (pos[:, :, None].astype(np.float64) * inv[None, None, :]).reshape(pos.shape[0], -1)
    return np.stack([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)


def frame_cu_seqlens(grid_thw: np.ndarray) -> tuple[np.ndarray, int]:
    """Attention boundaries when every frame attends within itself: ``(cu [frames+1] int32, longest frame)``."""
    frames = np.repeat(grid_thw[:, 1] * grid_thw[:, 2], grid_thw[:, 0])
    return np.concatenate([[0], np.cumsum(frames)]).astype(np.int32), int(frames.max())


def bilinear_pos_indices(grid_thw: np.ndarray, side: int, merge: int) -> tuple[np.ndarray, np.ndarray]:
    """Neighbours and weights for interpolating a ``side x side`` learned position table onto every patch, in
    merge-block order: ``(idx [4, L] int32, weight [4, L] float32)``."""
    idx_all, w_all = [], []
    for t, h, w in grid_thw.tolist():
        hi = np.linspace(0, side - 1, h, dtype=np.float32)
        wi = np.linspace(0, side - 1, w, dtype=np.float32)
        hf, wf = hi.astype(np.int32), wi.astype(np.int32)
        hc, wc = np.minimum(hf + 1, side - 1), np.minimum(wf + 1, side - 1)
        dh, dw = hi - hf, wi - wf
        idx = np.stack([(hf[:, None] * side + wf[None, :]), (hf[:, None] * side + wc[None, :]),
                        (hc[:, None] * side + wf[None, :]), (hc[:, None] * side + wc[None, :])])      # [4, h, w]
        wt = np.stack([(1 - dh)[:, None] * (1 - dw)[None, :], (1 - dh)[:, None] * dw[None, :],
                       dh[:, None] * (1 - dw)[None, :], dh[:, None] * dw[None, :]])

        def blk(a):  # [4, h, w] -> merge-block order, repeated for every frame
            a = a.reshape(4, h // merge, merge, w // merge, merge).transpose(0, 1, 3, 2, 4).reshape(4, -1)
            return np.tile(a, (1, t))

        idx_all.append(blk(idx))
        w_all.append(blk(wt))
    return np.concatenate(idx_all, axis=1).astype(np.int32), np.concatenate(w_all, axis=1).astype(np.float32)


def sinusoid_positions(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """Whisper-style table ``[length, channels]`` = ``[sin | cos]`` (fp32)."""
    inc = np.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-inc * torch.arange(channels // 2).float())
    t = torch.arange(length)[:, None].float() * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)
