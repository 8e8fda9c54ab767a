"""Tensor-parallel building blocks on top of :mod:`cornserve.ops`.

Sharding follows the Megatron scheme the reference uses for its encoders
(python/cornserve/task_executors/eric/models/layers/linear.py:76-554): column-parallel weights are
``[out/tp, in]``, row-parallel weights ``[out, in/tp]``, fused QKV is sharded per head with KV-head
replication when ``tp > kv_heads``.  Differences: checkpoints are sharded by explicit ``load_*``
methods instead of state-dict hooks, awkward inner sizes are zero-padded to TMA-friendly multiples,
and the row-parallel reduction can be handed to a fused GEMM+collective kernel.
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group


def _param(*shape: int, device, dtype, std: float | None = 0.02) -> nn.Parameter:
    t = torch.empty(*shape, device=device, dtype=dtype)
    if std is None:
        t.zero_()
    elif std == 1.0:
        t.fill_(1.0)
    else:
        # deterministic, cheap random init that also works for very large matrices
        t.normal_(0.0, std)
    return nn.Parameter(t, requires_grad=False)


def round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def quantize_fp8_(layer: nn.Module) -> None:
    """Replace a layer's bf16 weight ``[N, K]`` (``K % 128 == 0``) by e4m3 values with one fp32 scale per 128 x 128 block
    (``layer.fp8 = (wq, scales)``); the layer's ``forward`` then runs the block-scaled GEMM."""
    w = layer.weight.data
    if w.shape[1] % 128:
        raise ValueError(f"fp8 block scaling needs an input width that is a multiple of 128, got {w.shape[1]}")
    layer.fp8 = ops.quantize_fp8_weight(w)
    layer.weight = None


def _linear_fp8(x: torch.Tensor, fp8, bias) -> torch.Tensor:
    return ops.linear_fp8(x, fp8[0], fp8[1], bias).to(x.dtype)


class Linear(nn.Module):
    """Replicated linear layer ``y = act(x W^T + b) (+ residual)``."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, device=None,
                 dtype=torch.bfloat16, std: float = 0.02):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = _param(out_features, in_features, device=device, dtype=dtype, std=std)
        self.bias = _param(out_features, device=device, dtype=dtype, std=None) if bias else None

    def forward(self, x, act=None, residual=None, gate=None, gate_rows_per_batch=1, out_dtype=None):
        return ops.linear(x, self.weight, self.bias, act=act, residual=residual, gate=gate,
                          gate_rows_per_batch=gate_rows_per_batch, out_dtype=out_dtype)

    def load(self, weight: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
        if weight is not None:
            self.weight.data.copy_(weight.reshape(self.weight.shape))
        if bias is not None and self.bias is not None:
            self.bias.data.copy_(bias)


class ColumnParallelLinear(nn.Module):
    """Output features sharded over the group; the local output is ``[*, out/tp]``.

    ``out_features`` is zero-padded up to ``pad_multiple * tp`` so that every shard has a TMA-friendly
    width (padded rows of the weight are zero, so padded outputs are ``act(0)``-then-ignored).
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, group: ParallelGroup | None = None,
                 pad_multiple: int = 8, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.group = group or single_group()
        tp = self.group.size
        self.in_features, self.out_features = in_features, out_features
        self.out_padded = round_up(out_features, pad_multiple * tp)
        self.out_local = self.out_padded // tp
        self.weight = _param(self.out_local, in_features, device=device, dtype=dtype)
        self.bias = _param(self.out_local, device=device, dtype=dtype, std=None) if bias else None
        self._zero_padding()

    def _shard_range(self) -> tuple[int, int]:
        lo = self.group.rank * self.out_local
        return lo, min(lo + self.out_local, self.out_features)

    def _zero_padding(self) -> None:
        lo, hi = self._shard_range()
        n = max(hi - lo, 0)
        if n < self.out_local:
            self.weight.data[n:].zero_()

    def forward(self, x, act=None):
        return ops.linear(x, self.weight, self.bias, act=act)

    def load(self, weight: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
        lo, hi = self._shard_range()
        if weight is not None:
            weight = weight.reshape(self.out_features, -1)
            self.weight.data[: hi - lo].copy_(weight[lo:hi])
        if bias is not None and self.bias is not None:
            self.bias.data[: hi - lo].copy_(bias[lo:hi])
        self._zero_padding()


class MergedColumnParallelLinear(nn.Module):
    """Gate and up projections of a gated MLP in one weight ``[2 * I/tp, in]`` = ``[gate_shard; up_shard]``,
    consumed by the fused SwiGLU GEMM (activation and product happen in the epilogue)."""

    def __init__(self, in_features: int, intermediate: int, bias: bool = False, *, group: ParallelGroup | None = None,
                 pad_multiple: int = 8, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.group = group or single_group()
        tp = self.group.size
        self.in_features, self.intermediate = in_features, intermediate
        self.inter_padded = round_up(intermediate, pad_multiple * tp)
        self.inter_local = self.inter_padded // tp
        self.weight = _param(2 * self.inter_local, in_features, device=device, dtype=dtype)
        self.bias = _param(2 * self.inter_local, device=device, dtype=dtype, std=None) if bias else None
        self.fp8 = None
        self._zero_padding()

    def _shard_range(self) -> tuple[int, int]:
        lo = self.group.rank * self.inter_local
        return lo, min(lo + self.inter_local, self.intermediate)

    def _zero_padding(self) -> None:
        lo, hi = self._shard_range()
        n = max(hi - lo, 0)
        if n < self.inter_local:
            self.weight.data[n: self.inter_local].zero_()
            self.weight.data[self.inter_local + n:].zero_()
            if self.bias is not None:
                self.bias.data[n: self.inter_local].zero_()
                self.bias.data[self.inter_local + n:].zero_()

    def forward(self, x, act: str = "silu"):
        if self.fp8 is not None:
            return ops.act_mul(_linear_fp8(x, self.fp8, self.bias), act)
        return ops.swiglu_linear(x, self.weight, self.bias, act=act)

    def load(self, which: str, weight: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
        """``which`` is ``"gate"`` or ``"up"``."""
        lo, hi = self._shard_range()
        base = 0 if which == "gate" else self.inter_local
        if weight is not None:
            self.weight.data[base: base + hi - lo].copy_(weight[lo:hi])
        if bias is not None and self.bias is not None:
            self.bias.data[base: base + hi - lo].copy_(bias[lo:hi])


class RowParallelLinear(nn.Module):
    """Input features sharded over the group; partial sums are reduced over the group.

    Bias and residual are added on rank 0 only, *before* the reduction, so they ride along in the
    GEMM epilogue and the reduced result needs no further elementwise pass.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, *, group: ParallelGroup | None = None,
                 in_padded: int | None = None, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.group = group or single_group()
        tp = self.group.size
        self.in_features, self.out_features = in_features, out_features
        self.in_padded = in_padded or round_up(in_features, 8 * tp)
        self.in_local = self.in_padded // tp
        self.weight = _param(out_features, self.in_local, device=device, dtype=dtype)
        self.bias = _param(out_features, device=device, dtype=dtype, std=None) if bias else None
        self.fp8 = None
        self._zero_padding()

    def _shard_range(self) -> tuple[int, int]:
        lo = self.group.rank * self.in_local
        return lo, min(lo + self.in_local, self.in_features)

    def _zero_padding(self) -> None:
        lo, hi = self._shard_range()
        n = max(hi - lo, 0)
        if n < self.in_local:
            self.weight.data[:, n:].zero_()

    def forward(self, x, residual=None, act=None, reduce: bool = True):
        first = self.group.is_first
        if self.fp8 is not None:
            if act is not None:
                raise ValueError("the fp8 row-parallel projection has no activation epilogue")
            y = _linear_fp8(x, self.fp8, self.bias if first else None)
            if residual is not None and first:
                y = y + residual
        else:
            y = ops.linear(x, self.weight, self.bias if first else None, act=act if self.group.size == 1 else None,
                           residual=residual if first else None)
        if self.group.size > 1 and reduce:
            y = self.group.all_reduce(y)
        return y

    def load(self, weight: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
        lo, hi = self._shard_range()
        if weight is not None:
            self.weight.data[:, : hi - lo].copy_(weight[:, lo:hi])
        if bias is not None and self.bias is not None:
            self.bias.data.copy_(bias)
        self._zero_padding()


class QKVParallelLinear(nn.Module):
    """Fused q/k/v projection, sharded per head.  Local layout: ``[q heads | k heads | v heads] x d``.

    With ``tp > kv_heads`` every KV head is replicated on ``tp / kv_heads`` ranks.  Checkpoints may
    provide separate q/k/v tensors or one fused ``[q; k; v]`` tensor (``load_fused``)."""

    def __init__(self, hidden: int, head_dim: int, num_heads: int, num_kv_heads: int | None = None, bias: bool = True,
                 *, group: ParallelGroup | None = None, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.group = group or single_group()
        tp = self.group.size
        num_kv_heads = num_kv_heads or num_heads
        if num_heads % tp != 0:
            raise ValueError(f"{num_heads} heads cannot be split over tp={tp}")
        self.hidden, self.head_dim = hidden, head_dim
        self.num_heads, self.num_kv_heads = num_heads, num_kv_heads
        self.heads_local = num_heads // tp
        if num_kv_heads >= tp:
            if num_kv_heads % tp != 0:
                raise ValueError(f"{num_kv_heads} kv heads cannot be split over tp={tp}")
            self.kv_heads_local, self.kv_replicas = num_kv_heads // tp, 1
        else:
            if tp % num_kv_heads != 0:
                raise ValueError(f"tp={tp} is not a multiple of {num_kv_heads} kv heads")
            self.kv_heads_local, self.kv_replicas = 1, tp // num_kv_heads
        self.q_size = self.heads_local * head_dim
        self.kv_size = self.kv_heads_local * head_dim
        self.weight = _param(self.q_size + 2 * self.kv_size, hidden, device=device, dtype=dtype)
        self.bias = _param(self.q_size + 2 * self.kv_size, device=device, dtype=dtype, std=None) if bias else None
        self.fp8 = None

    def forward(self, x):
        if self.fp8 is not None:
            return _linear_fp8(x, self.fp8, self.bias)
        return ops.linear(x, self.weight, self.bias)

    def _rows(self, which: str) -> tuple[int, int, int]:
        """(destination row, source row, count) of this rank's shard of q, k or v."""
        r = self.group.rank
        if which == "q":
            return 0, r * self.q_size, self.q_size
        src = (r // self.kv_replicas) * self.kv_size
        dst = self.q_size if which == "k" else self.q_size + self.kv_size
        return dst, src, self.kv_size

    def load(self, which: str, weight: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
        dst, src, n = self._rows(which)
        if weight is not None:
            self.weight.data[dst: dst + n].copy_(weight[src: src + n])
        if bias is not None and self.bias is not None:
            self.bias.data[dst: dst + n].copy_(bias[src: src + n])

    def load_fused(self, weight: torch.Tensor | None = None, bias: torch.Tensor | None = None) -> None:
        """Checkpoint tensor is ``[q; k; v]`` stacked along dim 0."""
        qn, kn = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        for which, lo, hi in (("q", 0, qn), ("k", qn, qn + kn), ("v", qn + kn, qn + 2 * kn)):
            self.load(which, None if weight is None else weight[lo:hi], None if bias is None else bias[lo:hi])


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float = 1e-6, *, gemma: bool = False, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.eps, self.gemma = eps, gemma
        self.weight = _param(hidden, device=device, dtype=dtype, std=None if gemma else 1.0)

    def forward(self, x, residual=None):
        return ops.rms_norm(x, self.weight, self.eps, residual=residual, gemma=self.gemma)


class LayerNorm(nn.Module):
    def __init__(self, hidden: int, eps: float = 1e-5, *, affine: bool = True, bias: bool = True, device=None,
                 dtype=torch.bfloat16):
        super().__init__()
        self.eps = eps
        self.weight = _param(hidden, device=device, dtype=dtype, std=1.0) if affine else None
        self.bias = _param(hidden, device=device, dtype=dtype, std=None) if (affine and bias) else None

    def forward(self, x, scale=None, shift=None, rows_per_batch: int = 1, residual=None):
        return ops.layer_norm(x, self.weight, self.bias, self.eps, scale, shift, rows_per_batch, residual=residual)


class Embedding(nn.Module):
    def __init__(self, num: int, dim: int, *, device=None, dtype=torch.bfloat16):
        super().__init__()
        self.weight = _param(num, dim, device=device, dtype=dtype)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.gather_rows(self.weight, ids)


def sinusoid_table(length: int, channels: int, max_timescale: float = 10000.0) -> torch.Tensor:
    """Whisper-style sinusoidal position table ``[length, channels]`` (fp32)."""
    log_inc = math.log(max_timescale) / (channels // 2 - 1)
    inv = torch.exp(-log_inc * torch.arange(channels // 2, dtype=torch.float32))
    t = torch.arange(length, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([t.sin(), t.cos()], dim=1)
