"""Mixture-of-experts forward: top-k routing, (expert-parallel) dispatch, expert SwiGLU FFNs, combine.

The reference has no MoE code of its own (the Qwen3-Omni thinker runs inside its vLLM dependency).
Routing math follows Qwen3-MoE: softmax over all experts in fp32, top-k, optional renormalisation.

Single group member: tokens are sorted by expert and each expert's contiguous slice goes through the
grouped tcgen05 GEMMs.  Expert parallel (``group.size > 1``): every rank owns ``E / ep`` experts;
token rows travel to the owning rank and back (``dispatch`` / ``combine``).
"""

from __future__ import annotations

import torch

from .. import ops
from .state import ParallelGroup


def route(logits: torch.Tensor, top_k: int, norm_topk: bool) -> tuple[torch.Tensor, torch.Tensor]:
    """``(weights [T, k] fp32, experts [T, k] int64)`` from router logits ``[T, E]``."""
    probs = torch.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    if norm_topk:
        w = w / w.sum(dim=-1, keepdim=True)
    return w, idx


def expert_ffn(x_sorted: torch.Tensor, counts: list[int], w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Apply expert ``e`` to rows ``[offset_e, offset_e + counts[e])`` of ``x_sorted``."""
    out = torch.empty((x_sorted.shape[0], w_down.shape[1]), device=x_sorted.device, dtype=x_sorted.dtype)
    off = 0
    for e, n in enumerate(counts):
        if n == 0:
            continue
        h = ops.swiglu_linear(x_sorted[off: off + n], w_gate_up[e])
        ops.linear(h, w_down[e], out=out[off: off + n])
        off += n
    return out


def moe_forward(x: torch.Tensor, router_logits: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                top_k: int, norm_topk: bool, group: ParallelGroup) -> torch.Tensor:
    T, H = x.shape
    E_local = w_gate_up.shape[0]
    E = E_local * group.size
    w, idx = route(router_logits, top_k, norm_topk)
    flat_e = idx.reshape(-1)                      # [T*k]
    order = torch.argsort(flat_e, stable=True)    # assignment slots sorted by expert
    token_of = torch.div(order, top_k, rounding_mode="floor")
    counts = torch.bincount(flat_e, minlength=E)
    x_sorted = ops.gather_rows(x, token_of.to(torch.int32))
    if group.size == 1:
        y_sorted = expert_ffn(x_sorted, counts.tolist(), w_gate_up, w_down)
    else:
        y_sorted = _expert_parallel(x_sorted, counts, w_gate_up, w_down, group)
    # combine: weight each assignment and sum the k contributions of every token
    wy = y_sorted.float() * w.reshape(-1)[order].unsqueeze(1)
    out = torch.zeros((T, H), device=x.device, dtype=torch.float32)
    out.index_add_(0, token_of, wy)
    return out.to(x.dtype)


def _expert_parallel(x_sorted: torch.Tensor, counts: torch.Tensor, w_gate_up, w_down, group: ParallelGroup) -> torch.Tensor:
    """Variable-split all-to-all dispatch, local experts, all-to-all combine (library collectives;
    the fused peer-memory kernel in ``parallel.fused`` replaces this on NVLink)."""
    import torch.distributed as dist

    ep, e_local = group.size, w_gate_up.shape[0]
    send_counts = counts.view(ep, e_local)                     # rows for each (dst rank, its expert)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group.group)
    send_rows = send_counts.sum(1).tolist()
    recv_rows = recv_counts.sum(1).tolist()
    recv = torch.empty((sum(recv_rows), x_sorted.shape[1]), device=x_sorted.device, dtype=x_sorted.dtype)
    dist.all_to_all_single(recv, x_sorted.contiguous(), recv_rows, send_rows, group=group.group)
    # received rows are grouped by source rank, then by expert: regroup by expert
    rc = recv_counts.tolist()
    src_off, chunks = 0, [[] for _ in range(e_local)]
    for s in range(ep):
        for e in range(e_local):
            n = rc[s][e]
            chunks[e].append((src_off, n))
            src_off += n
    perm = torch.cat([torch.arange(o, o + n, device=recv.device) for e in range(e_local) for (o, n) in chunks[e]]) \
        if recv.shape[0] > 0 else torch.empty(0, dtype=torch.long, device=recv.device)
    by_expert = recv[perm]
    per_expert = [sum(n for _, n in chunks[e]) for e in range(e_local)]
    y = expert_ffn(by_expert, per_expert, w_gate_up, w_down)
    back = torch.empty_like(y)
    back[perm] = y
    out = torch.empty((x_sorted.shape[0], y.shape[1]), device=y.device, dtype=y.dtype)
    dist.all_to_all_single(out, back, send_rows, recv_rows, group=group.group)
    return out
