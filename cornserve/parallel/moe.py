"""Mixture-of-experts forward: top-k routing, (expert-parallel) dispatch, expert SwiGLU FFNs, combine.

The reference has no MoE code of its own (the Qwen3-Omni thinker runs inside its vLLM dependency).
Routing math follows Qwen3-MoE: softmax over all experts in fp32, top-k, optional renormalisation.

On CUDA the layer runs through :class:`FusedMoE`: routing, slot assignment, the token exchange and the grouped
tcgen05 GEMMs are kernels of one stream that meet the other ranks only through counters in peer memory; nothing
returns to the host (so a decode step with experts can sit in a CUDA graph).  Every rank owns ``E / ep`` experts.
The functions below it are the plain restatement used on the CPU (with library collectives when ``group.size > 1``).
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p

import torch

from .. import ops
from ..ops import _lib
from .state import ParallelGroup

_P, _I, _L = c_void_p, c_int, c_longlong
_lib.register_signature("cs_moe_route", [_P, _L, _I, _I, _I, _I, _P, _P, _P, _P, _I, _I, _P, _P, _P], _I)
_lib.register_signature("cs_moe_layout", [_P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P], _I)
_lib.register_signature("cs_moe_dispatch", [_P, _L, _I, _I, _I, _I, _I, _I, _I, _P, _P, _P, _P, _P, _L, _P, _P, _P, _P], _I)
_lib.register_signature("cs_moe_wait", [_P, _P, _I, _I, _P], _I)
_lib.register_signature("cs_moe_combine", [_P, _L, _P, _I, _I, _I, _I, _P, _P, _P, _P, _L, _I, _I, _P, _P, _P], _I)
_lib.register_signature("cs_gemm_bf16_grouped", [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _P, _P, _P, _I, _P, _P, _L, _P, _P, _P], _I)


class _Shared:
    """A buffer that every rank of the group can store into: symmetric memory, or a plain tensor for one rank."""

    def __init__(self, group: ParallelGroup, numel: int, dtype: torch.dtype, zero: bool):
        if group.size > 1:
            buf = group.fabric.alloc(numel, dtype, zero=zero)
            self.local, ptrs = buf.local, buf.ptrs
            self._keep = buf
        else:
            self.local = (torch.zeros if zero else torch.empty)(numel, device=group.device, dtype=dtype)
            ptrs = [self.local.data_ptr()]
        self.ptrs = ctypes.cast((c_void_p * len(ptrs))(*ptrs), c_void_p)
        self._arr = self.ptrs


class FusedMoE:
    """Expert-parallel mixture-of-experts layer over peer memory (one instance serves every layer of a model).

    ``forward(x, logits, w_gate_up, w_down)``: route -> layout -> dispatch (rows stored straight into the owning
    rank's expert segments) -> grouped gate|up GEMM with SwiGLU -> grouped down GEMM whose epilogue stores every
    row at its token's owner -> weighted combine.  With ``replicated=True`` the ranks hold the same tokens (the
    usual tensor-parallel decoder): each rank routes a slice of them and the combine kernel writes every result row
    into all ranks' outputs.
    """

    def __init__(self, group: ParallelGroup, num_experts: int, top_k: int, hidden: int, intermediate: int, max_tokens: int,
                 norm_topk: bool = True):
        if group.size > 1 and group.fabric is None:
            raise RuntimeError("expert parallelism over peer memory needs the fabric")
        if num_experts % group.size or num_experts > 256 or top_k > 16 or hidden % 8 or intermediate % 8:
            raise ValueError("unsupported expert configuration")
        self.group, self.E, self.k, self.H, self.I = group, num_experts, top_k, hidden, intermediate
        self.El = num_experts // group.size
        self.norm = norm_topk
        W, dev = group.size, group.device
        self.max_tokens = max_tokens
        self.cap_rows = (W * max_tokens * top_k + self.El * 128 + 127) // 128 * 128   # every token could land here
        i32, bf = torch.int32, torch.bfloat16
        self.counts_all = _Shared(group, W * num_experts, i32, True)
        self.counts_flag = _Shared(group, 4, i32, True)
        self.x_recv = _Shared(group, self.cap_rows * hidden, bf, False)
        self.row_meta = _Shared(group, self.cap_rows * 2, i32, True)
        self.disp_flag = _Shared(group, 4, i32, True)
        self.y_back = _Shared(group, max_tokens * top_k * hidden, bf, False)
        self.comb_flag = _Shared(group, 4, i32, True)
        self.out_all = _Shared(group, W * max_tokens * hidden, bf, False)
        self.out_flag = _Shared(group, 4, i32, True)
        z = lambda n: torch.zeros(n, device=dev, dtype=i32)  # noqa: E731
        self.counts, self.cursor, self.base = z(num_experts), z(num_experts), z(num_experts)
        self.tile_expert, self.tile_valid = z(self.cap_rows // 16), z(self.cap_rows // 16)
        self.num_tiles, self.overflow, self.epoch = z(1), z(1), z(1)
        self.done = z(4)
        self.topk_w = torch.empty(max_tokens * top_k, device=dev, dtype=torch.float32)
        self.topk_e = z(max_tokens * top_k)
        self.h = torch.empty(self.cap_rows * intermediate, device=dev, dtype=bf)
        self.out_local = torch.empty(max_tokens * hidden, device=dev, dtype=bf)
        if group.size > 1:
            group.barrier()

    def tile_rows_for(self, total_tokens: int) -> int:
        """Row tile of the grouped GEMMs: large when experts see many rows, small when few (less padding read)."""
        avg = total_tokens * self.k / self.E
        return 128 if avg >= 64 else 64 if avg >= 24 else 32 if avg >= 8 else 16

    def forward(self, x: torch.Tensor, logits: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                replicated: bool = False) -> torch.Tensor:
        g, lib = self.group, _lib.load()
        W, r, E, k, H, I = g.size, g.rank, self.E, self.k, self.H, self.I
        T_all = x.shape[0]
        assert x.dtype == torch.bfloat16 and logits.dtype == torch.float32 and x.stride(1) == 1 and logits.stride(1) == 1
        assert w_gate_up.is_contiguous() and w_down.is_contiguous()
        if replicated and W > 1:
            per = -(-T_all // W)
            row0, T = min(r * per, T_all), max(0, min(T_all, (r + 1) * per) - r * per)
            total = T_all
        else:
            row0, T, total = 0, T_all, T_all * W  # estimate of the tokens of all ranks (only picks the tile size)
        if T > self.max_tokens or (replicated and T_all > W * self.max_tokens):
            raise ValueError(f"{T} tokens exceed the layer's capacity of {self.max_tokens}")
        xs, ls = x[row0: row0 + T], logits[row0: row0 + T]
        tile = self.tile_rows_for(total)
        st = ops._stream()
        chk = ops._chk
        chk(lib.cs_moe_route(ls.data_ptr() if T else None, logits.stride(0), T, E, k, int(self.norm), self.topk_w.data_ptr(),
                             self.topk_e.data_ptr(), self.counts.data_ptr(), self.done[0:].data_ptr(), W, r,
                             self.counts_all.ptrs, self.counts_flag.ptrs, st), "cs_moe_route")
        chk(lib.cs_moe_layout(self.counts_all.local.data_ptr(), self.counts_flag.local.data_ptr(), self.epoch.data_ptr(), W, r, E,
                              tile, self.cap_rows, self.cap_rows // tile, self.base.data_ptr(), self.cursor.data_ptr(),
                              self.tile_expert.data_ptr(), self.tile_valid.data_ptr(), self.num_tiles.data_ptr(),
                              self.overflow.data_ptr(), st), "cs_moe_layout")
        chk(lib.cs_moe_dispatch(xs.data_ptr() if T else None, x.stride(0), T, k, H, E, W, r, self.cap_rows, self.topk_e.data_ptr(),
                                self.base.data_ptr(), self.cursor.data_ptr(), self.overflow.data_ptr(), self.x_recv.ptrs, H,
                                self.row_meta.ptrs, self.disp_flag.ptrs, self.done[1:].data_ptr(), st), "cs_moe_dispatch")
        chk(lib.cs_moe_wait(self.disp_flag.local.data_ptr(), self.epoch.data_ptr(), W, 1, st), "cs_moe_wait")
        chk(lib.cs_gemm_bf16_grouped(self.x_recv.local.data_ptr(), H, w_gate_up.data_ptr(), H, self.h.data_ptr(), I, self.cap_rows,
                                     I, H, 1, self.El, tile, self.tile_expert.data_ptr(), self.tile_valid.data_ptr(),
                                     self.num_tiles.data_ptr(), 0, None, None, 0, None, None, st), "cs_gemm_bf16_grouped")
        chk(lib.cs_gemm_bf16_grouped(self.h.data_ptr(), I, w_down.data_ptr(), I, None, 0, self.cap_rows, H, I, 0, self.El, tile,
                                     self.tile_expert.data_ptr(), self.tile_valid.data_ptr(), self.num_tiles.data_ptr(), W,
                                     self.y_back.ptrs, self.comb_flag.ptrs, H, self.row_meta.local.data_ptr(),
                                     self.done[2:].data_ptr(), st), "cs_gemm_bf16_grouped")
        gather = W if (replicated and W > 1) else 0
        chk(lib.cs_moe_combine(self.y_back.local.data_ptr(), H, self.topk_w.data_ptr(), T, k, H, W, self.comb_flag.local.data_ptr(),
                               self.epoch.data_ptr(), self.done[3:].data_ptr(), self.out_local.data_ptr(), H, gather, row0,
                               self.out_all.ptrs, self.out_flag.ptrs, st), "cs_moe_combine")
        ops._count(7)
        ops.count_path("moe_dispatch_gemm_combine")
        if gather:
            chk(lib.cs_moe_wait(self.out_flag.local.data_ptr(), self.epoch.data_ptr(), W, 0, st), "cs_moe_wait")
            ops._count()
            return self.out_all.local[: T_all * H].view(T_all, H)
        return self.out_local[: T * H].view(T, H)


_layers: dict[tuple, FusedMoE] = {}


def fused_layer(group: ParallelGroup, num_experts: int, top_k: int, hidden: int, intermediate: int, tokens: int,
                norm_topk: bool) -> FusedMoE:
    """The shared :class:`FusedMoE` of a model (all its layers have the same shape), grown when a larger batch
    arrives.  Collective when ``group.size > 1``: every rank sees the same batch sizes, so they grow together."""
    key = (id(group), num_experts, top_k, hidden, intermediate, bool(norm_topk))
    cur = _layers.get(key)
    if cur is None or cur.max_tokens < tokens:
        cap = 1024
        while cap < tokens:
            cap *= 2
        cur = _layers[key] = FusedMoE(group, num_experts, top_k, hidden, intermediate, cap, norm_topk)
    return cur


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
