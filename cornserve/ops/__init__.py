"""Operator front-end.

Every function takes torch tensors.  CUDA bf16 tensors go to the hand-written sm_100a kernels in
``libcornserve.so`` (tcgen05 GEMM and attention, fused norms / rotary / gather kernels);
CPU tensors go to the fp32 restatements in :mod:`cornserve.ops.reference`.  There is no
PyTorch-kernel fallback for CUDA tensors: a missing library raises.
"""

from __future__ import annotations

import math

import torch

from . import _lib, reference
from .reference import ACTS

__all__ = [
    "linear", "swiglu_linear", "rms_norm", "layer_norm", "rope_", "mrope_table", "rope_kv_write_",
    "attention_varlen", "attention_paged", "act_mul", "gather_rows", "scatter_rows_", "argmax",
    "flow_step_", "pcm16", "decode_advance_", "l2_flush", "check_error", "kernel_launches", "reset_launch_count",
    "count_path", "path_counts", "push_bytes_", "apply_penalties_", "count_tokens_",
    "head_norm_rope_", "softmax_rows", "im2col3x3", "im2col1d", "dwconv1d", "to_rgb8", "conv3x3", "conv1d_causal",
    "conv_transpose1d_causal", "bilinear_embed_add_",
]

_launches = 0


def kernel_launches() -> int:
    """Number of launches of this library's kernels issued through this module so far."""
    return _launches


def reset_launch_count() -> None:
    global _launches
    _launches = 0


def _count(n: int = 1) -> None:
    global _launches
    _launches += n


_paths: dict[str, int] = {}


def count_path(name: str, n: int = 1) -> None:
    """Count ``n`` launches of a named fused path (e.g. the GEMM + all-reduce + norm tail of a tensor-parallel decoder)."""
    _paths[name] = _paths.get(name, 0) + n


def path_counts() -> dict[str, int]:
    """Launches per named fused path since the process started (graph replays included by their owners)."""
    return dict(_paths)


def bind_thread(device: torch.device | str) -> None:
    """Make ``device`` the CUDA device of the calling thread.  The current device is a per-thread setting and new
    threads start on device 0, while the kernels of this library launch on the current device: every thread that
    runs them for a model on another GPU calls this first."""
    device = torch.device(device)
    if device.type == "cuda":
        torch.cuda.set_device(device)


def _on_current_device(t: torch.Tensor) -> None:
    if t.device.index is not None and t.device.index != torch.cuda.current_device():
        raise RuntimeError(f"tensor on {t.device} but the thread's CUDA device is {torch.cuda.current_device()}: "
                           "call ops.bind_thread(device) at the start of the thread")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _chk(rc: int, name: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{name} failed with code {rc}")


def check_error(where: str = "") -> None:
    _lib.check_error(where)


def _as2d(x: torch.Tensor) -> torch.Tensor:
    if x.dim() == 2:
        return x
    return x.reshape(-1, x.shape[-1])


def _rowmajor(x: torch.Tensor) -> torch.Tensor:
    if x.stride(-1) != 1:
        x = x.contiguous()
    return x


# --------------------------------------------------------------------------------------------
# GEMM
# --------------------------------------------------------------------------------------------
SKINNY_MAX_M = 128          # largest row count the weight-streaming split-K kernel is considered for


def _use_skinny(M: int, N: int, K: int) -> bool:
    """Measured crossover on B200: the split-K kernel wins whenever K is long (down projections) and
    for very few rows; otherwise the persistent tiled kernel already streams W at full width."""
    if M > SKINNY_MAX_M:
        return False
    return K >= 8192 or M <= 32
_SKINNY_WS_BYTES = 64 << 20
_SKINNY_COUNTERS = 8192
_skinny_ws: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}


def _skinny_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Split-K scratch (fp32 partials + per-tile counters) of the current stream of ``device``.

    Kernels on one stream run in order, so they can share one scratch area; different streams get
    their own.  The buffers are created on first use (before any graph capture: engines warm up first).
    """
    key = (device.index or 0, torch.cuda.current_stream(device).cuda_stream)
    w = _skinny_ws.get(key)
    if w is None:
        w = (torch.empty(_SKINNY_WS_BYTES, device=device, dtype=torch.uint8),
             torch.zeros(_SKINNY_COUNTERS, device=device, dtype=torch.int32))
        _skinny_ws[key] = w
    return w


def _skinny(x2, w, bias, act, r2, out2, M, N, K, swiglu, fp32, splits):
    # A stored weight (an ``nn.Parameter``) is fetched while the kernel before this one still runs; anything else may
    # be that kernel's output (attention scores against keys, a slice made a moment ago) and is fetched after it.
    lib = _lib.load()
    ws, counters = _skinny_workspace(x2.device)
    rc = lib.cs_gemm_skinny(
        x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0), out2.data_ptr(), out2.stride(0),
        _ptr(bias), _ptr(r2), 0 if r2 is None else r2.stride(0), M, N, K, ACTS[act or "none"],
        1 if swiglu else 0, (1 if fp32 else 0) | (0 if isinstance(w, torch.nn.Parameter) else 2), splits,
        ws.data_ptr(), ws.numel(), counters.data_ptr(),
        counters.numel(), _stream(),
    )
    _chk(rc, "cs_gemm_skinny")
    _count()


def linear(
    x: torch.Tensor,
    w: torch.Tensor,
    bias: torch.Tensor | None = None,
    *,
    act: str | None = None,
    residual: torch.Tensor | None = None,
    gate: torch.Tensor | None = None,
    gate_rows_per_batch: int = 1,
    out: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    bn: int = 0,
    stages: int = 0,
    skinny: bool | None = None,
    splits: int = 0,
) -> torch.Tensor:
    """``act(x @ w.T + bias) * gate + residual`` with w in the nn.Linear layout ``[N, K]``.

    Up to ``SKINNY_MAX_M`` rows the weight-streaming split-K kernel is used (``skinny=False`` or an
    explicit ``bn`` forces the tiled kernel).

    ``gate`` is ``[rows / gate_rows_per_batch, N]`` (one gate row per batch element, as in AdaLN).
    """
    shape = x.shape
    x2 = _rowmajor(_as2d(x))
    if not x2.is_cuda:
        r2 = None if residual is None else _as2d(residual)
        y = reference.linear(x2, w, bias, act, r2, gate, gate_rows_per_batch, out_dtype)
        if out is not None:
            out.copy_(y.view(out.shape))
            return out
        return y.view(*shape[:-1], w.shape[0])
    assert x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "CUDA GEMM is bf16"
    _on_current_device(x2)
    M, K = x2.shape
    N = w.shape[0]
    assert w.shape[1] == K and w.stride(1) == 1
    fp32 = out_dtype == torch.float32
    if out is None:
        out = torch.empty((M, N), device=x.device, dtype=torch.float32 if fp32 else torch.bfloat16)
    o2 = _as2d(out)
    r2 = None if residual is None else _rowmajor(_as2d(residual))
    if gate is None and bn == 0 and M <= 256 and (skinny or (skinny is None and _use_skinny(M, N, K))):
        _skinny(x2, w, bias, act, r2, o2, M, N, K, False, fp32, splits)
        return out.view(*shape[:-1], N) if out.dim() == 2 and len(shape) != 2 else out
    lib = _lib.load()
    rc = lib.cs_gemm_bf16(
        x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0), o2.data_ptr(), o2.stride(0),
        _ptr(bias), _ptr(r2), 0 if r2 is None else r2.stride(0),
        _ptr(gate), 0 if gate is None else gate.stride(0), gate_rows_per_batch,
        M, N, K, ACTS[act or "none"], 0, 1 if fp32 else 0, bn, stages, _stream(),
    )
    _chk(rc, "cs_gemm_bf16")
    _count()
    return out.view(*shape[:-1], N) if out.dim() == 2 and len(shape) != 2 else out


def swiglu_linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None, *, act: str = "silu",
                  bn: int = 0, stages: int = 0, skinny: bool | None = None, splits: int = 0) -> torch.Tensor:
    """``act(x @ Wg.T) * (x @ Wu.T)`` with ``w = cat([Wg, Wu])`` of shape ``[2I, K]``; one kernel."""
    shape = x.shape
    x2 = _rowmajor(_as2d(x))
    n = w.shape[0] // 2
    if not x2.is_cuda:
        return reference.swiglu_linear(x2, w, bias, act).view(*shape[:-1], n)
    M, K = x2.shape
    out = torch.empty((M, n), device=x.device, dtype=torch.bfloat16)
    if bn == 0 and M <= 256 and (skinny or (skinny is None and _use_skinny(M, n, K))):
        _skinny(x2, w, bias, act, None, out, M, n, K, True, False, splits)
        return out.view(*shape[:-1], n)
    lib = _lib.load()
    rc = lib.cs_gemm_bf16(
        x2.data_ptr(), x2.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0),
        _ptr(bias), None, 0, None, 0, 1, M, n, K, ACTS[act], 1, 0, bn, stages, _stream(),
    )
    _chk(rc, "cs_gemm_bf16(swiglu)")
    _count()
    return out.view(*shape[:-1], n)


# --------------------------------------------------------------------------------------------
# norms
# --------------------------------------------------------------------------------------------
def _norm(x, w, b, eps, mode, residual, scale, shift, rows_per_batch):
    shape = x.shape
    x2 = _rowmajor(_as2d(x))
    rows, H = x2.shape
    y = torch.empty((rows, H), device=x.device, dtype=x.dtype)
    r2 = None if residual is None else _rowmajor(_as2d(residual))
    new_res = torch.empty_like(y) if residual is not None else None
    lib = _lib.load()
    rc = lib.cs_norm(
        x2.data_ptr(), x2.stride(0), _ptr(r2), 0 if r2 is None else r2.stride(0),
        _ptr(new_res), H, _ptr(w), _ptr(b), _ptr(scale), _ptr(shift),
        0 if scale is None else scale.stride(0), rows_per_batch,
        y.data_ptr(), H, rows, H, float(eps), mode, _stream(),
    )
    _chk(rc, "cs_norm")
    _count()
    y = y.view(shape)
    if residual is not None:
        return y, new_res.view(shape)
    return y


def rms_norm(x, w, eps: float = 1e-6, residual=None, gemma: bool = False):
    """RMSNorm in fp32.  With ``residual`` returns ``(norm(x + residual), x + residual)``."""
    if not x.is_cuda:
        return reference.rms_norm(x, w, eps, residual, gemma)
    return _norm(x, w, None, eps, 1 if gemma else 0, residual, None, None, 1)


def layer_norm(x, w, b, eps: float = 1e-5, scale=None, shift=None, rows_per_batch: int = 1, residual=None):
    """LayerNorm; optional AdaLN modulation ``y * (1 + scale[b]) + shift[b]`` with one row per batch."""
    if not x.is_cuda:
        return reference.layer_norm(x, w, b, eps, scale, shift, rows_per_batch, residual)
    return _norm(x, w, b, eps, 2, residual, scale, shift, rows_per_batch)


# --------------------------------------------------------------------------------------------
# rotary
# --------------------------------------------------------------------------------------------
def rope_(x: torch.Tensor, cs: torch.Tensor, rot: int | None = None) -> torch.Tensor:
    """In-place rotate-half RoPE on ``x`` = ``[T, heads, d]`` (a view with token stride is fine)."""
    T, heads, d = x.shape
    rot = rot or d
    if not x.is_cuda:
        x.copy_(reference.rope(x, cs, rot))
        return x
    assert x.stride(2) == 1 and x.stride(1) == d and cs.dtype == torch.float32 and cs.is_contiguous()
    lib = _lib.load()
    _chk(lib.cs_rope(x.data_ptr(), x.stride(0), T, heads, d, rot, cs.data_ptr(), _stream()), "cs_rope")
    _count()
    return x


def mrope_table(positions: torch.Tensor, half: int, theta: float, sections=None) -> torch.Tensor:
    """cos/sin table ``[T, 2, half]`` from ``positions`` ``[3, T]`` (int32) with M-RoPE sections."""
    sections = sections or [half, 0, 0]
    if not positions.is_cuda:
        return reference.mrope_table(positions, half, theta, sections)
    positions = positions.to(torch.int32).contiguous()
    T = positions.shape[1]
    cs = torch.empty((T, 2, half), device=positions.device, dtype=torch.float32)
    lib = _lib.load()
    _chk(lib.cs_mrope_table(positions.data_ptr(), T, half, float(theta), sections[0], sections[1],
                            cs.data_ptr(), _stream()), "cs_mrope_table")
    _count()
    return cs


def rope_kv_write_(qkv: torch.Tensor, Hq: int, Hkv: int, d: int, cs: torch.Tensor, cache: torch.Tensor,
                   slot: torch.Tensor) -> torch.Tensor:
    """Rotate q (in place) and k, and append k, v to the paged cache ``[pages, 2, Hkv, page, d]``.

    Returns the query view ``[T, Hq, d]`` into ``qkv``.
    """
    T = qkv.shape[0]
    page = cache.shape[3]
    if not qkv.is_cuda:
        q = reference.rope_kv_write(qkv, Hq, Hkv, d, cs, cache, slot, page)
        return q
    assert qkv.stride(1) == 1 and slot.dtype == torch.int32
    lib = _lib.load()
    _chk(lib.cs_rope_kv_write(qkv.data_ptr(), qkv.stride(0), T, Hq, Hkv, d, cs.data_ptr(), cache.data_ptr(),
                              slot.data_ptr(), page, _stream()), "cs_rope_kv_write")
    _count()
    return qkv[:, : Hq * d].view(T, Hq, d)


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def attention_varlen(q, k, v, cu_q, cu_k, max_q_len: int, scale: float | None = None, causal: bool = False,
                     out: torch.Tensor | None = None, window: int = 0,
                     row_bounds: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """Packed variable-length attention.  q ``[Tq, Hq, d]``, k/v ``[Tk, Hkv, d]`` (strided views are
    fine as long as heads are ``d`` apart); ``cu_*`` are int32 prefix sums.  Returns ``[Tq, Hq, d]``.
    ``window > 0`` (causal only): each query sees the last ``window`` keys up to its own position.
    ``row_bounds`` = ``(lo [Tq], hi [Tq])`` int32 (self attention only): token ``t`` sees keys ``[lo[t], hi[t])`` of the
    packed numbering; with it ``cu_*`` may group several short sequences (attention windows) into one, so that they
    share a 128-row tile instead of occupying one each."""
    Tq, Hq, d = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not q.is_cuda:
        if row_bounds is not None:
            lo, hi = (t.long() for t in row_bounds)
            pos = torch.arange(k.shape[0])
            mask = (pos[None, :] >= lo[:, None]) & (pos[None, :] < hi[:, None])          # [Tq, Tk]
            g = Hq // k.shape[1]
            kk, vv = k.float().repeat_interleave(g, dim=1), v.float().repeat_interleave(g, dim=1)
            sc = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
            sc = sc.masked_fill(~mask[None], float("-inf"))
            o = torch.einsum("hqk,khd->qhd", torch.softmax(sc, dim=-1), vv).to(q.dtype)
        else:
            o = reference.attention_varlen(q, k, v, cu_q, cu_k, scale, causal, window)
        if out is not None:
            out.copy_(o)
            return out
        return o
    Tk, Hkv, _ = k.shape
    for t in (q, k, v):
        assert t.stride(2) == 1 and t.stride(1) == d and t.dtype == torch.bfloat16
    if out is None:
        out = torch.empty((Tq, Hq, d), device=q.device, dtype=torch.bfloat16)
    B = cu_q.numel() - 1
    lib = _lib.load()
    rc = lib.cs_attention(
        q.data_ptr(), q.stride(0), k.data_ptr(), k.stride(0), v.data_ptr(), v.stride(0),
        out.data_ptr(), out.stride(0), cu_q.data_ptr(), cu_k.data_ptr(), None, None, 0, 0,
        B, Tq, Tk, max_q_len, Hq, Hkv, d, float(scale), 1 if causal else 0, 0, 1, None, 0, int(window),
        None if row_bounds is None else row_bounds[0].data_ptr(), None if row_bounds is None else row_bounds[1].data_ptr(), _stream(),
    )
    _chk(rc, "cs_attention")
    _count()
    return out


def _decode_kv_splits(items: int, sms: int, max_tiles: int) -> int:
    """Split count for decode attention.  The kernel is persistent with a static round-robin assignment of
    work items to SMs, so the time is ``ceil(items * s / sms) / s`` item-lengths: take the smallest ``s`` that
    gets within 3% of the best balance, keeping at least two key tiles per split."""
    best_s, best = 1, float("inf")
    for s in range(1, 17):
        if s > 1 and 2 * s > max_tiles:
            break
        cost = -(-items * s // sms) / s
        if cost < best * 0.97:
            best, best_s = cost, s
    return best_s


def attention_paged(q, cache, block_table, kv_len, cu_q, max_q_len: int, scale: float | None = None,
                    causal: bool = True, pack_gqa: bool = False, out: torch.Tensor | None = None,
                    kv_splits: int = 0) -> torch.Tensor:
    """Attention of packed queries over a paged KV cache ``[pages, 2, Hkv, 128, d]``.

    ``kv_len[s]`` counts the keys of sequence ``s`` *including* the ones just appended for these
    queries.  ``pack_gqa`` packs the query heads of one KV head into one tile (decode)."""
    Tq, Hq, d = q.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(d)
    if not q.is_cuda:
        o = reference.attention_paged(q, cache, block_table, kv_len, cu_q, scale, causal)
        if out is not None:
            out.copy_(o)
            return out
        return o
    pages, _, Hkv, page, _ = cache.shape
    assert page == 128, "the paged kernel uses 128-token pages"
    assert q.stride(2) == 1 and q.stride(1) == d and cache.is_contiguous()
    if out is None:
        out = torch.empty((Tq, Hq, d), device=q.device, dtype=torch.bfloat16)
    B = cu_q.numel() - 1
    lib = _lib.load()
    if max_q_len == 1 and Tq == B and d == 128 and Hq // Hkv <= 16 and pack_gqa and causal:
        # decode: the swapped-operand kernel (keys on the 128-row side of the tile, grouped query heads on the other)
        if kv_splits == 0:
            kv_splits = _decode_kv_splits(B * Hkv, lib.cs_sm_count(), block_table.shape[1])
        ws_ptr, ws_bytes = None, 0
        if kv_splits > 1:
            ws, _ = _skinny_workspace(q.device)
            if B * Hq * kv_splits * 130 * 4 > ws.numel():
                kv_splits = 1
            else:
                ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
        rc = lib.cs_attention_decode(q.data_ptr(), q.stride(0), cache.data_ptr(), out.data_ptr(), out.stride(0),
                                     kv_len.data_ptr(), block_table.data_ptr(), block_table.stride(0), pages, B, Hq, Hkv,
                                     float(scale), kv_splits, ws_ptr, ws_bytes, _stream())
        _chk(rc, "cs_attention_decode")
        _count(2 if kv_splits > 1 else 1)
        return out
    if kv_splits == 0:
        # decode (one query token per sequence): spread the keys of each sequence over idle SMs
        items = B * (Hkv if pack_gqa else Hq)
        kv_splits = _decode_kv_splits(items, lib.cs_sm_count(), block_table.shape[1]) if max_q_len == 1 else 1
    ws_ptr, ws_bytes = None, 0
    if kv_splits > 1:
        ws, _ = _skinny_workspace(q.device)
        need = Tq * Hq * kv_splits * (d + 2) * 4
        if need > ws.numel():
            kv_splits = 1
        else:
            ws_ptr, ws_bytes = ws.data_ptr(), ws.numel()
    rc = lib.cs_attention(
        q.data_ptr(), q.stride(0), cache.data_ptr(), 0, None, 0, out.data_ptr(), out.stride(0),
        cu_q.data_ptr(), None, kv_len.data_ptr(), block_table.data_ptr(), block_table.stride(0), pages,
        B, Tq, 0, max_q_len, Hq, Hkv, d, float(scale), 1 if causal else 0, 1 if pack_gqa else 0,
        kv_splits, ws_ptr, ws_bytes, 0, None, None, _stream(),
    )
    _chk(rc, "cs_attention(paged)")
    _count(2 if kv_splits > 1 else 1)
    return out


# --------------------------------------------------------------------------------------------
# misc
# --------------------------------------------------------------------------------------------
def act_mul(gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """``act(gu[..., :I]) * gu[..., I:]``."""
    if not gu.is_cuda:
        return reference.act_mul(gu, act)
    g2 = _rowmajor(_as2d(gu))
    rows, two_i = g2.shape
    n = two_i // 2
    y = torch.empty((rows, n), device=gu.device, dtype=gu.dtype)
    lib = _lib.load()
    _chk(lib.cs_act_mul(g2.data_ptr(), g2.stride(0), y.data_ptr(), n, rows, n, ACTS[act], _stream()), "cs_act_mul")
    _count()
    return y.view(*gu.shape[:-1], n)


def gather_rows(src: torch.Tensor, idx: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[i] = src[idx[i]]`` for 2-D ``src`` (rows of a multiple of 16 bytes)."""
    if not src.is_cuda:
        r = src[idx.long()]
        if out is not None:
            out.copy_(r)
            return out
        return r
    n = idx.numel()
    row_bytes = src.shape[1] * src.element_size()
    if out is None:
        out = torch.empty((n, src.shape[1]), device=src.device, dtype=src.dtype)
    idx = idx.to(torch.int32)
    lib = _lib.load()
    _chk(lib.cs_gather_rows(src.data_ptr(), src.stride(0) * src.element_size(), out.data_ptr(),
                            out.stride(0) * out.element_size(), idx.data_ptr(), n, row_bytes, 0, _stream()),
         "cs_gather_rows")
    _count()
    return out


def scatter_rows_(dst: torch.Tensor, idx: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """``dst[idx[i]] = src[i]`` (negative indices are skipped)."""
    if not dst.is_cuda:
        ok = idx >= 0
        dst[idx[ok].long()] = src[ok]
        return dst
    n = idx.numel()
    row_bytes = src.shape[1] * src.element_size()
    idx = idx.to(torch.int32)
    lib = _lib.load()
    _chk(lib.cs_gather_rows(src.data_ptr(), src.stride(0) * src.element_size(), dst.data_ptr(),
                            dst.stride(0) * dst.element_size(), idx.data_ptr(), n, row_bytes, 1, _stream()),
         "cs_gather_rows(scatter)")
    _count()
    return dst


def push_bytes_(dst: torch.Tensor, src: torch.Tensor) -> torch.Tensor:
    """Copy the bytes of contiguous ``src`` into contiguous ``dst`` (same byte count) with this library's copy
    kernel, launched on ``src``'s GPU.  ``dst`` may be memory of another GPU mapped into this process (CUDA IPC): the
    kernel then stores over NVLink, which is how the sidecar places encoder rows in the consumer's slab."""
    nbytes = src.numel() * src.element_size()
    if dst.numel() * dst.element_size() != nbytes:
        raise ValueError("push_bytes_: size mismatch")
    if not (src.is_contiguous() and dst.is_contiguous()):
        raise ValueError("push_bytes_: both tensors must be contiguous")
    if not src.is_cuda:
        dst.view(torch.uint8).reshape(-1).copy_(src.view(torch.uint8).reshape(-1))
        return dst
    _on_current_device(src)
    lib = _lib.load()
    _chk(lib.cs_push_bytes(src.data_ptr(), dst.data_ptr(), nbytes, _stream()), "cs_push_bytes")
    _count()
    return dst


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Greedy sampling: int32 arg-max of each row (lowest index wins ties)."""
    if not logits.is_cuda:
        return reference.argmax(logits)
    rows, V = logits.shape
    if out is None:
        out = torch.empty((rows,), device=logits.device, dtype=torch.int32)
    scratch = torch.empty(rows * 128, device=logits.device, dtype=torch.float32)
    lib = _lib.load()
    _chk(lib.cs_argmax(logits.data_ptr(), logits.stride(0), rows, V, 1 if logits.dtype == torch.float32 else 0,
                       out.data_ptr(), scratch.data_ptr(), _stream()), "cs_argmax")
    _count(2)
    return out


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_p: torch.Tensor, top_k: torch.Tensor,
                seed: torch.Tensor, draws: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """One token per row of fp32 ``logits`` by temperature / top-k / top-p sampling (int32).

    Per row: ``temperature`` (<= 0: arg-max), ``top_p`` in (0, 1] and ``top_k`` (<= 0: off) restrict the candidates
    (top-k first, top-p over what is left; ties at a cut-off stay in), ``seed`` (int64) names the row's random stream
    and ``draws`` (int32, advanced in place) the position in it, so a (seed, draw) pair always gives the same token."""
    if not logits.is_cuda:
        return reference.sample_rows(logits, temperature, top_p, top_k, seed, draws)
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    assert temperature.dtype == torch.float32 and top_p.dtype == torch.float32 and top_k.dtype == torch.int32
    assert seed.dtype == torch.int64 and draws.dtype == torch.int32
    assert all(t.is_contiguous() and t.numel() >= rows for t in (temperature, top_p, top_k, seed, draws))
    if out is None:
        out = torch.empty((rows,), device=logits.device, dtype=torch.int32)
    lib = _lib.load()
    _chk(lib.cs_sample_rows(logits.data_ptr(), logits.stride(0), rows, V, temperature.data_ptr(), top_p.data_ptr(),
                            top_k.data_ptr(), seed.data_ptr(), draws.data_ptr(), out.data_ptr(), _stream()), "cs_sample_rows")
    _count()
    return out


def apply_penalties_(logits: torch.Tensor, counts: torch.Tensor, frequency: torch.Tensor, presence: torch.Tensor) -> torch.Tensor:
    """OpenAI ``frequency_penalty`` / ``presence_penalty`` in place on fp32 ``logits [rows, V]``: every token a row has
    generated ``c > 0`` times (``counts [rows, V]`` int32) loses ``frequency[row] * c + presence[row]``."""
    if not logits.is_cuda:
        c = counts[: logits.shape[0], : logits.shape[1]].to(logits.dtype)
        logits -= frequency[: logits.shape[0], None] * c + presence[: logits.shape[0], None] * (c > 0)
        return logits
    rows, V = logits.shape
    assert logits.dtype == torch.float32 and counts.dtype == torch.int32 and counts.shape[1] >= V and counts.shape[0] >= rows
    assert frequency.dtype == torch.float32 and presence.dtype == torch.float32
    lib = _lib.load()
    _chk(lib.cs_apply_penalties(logits.data_ptr(), logits.stride(0), counts.data_ptr(), counts.stride(0), frequency.data_ptr(),
                                presence.data_ptr(), rows, V, _stream()), "cs_apply_penalties")
    _count()
    return logits


def count_tokens_(counts: torch.Tensor, tokens: torch.Tensor, active: torch.Tensor | None = None) -> torch.Tensor:
    """``counts[r, tokens[r]] += 1`` for every row (rows whose ``active`` flag is 0 are skipped)."""
    rows = tokens.shape[0]
    if not counts.is_cuda:
        for r in range(rows):
            if active is None or int(active[r]) != 0:
                counts[r, int(tokens[r])] += 1
        return counts
    assert counts.dtype == torch.int32 and tokens.dtype == torch.int32 and (active is None or active.dtype == torch.int32)
    lib = _lib.load()
    _chk(lib.cs_count_tokens(counts.data_ptr(), counts.stride(0), tokens.data_ptr(), _ptr(active), rows, counts.shape[1], _stream()),
         "cs_count_tokens")
    _count()
    return counts


def flow_step_(x: torch.Tensor, cond: torch.Tensor, uncond: torch.Tensor | None, cfg: float, dt: float,
               norm_rescale: bool = False) -> torch.Tensor:
    """In-place flow-matching Euler step with classifier-free guidance on fp32 latents ``[rows, C]``."""
    if not x.is_cuda:
        x.copy_(reference.flow_step(x, cond, uncond, cfg, dt, norm_rescale))
        return x
    rows, C = x.shape
    assert x.dtype == torch.float32 and cond.dtype == torch.bfloat16 and cond.is_contiguous()
    lib = _lib.load()
    _chk(lib.cs_flow_step(x.data_ptr(), cond.data_ptr(), _ptr(uncond), rows, C, float(cfg), float(dt),
                          1 if norm_rescale else 0, _stream()), "cs_flow_step")
    _count()
    return x


def pcm16(x: torch.Tensor) -> torch.Tensor:
    """fp32 waveform in [-1, 1] -> int16 PCM."""
    if not x.is_cuda:
        return reference.pcm16(x)
    xf = x.float().contiguous()
    y = torch.empty(xf.shape, device=x.device, dtype=torch.int16)
    lib = _lib.load()
    _chk(lib.cs_pcm16(xf.data_ptr(), y.data_ptr(), xf.numel(), _stream()), "cs_pcm16")
    _count()
    return y


def decode_advance_(sampled, input_ids, positions, kv_len, slot, block_table, active, out_log, step_counter,
                    page: int = 128) -> None:
    """Feed sampled tokens back as next inputs and advance positions / key counts / cache slots of the
    active sequences on the device (keeps multi-step decode free of host round trips)."""
    B = sampled.numel()
    if not sampled.is_cuda:
        step = int(step_counter.item())
        step_counter += 1
        input_ids.copy_(sampled)
        if step < out_log.shape[0]:
            out_log[step] = sampled
        act = active.bool()
        positions[:, act] += 1
        kv_len[act] += 1
        kv = kv_len.long()
        new_slot = block_table[torch.arange(B), (kv - 1) // page].long() * page + (kv - 1) % page
        slot[act] = new_slot[act].to(slot.dtype)
        return
    lib = _lib.load()
    _chk(lib.cs_decode_advance(sampled.data_ptr(), input_ids.data_ptr(), positions.data_ptr(), kv_len.data_ptr(),
                               slot.data_ptr(), block_table.data_ptr(), block_table.stride(0), active.data_ptr(),
                               out_log.data_ptr(), out_log.shape[0], step_counter.data_ptr(), B, page, _stream()),
         "cs_decode_advance")
    _count()


def l2_flush(buf: torch.Tensor, value: int = 0) -> None:
    """Overwrite ``buf`` (should be larger than L2) to evict cached lines between timed iterations."""
    if not buf.is_cuda:
        return
    lib = _lib.load()
    _chk(lib.cs_l2_flush(buf.data_ptr(), buf.numel() * buf.element_size(), value, _stream()), "cs_l2_flush")
    _count()


# --------------------------------------------------------------------------------------------
# generator models: per-head norm + rotary, soft-max, convolutions as tap gather + tcgen05 GEMM
# --------------------------------------------------------------------------------------------
def head_norm_rope_(x: torch.Tensor, w: torch.Tensor | None, eps: float, cs: torch.Tensor | None, *,
                    w2: torch.Tensor | None = None, seg: int = 0, n_first: int = 0) -> torch.Tensor:
    """In place on ``x`` = ``[T, heads, d]`` (token-strided view is fine): RMSNorm over ``d`` with weight
    ``w`` (skipped when ``None``), then rotate-half RoPE with ``cs`` = ``[T, 2, d/2]`` (skipped when ``None``).
    With ``w2``, rows whose index inside a segment of ``seg`` rows is ``>= n_first`` are normalised with ``w2``
    (two token streams interleaved segment by segment)."""
    T, heads, d = x.shape
    if not x.is_cuda:
        if w2 is None:
            x.copy_(reference.head_norm_rope(x, w, eps, cs))
        else:
            first = (torch.arange(T, device=x.device) % seg) < n_first
            a = reference.head_norm_rope(x, w, eps, cs)
            b = reference.head_norm_rope(x, w2, eps, cs)
            x.copy_(torch.where(first[:, None, None], a, b))
        return x
    assert x.stride(2) == 1 and x.stride(1) == d and x.dtype == torch.bfloat16
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.shape[-1] * 2 == d)
    lib = _lib.load()
    _chk(lib.cs_head_norm_rope(x.data_ptr(), x.stride(0), T, heads, d, _ptr(w), float(eps), _ptr(cs), _ptr(w2), seg, n_first,
                               _stream()), "cs_head_norm_rope")
    _count()
    return x


def qk_norm_rope_(x: torch.Tensor, heads: int, d: int, part_stride: int, wq: torch.Tensor, wk: torch.Tensor, eps: float,
                  cs: torch.Tensor, *, wq2: torch.Tensor | None = None, wk2: torch.Tensor | None = None, seg: int = 0,
                  n_first: int = 0) -> torch.Tensor:
    """In place on the q and k parts of a fused projection ``x`` = ``[T, >= part_stride + heads*d]``: q heads start at
    column 0, k heads at column ``part_stride``.  Each head row gets :func:`head_norm_rope_` with ``wq`` / ``wk``
    (``wq2`` / ``wk2`` for rows past ``n_first`` inside a segment of ``seg`` rows).  One launch for ``d == 128``."""
    T = x.shape[0]
    if not (x.is_cuda and d == 128):
        for off, w, w2 in ((0, wq, wq2), (part_stride, wk, wk2)):
            head_norm_rope_(x[:, off:off + heads * d].view(T, heads, d), w, eps, cs, w2=w2, seg=seg, n_first=n_first)
        return x
    assert x.stride(1) == 1 and x.dtype == torch.bfloat16 and x.shape[1] >= part_stride + heads * d
    assert cs.dtype == torch.float32 and cs.is_contiguous() and cs.shape[-1] * 2 == d and cs.shape[0] >= T
    lib = _lib.load()
    _chk(lib.cs_qk_norm_rope128(x.data_ptr(), x.stride(0), T, heads, part_stride, _ptr(wq), _ptr(wk), _ptr(wq2), _ptr(wk2),
                                float(eps), _ptr(cs), seg, n_first, _stream()), "cs_qk_norm_rope128")
    _count()
    return x


def softmax_rows(x: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Row soft-max of ``scale * x`` for a 2-D bf16 matrix (columns a multiple of 8)."""
    if not x.is_cuda:
        return reference.softmax_rows(x, scale)
    x = _rowmajor(x)
    rows, cols = x.shape
    y = torch.empty_like(x)
    lib = _lib.load()
    _chk(lib.cs_softmax_rows(x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), rows, cols, float(scale),
                             _stream()), "cs_softmax_rows")
    _count()
    return y


def im2col3x3(x: torch.Tensor, B: int, H: int, W: int, up: int = 1, silu: bool = False, stride: int = 1) -> torch.Tensor:
    """Channels-last image ``[B*H*W, C]`` -> ``[B*Ho*Wo, 9 C]`` GEMM operand of a 3x3 convolution with padding 1
    (``Ho = (up*H - 1) // stride + 1``)."""
    if not x.is_cuda:
        return reference.im2col3x3(x, B, H, W, up, silu, stride)
    C = x.shape[-1]
    assert x.is_contiguous() and x.dtype == torch.bfloat16
    Ho, Wo = (H * up - 1) // stride + 1, (W * up - 1) // stride + 1
    out = torch.empty((B * Ho * Wo, 9 * C), device=x.device, dtype=x.dtype)
    lib = _lib.load()
    _chk(lib.cs_im2col3x3(x.data_ptr(), out.data_ptr(), B, H, W, C, up, 1 if silu else 0, stride, _stream()),
         "cs_im2col3x3")
    _count()
    return out


def im2col1d(x: torch.Tensor, B: int, T: int, To: int, taps: int, first: int, dilation: int = 1,
             alpha: torch.Tensor | None = None, beta: torch.Tensor | None = None, stride: int = 1) -> torch.Tensor:
    """Channels-last sequence ``[B*T, C]`` -> ``[B*To, taps*C]``: row ``t``, tap ``j`` reads time
    ``t*stride + first + j*dilation``; with ``alpha``/``beta`` (fp32 ``[C]``) SnakeBeta is applied on the fly."""
    if not x.is_cuda:
        return reference.im2col1d(x, B, T, To, taps, first, dilation, alpha, beta, stride)
    C = x.shape[-1]
    assert x.is_contiguous() and x.dtype == torch.bfloat16
    out = torch.empty((B * To, taps * C), device=x.device, dtype=x.dtype)
    lib = _lib.load()
    _chk(lib.cs_im2col1d(x.data_ptr(), out.data_ptr(), B, T, To, C, taps, first, dilation, stride,
                         0 if alpha is None else 1, _ptr(alpha), _ptr(beta), _stream()), "cs_im2col1d")
    _count()
    return out


def dwconv1d(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, B: int, T: int) -> torch.Tensor:
    """Depth-wise causal 1-D convolution on ``[B*T, C]`` with ``w`` = ``[C, k]``."""
    if not x.is_cuda:
        return reference.dwconv1d(x, w, bias, B, T)
    C, k = w.shape
    y = torch.empty_like(x)
    lib = _lib.load()
    _chk(lib.cs_dwconv1d(x.data_ptr(), y.data_ptr(), w.data_ptr(), _ptr(bias), B, T, C, k, _stream()), "cs_dwconv1d")
    _count()
    return y


def to_rgb8(x: torch.Tensor) -> torch.Tensor:
    """Channels-last image rows ``[pixels, >=3]`` in [-1, 1] -> uint8 ``[pixels, 3]``."""
    if not x.is_cuda:
        return reference.to_rgb8(x)
    y = torch.empty((x.shape[0], 3), device=x.device, dtype=torch.uint8)
    lib = _lib.load()
    _chk(lib.cs_to_rgb8(x.data_ptr(), x.stride(0), y.data_ptr(), x.shape[0], _stream()), "cs_to_rgb8")
    _count()
    return y


def conv3x3(x: torch.Tensor, w2d: torch.Tensor, bias: torch.Tensor | None, B: int, H: int, W: int, *, up: int = 1,
            silu: bool = False, residual: torch.Tensor | None = None, stride: int = 1, act: str | None = None) -> torch.Tensor:
    """3x3 convolution (padding 1) on a channels-last image; ``w2d`` is ``[Cout, 9*Cin]`` in (ky, kx, cin) order.
    ``silu`` applies SiLU to the input first, ``up=2`` convolves the nearest-neighbour 2x upsampled image."""
    cols = im2col3x3(x, B, H, W, up, silu, stride)
    return linear(cols, w2d, bias, residual=residual, act=act)


def conv1d_causal(x: torch.Tensor, w2d: torch.Tensor, bias: torch.Tensor | None, B: int, T: int, k: int,
                  dilation: int = 1, *, alpha=None, beta=None, residual: torch.Tensor | None = None) -> torch.Tensor:
    """Causal dilated 1-D convolution on ``[B*T, Cin]``; ``w2d`` is ``[Cout, k*Cin]`` in (tap, cin) order.  With
    ``alpha``/``beta`` SnakeBeta is applied to the input on the fly."""
    if k == 1 and alpha is None:
        return linear(x, w2d, bias, residual=residual)
    cols = im2col1d(x, B, T, T, k, -(k - 1) * dilation, dilation, alpha, beta)
    return linear(cols, w2d, bias, residual=residual)


def conv_transpose1d_causal(x: torch.Tensor, w2d: torch.Tensor, bias_rep: torch.Tensor | None, B: int, T: int,
                            stride: int, kernel: int, *, alpha=None, beta=None) -> tuple[torch.Tensor, int]:
    """Transposed 1-D convolution with the trimming used by causal vocoders.

    ``kernel == stride``: every input step yields ``stride`` outputs (``w2d`` = ``[stride*Cout, Cin]``).
    ``kernel == 2*stride``: outputs are trimmed by ``stride`` on both sides, so output ``(t-1)*stride + p`` is
    ``W[:, :, p] x[t] + W[:, :, p + stride] x[t-1]`` for ``t`` in ``1..T-1`` (``w2d`` = ``[stride*Cout, 2*Cin]``,
    input taps ordered (x[t], x[t-1])).  Returns ``([B*To, Cout], To)``."""
    if kernel == stride:
        xin = x if alpha is None else im2col1d(x, B, T, T, 1, 0, 1, alpha, beta)
        y = linear(xin, w2d, bias_rep)
        return y.view(B * T * stride, -1), T * stride
    assert kernel == 2 * stride
    # rows t = 1..T-1: taps (x[t], x[t-1])  ->  first = +1 with dilation -1
    cols = im2col1d(x, B, T, T - 1, 2, 1, -1, alpha, beta)
    y = linear(cols, w2d, bias_rep)
    return y.view(B * (T - 1) * stride, -1), (T - 1) * stride


def bilinear_embed_add_(x: torch.Tensor, table: torch.Tensor, idx: torch.Tensor, wgt: torch.Tensor) -> torch.Tensor:
    """``x[l] += sum_i wgt[i, l] * table[idx[i, l]]`` for ``idx``/``wgt`` of shape ``[4, L]`` (int32 / fp32): the
    bilinear interpolation of a learned 2-D position table, added in place."""
    if not x.is_cuda:
        pos = (table.float()[idx.long()] * wgt.float()[:, :, None]).sum(0)
        x.copy_((x.float() + pos).to(x.dtype))
        return x
    L, H = x.shape
    assert x.stride(1) == 1 and table.stride(1) == 1 and idx.dtype == torch.int32 and wgt.dtype == torch.float32
    lib = _lib.load()
    _chk(lib.cs_bilinear_embed_add(x.data_ptr(), x.stride(0), table.data_ptr(), table.stride(0), idx.contiguous().data_ptr(),
                                   wgt.contiguous().data_ptr(), L, H, _stream()), "cs_bilinear_embed_add")
    _count()
    return x


def kv_copy_pages(dst: torch.Tensor, src: torch.Tensor, src_pages: torch.Tensor, dst_pages: torch.Tensor) -> None:
    """``dst[:, dst_pages[i]] = src[:, src_pages[i]]`` for KV caches ``[layers, pages, ...]`` (page-contiguous).

    ``src`` may live on another GPU of the node or belong to another process (a CUDA-IPC mapping): the kernel runs on
    ``dst``'s device and reads the pages over NVLink.  Page lists are int32 tensors on ``dst``'s device."""
    assert dst.shape[0] == src.shape[0] and dst.shape[2:] == src.shape[2:] and dst.dtype == src.dtype
    if not dst.is_cuda:
        dst[:, dst_pages.long()] = src[:, src_pages.long()]
        return
    assert src.is_cuda and dst[0, 0].is_contiguous() and src[0, 0].is_contiguous()
    lib = _lib.load()
    if src.device != dst.device:
        with torch.cuda.device(dst.device):
            rc = lib.cs_enable_peer_access(src.device.index)
        if rc != 0:
            raise RuntimeError(f"{dst.device} cannot read the memory of {src.device} (code {rc})")
    page_bytes = dst[0, 0].numel() * dst.element_size()
    with torch.cuda.device(dst.device):
        _chk(lib.cs_kv_copy_pages(dst.data_ptr(), src.data_ptr(), dst.stride(0) * dst.element_size(),
                                  src.stride(0) * src.element_size(), page_bytes, dst.shape[0], int(src_pages.numel()),
                                  dst.shape[1], src.shape[1], src_pages.data_ptr(), dst_pages.data_ptr(), _stream()),
             "cs_kv_copy_pages")
    _count()


# ---------------------------------------------------------------------------------------------------------
# fp8 (e4m3) linear layers with block scales: 1 x 128 blocks of the activations, 128 x 128 blocks of the weight
# ---------------------------------------------------------------------------------------------------------
FP8_MAX = 448.0


def quantize_fp8_weight(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``w`` ``[N, K]`` (``K % 128 == 0``) -> ``(wq [N, K] float8_e4m3fn, scales [ceil(N/128), K/128] fp32)``; done once
    per checkpoint, so plain tensor ops."""
    N, K = w.shape
    assert K % 128 == 0
    nb = -(-N // 128)
    wp = torch.zeros((nb * 128, K), device=w.device, dtype=torch.float32)
    wp[:N] = w.float()
    blocks = wp.view(nb, 128, K // 128, 128)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / FP8_MAX, torch.ones_like(amax))
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX).view(nb * 128, K)[:N]
    return q.to(torch.float8_e4m3fn).contiguous(), scale.contiguous()


def quantize_fp8_rows(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``x`` ``[M, K]`` bf16 -> ``(xq [M, K] float8_e4m3fn, scales [K/128, M] fp32)``: one scale per row and 128 columns."""
    M, K = x.shape
    assert K % 128 == 0
    if not x.is_cuda:
        b = x.float().view(M, K // 128, 128)
        amax = b.abs().amax(dim=2)
        scale = torch.where(amax > 0, amax * (1.0 / FP8_MAX), torch.ones_like(amax))  # same arithmetic as the kernel
        q = (b * (1.0 / scale)[:, :, None]).clamp(-FP8_MAX, FP8_MAX).view(M, K).to(torch.float8_e4m3fn)
        return q, scale.t().contiguous()
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    q = torch.empty((M, K), device=x.device, dtype=torch.float8_e4m3fn)
    scales = torch.empty((K // 128, M), device=x.device, dtype=torch.float32)
    lib = _lib.load()
    _chk(lib.cs_quant_fp8_rows(x.data_ptr(), x.stride(0), M, K, q.data_ptr(), q.stride(0), scales.data_ptr(), scales.stride(0),
                               _stream()), "cs_quant_fp8_rows")
    _count()
    return q, scales


def linear_fp8(x: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor, bias: torch.Tensor | None = None,
               xq: tuple[torch.Tensor, torch.Tensor] | None = None) -> torch.Tensor:
    """``x @ dequant(wq).T + bias`` with the activations quantised on the fly (or given as ``xq``): the product of every
    128-wide K block is scaled and summed in fp32 by the GEMM kernel itself.  Returns bf16 (fp32 on the CPU)."""
    M, K = x.shape
    N = wq.shape[0]
    q, sa = xq if xq is not None else quantize_fp8_rows(x)
    if not x.is_cuda:
        a = (q.float().view(M, K // 128, 128) * sa.t()[:, :, None]).view(M, K)
        nb = w_scale.shape[0]
        wp = torch.zeros((nb * 128, K), dtype=torch.float32)
        wp[:N] = wq.float()
        w = (wp.view(nb, 128, K // 128, 128) * w_scale[:, None, :, None]).view(nb * 128, K)[:N]
        y = a @ w.t()
        return y if bias is None else y + bias.float()
    _on_current_device(x)
    assert wq.dtype == torch.float8_e4m3fn and wq.is_contiguous() and w_scale.is_contiguous() and w_scale.dtype == torch.float32
    out = torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
    lib = _lib.load()
    _chk(lib.cs_gemm_fp8_blockscaled(q.data_ptr(), q.stride(0), wq.data_ptr(), wq.stride(0), sa.data_ptr(), sa.stride(0),
                                     w_scale.data_ptr(), out.data_ptr(), out.stride(0), _ptr(bias), M, N, K, _stream()),
         "cs_gemm_fp8_blockscaled")
    _count()
    return out
