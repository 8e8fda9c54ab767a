"""Python front-ends of the fused compute+collective kernels."""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..ops import _lib
from ..ops import _ptr, _skinny_workspace, _stream, _count, count_path  # noqa: F401  (shared helpers)
from .fabric import Fabric, SymmetricBuffer
from .state import ParallelGroup

P, I, L, F = c_void_p, c_int, c_longlong, c_float
_lib.register_signature("cs_gemm_skinny_allreduce",
                        [P, L, P, L, P, L, P, P, L, P, P, L, F, I, I, I, I, P, L, P, I, I, I, P, P, I, I, I, P, P, P, P], I)


class FusedRowParallel:
    """``h = all_reduce(x @ w.T) + residual`` and ``RMSNorm(h)`` in ONE kernel per rank (decode-time
    o_proj / down_proj of a tensor-parallel LLM).  Partial tiles travel GPU-to-GPU as plain peer stores from
    the GEMM epilogue; there is no NCCL call.  One instance serves every projection with the same output
    width ``n`` (they share receive buffers and arrival counters, which all ranks advance in lock-step).
    """

    def __init__(self, group: ParallelGroup, n: int, m_cap: int = 256):
        if group.fabric is None:
            raise RuntimeError("FusedRowParallel needs the peer-memory fabric")
        self.group, self.n, self.m_cap = group, n, m_cap
        self.n_cap = (n + 7) // 8 * 8
        self.tiles_cap = (n + 127) // 128
        fab: Fabric = group.fabric
        self.recv: SymmetricBuffer = fab.alloc(2 * group.size * m_cap * self.n_cap, torch.bfloat16)
        self.flags: SymmetricBuffer = fab.alloc(2 * self.tiles_cap, torch.int32)
        dev = group.device
        self.ssq = torch.zeros(m_cap, device=dev, dtype=torch.float32)
        self.done = torch.zeros(2, device=dev, dtype=torch.int32)
        self.epoch = torch.zeros(1, device=dev, dtype=torch.int32)
        self._recv_ptrs = self.recv.ptr_array()
        self._flag_ptrs = self.flags.ptr_array()

    def __call__(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, residual: torch.Tensor | None,
                 norm_w: torch.Tensor | None, eps: float = 1e-6, splits: int = 0):
        """Returns ``(h, normed)``; ``normed`` is ``None`` without ``norm_w``."""
        M, K = x.shape
        N = w.shape[0]
        assert N == self.n and M <= self.m_cap and x.dtype == torch.bfloat16
        h = torch.empty((M, N), device=x.device, dtype=torch.bfloat16)
        normed = torch.empty_like(h) if norm_w is not None else None
        ws, counters = _skinny_workspace(x.device)
        lib = _lib.load()
        rc = lib.cs_gemm_skinny_allreduce(
            x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), h.data_ptr(), h.stride(0),
            _ptr(bias if self.group.is_first else None), _ptr(residual), 0 if residual is None else residual.stride(0),
            _ptr(norm_w), _ptr(normed), N, float(eps), M, N, K, splits, ws.data_ptr(), ws.numel(),
            counters.data_ptr(), counters.numel(), self.group.size, self.group.rank,
            ctypes.cast(self._recv_ptrs, c_void_p), ctypes.cast(self._flag_ptrs, c_void_p),
            self.m_cap, self.n_cap, self.tiles_cap, self.ssq.data_ptr(), self.done.data_ptr(), self.epoch.data_ptr(),
            _stream())
        if rc != 0:
            raise RuntimeError(f"cs_gemm_skinny_allreduce failed with code {rc}")
        _count()
        count_path("llm_gemm_allreduce_norm")
        return h, normed


# ------------------------------------------------------------------------------------------------------------
# Tensor-parallel encoder blocks: all-gather -> GEMM and GEMM -> reduce-scatter without library collectives
# ------------------------------------------------------------------------------------------------------------
from ctypes import c_uint  # noqa: E402

import torch.distributed as dist  # noqa: E402

_lib.register_signature("cs_gemm_bf16_tp",
                        [P, L, P, L, P, L, P, I, I, I, I, I, I, P, I, c_uint, I, I, I, P, P, I, L, P], I)
_lib.register_signature("cs_tp_reduce_norm_push",
                        [I, I, I, I, I, P, L, P, c_uint, P, P, L, P, L, P, F, P, I, P, P, L, I, P], I)

_ACTS = {"none": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "quick_gelu": 4, "relu": 5}


class FusedEncoderTP:
    """Peer-memory plumbing of a tensor-parallel encoder tower whose activations are sharded by rows between blocks.

    Per half-block three kernels run on every rank and meet only through counters in peer memory:

    * :meth:`gemm_push` - row-parallel GEMM whose epilogue stores bf16 partial tiles straight into the receive buffer
      of the rank that owns the rows (the reduce-scatter is the GEMM's store);
    * :meth:`reduce_norm_push` - per owned row: wait for all partials, add bias + residual, keep the new residual
      shard, RMSNorm, write the normalised row into every rank's operand buffer (the all-gather is this store);
    * :meth:`gemm_gathered` - column-parallel GEMM whose TMA producer waits per 128-row chunk of that operand.

    ``begin(S)`` is called once per forward pass: it fixes the row ownership (``rows_per_rank`` a multiple of 128),
    clears the counters and meets the peers once (the only library collective of the pass).
    Operand buffers: 0 and 1 alternate between the attention and MLP halves; 2 is read four rows at a time by the
    patch merger.
    """

    def __init__(self, group: ParallelGroup, hidden: int, max_rows: int):
        if group.fabric is None:
            raise RuntimeError("FusedEncoderTP needs the peer-memory fabric")
        self.group, self.H = group, hidden
        T = group.size
        self.R_cap = -(-max_rows // (T * 128)) * 128
        self.S_cap = self.R_cap * T
        fab: Fabric = group.fabric
        self.gather = [fab.alloc(self.S_cap * hidden, torch.bfloat16, zero=False) for _ in range(3)]
        self.recv = fab.alloc(T * self.R_cap * hidden, torch.bfloat16, zero=False)
        # Two sets of arrival counters, used by alternate passes.  A pass starts by clearing the set of the NEXT pass
        # on its own stream, so no rank ever has to wait for the others before it pushes: a peer can only be one pass
        # ahead, and it reaches that pass only after this rank's pushes of the current one, which are ordered behind
        # the clear.  (Every push of a pass is awaited by a kernel of the same pass on the receiving rank, so the set
        # of the previous pass is quiet by the time it is cleared.)  The allocation itself is collective and zeroed.
        self._gflag_sets = [[fab.alloc(self.S_cap // 128 + 1, torch.int32) for _ in range(3)] for _ in range(2)]
        self._rflag_sets = [fab.alloc(self.R_cap // 128 + 1, torch.int32) for _ in range(2)]
        self._gptr = [b.ptr_array() for b in self.gather]
        self._gfptr_sets = [[b.ptr_array() for b in fs] for fs in self._gflag_sets]
        self._rptr = self.recv.ptr_array()
        self._rfptr_sets = [b.ptr_array() for b in self._rflag_sets]
        self.cur = 1
        self.S = self.R = self.rows_local = 0
        self.g_epoch = [0, 0, 0]
        self.r_epoch = 0
        self._last_push_tiles_n = 0

    @property
    def gflags(self):
        return self._gflag_sets[self.cur]

    @property
    def rflags(self):
        return self._rflag_sets[self.cur]

    @property
    def _gfptr(self):
        return self._gfptr_sets[self.cur]

    @property
    def _rfptr(self):
        return self._rfptr_sets[self.cur]

    def begin(self, S: int) -> None:
        T, r = self.group.size, self.group.rank
        R = -(-S // (T * 128)) * 128
        if R > self.R_cap:
            raise ValueError(f"{S} rows exceed the capacity of this fused context ({self.S_cap})")
        self.S, self.R = S, R
        self.rows_local = max(0, min(R, S - r * R))
        self.cur ^= 1
        nxt = self.cur ^ 1
        for f in (*self._gflag_sets[nxt], self._rflag_sets[nxt]):   # the counters of the pass after this one
            f.local.zero_()
        self.g_epoch = [0, 0, 0]
        self.r_epoch = 0

    @property
    def row_range(self) -> tuple[int, int]:
        lo = self.group.rank * self.R
        return lo, lo + self.rows_local

    # -- kernels ---------------------------------------------------------------------------------------------
    def reduce_norm_push(self, *, bias: torch.Tensor | None, residual: torch.Tensor, norm_w: torch.Tensor | None, eps: float,
                         dst: int | None, reduce: bool = True, gather_chunk: int = 128, norm_b: torch.Tensor | None = None,
                         layer_norm: bool = False) -> torch.Tensor:
        """``x' = sum_ranks(partials) + bias + residual`` on this rank's rows (``reduce=False``: ``x' = residual``),
        then ``RMSNorm(x')`` (or ``LayerNorm`` with ``norm_b``) pushed into operand buffer ``dst`` of every rank.
        Returns ``x'`` (the residual shard)."""
        g = self.group
        rows, H = self.rows_local, self.H
        x_out = torch.empty((rows, H), device=g.device, dtype=torch.bfloat16) if reduce else residual
        if dst is not None:
            self.g_epoch[dst] += 1
        lib = _lib.load()
        rc = lib.cs_tp_reduce_norm_push(
            rows, H, g.size, g.rank, self.R,
            self.recv.local.data_ptr() if reduce else None, H, self.rflags.local.data_ptr(),
            self.r_epoch * self._last_push_tiles_n * g.size,
            _ptr(bias) if reduce else None, residual.data_ptr(), residual.stride(0),
            x_out.data_ptr() if reduce else None, H, _ptr(norm_w), float(eps), _ptr(norm_b), 1 if layer_norm else 0,
            ctypes.cast(self._gptr[dst], c_void_p) if dst is not None else None,
            ctypes.cast(self._gfptr[dst], c_void_p) if dst is not None else None, H, gather_chunk, _stream())
        if rc != 0:
            raise RuntimeError(f"cs_tp_reduce_norm_push failed with code {rc}")
        _count()
        count_path("encoder_reduce_norm_allgather")
        return x_out

    def gemm_gathered(self, src: int, w: torch.Tensor, bias: torch.Tensor | None, *, act: str | None = None,
                      swiglu: bool = False, a_rpr: int = 1) -> torch.Tensor:
        """``act(A w.T + bias)`` where ``A`` is operand buffer ``src`` (``[S / a_rpr, a_rpr * H]``), consumed chunk by
        chunk as the peers' rows land."""
        g = self.group
        M, K = self.S // a_rpr, self.H * a_rpr
        N = w.shape[0] // (2 if swiglu else 1)
        out = torch.empty((M, N), device=g.device, dtype=torch.bfloat16)
        m_rot = (g.rank * self.R // a_rpr) // 128
        lib = _lib.load()
        rc = lib.cs_gemm_bf16_tp(
            self.gather[src].local.data_ptr(), K, w.data_ptr(), w.stride(0), out.data_ptr(), N, _ptr(bias), M, N, K,
            _ACTS[act or "none"], 1 if swiglu else 0, 0, self.gflags[src].local.data_ptr(), a_rpr, self.g_epoch[src], m_rot,
            0, 0, None, None, 128, 0, _stream())
        if rc != 0:
            raise RuntimeError(f"cs_gemm_bf16_tp (gathered) failed with code {rc}")
        _count()
        count_path("encoder_allgather_gemm")
        return out

    def gemm_push(self, x: torch.Tensor, w: torch.Tensor) -> None:
        """Row-parallel ``x w.T``: this rank's partial sums travel to the owners of the rows from the epilogue."""
        g = self.group
        M, K = x.shape
        N = w.shape[0]
        assert M == self.S and N == self.H and x.stride(1) == 1
        tiles_m = -(-M // 128)
        bn = 256 if tiles_m * -(-N // 256) >= 148 else 128
        self._last_push_tiles_n = -(-N // bn)
        self.r_epoch += 1
        lib = _lib.load()
        rc = lib.cs_gemm_bf16_tp(
            x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), None, 0, None, M, N, K, 0, 0, bn, None, 1, 0,
            (((g.rank + 1) % g.size) * self.R) // 128, g.size, g.rank, ctypes.cast(self._rptr, c_void_p), ctypes.cast(self._rfptr, c_void_p),
            self.R, self.H, _stream())
        if rc != 0:
            raise RuntimeError(f"cs_gemm_bf16_tp (push) failed with code {rc}")
        _count()
        count_path("encoder_gemm_reducescatter")


# ------------------------------------------------------------------------------------------------------------
# Ulysses sequence parallelism for the diffusion transformer without library all-to-all
# ------------------------------------------------------------------------------------------------------------
_lib.register_signature("cs_gemm_bf16_a2a", [P, L, P, L, P, I, I, I, I, I, P, P, L, I, I, I, I, I, I, P], I)
_lib.register_signature("cs_a2a_push_heads", [P, L, I, I, I, I, I, P, L, P, P, P], I)
_lib.register_signature("cs_wait_flag", [P, c_uint, P], I)


class FusedUlysses:
    """Token shards outside attention, head shards inside it, with the exchanges done by the kernels themselves:

    * the q|k|v projection's epilogue stores every 128-column head tile straight into the buffer of the rank that
      owns the head (:meth:`qkv_scatter`), so the "tokens -> heads" all-to-all is the GEMM's store;
    * after attention one copy kernel returns every rank's head slice of every token to the token's owner
      (:meth:`push_heads`), landing in the operand buffer of the output projection;
    * consumers are ordered behind the peers' stores by one-thread wait kernels (bounded) on arrival counters.

    ``begin_pass`` (once per denoiser forward) clears the counters and meets the peers once.
    """

    def __init__(self, group: ParallelGroup, hidden: int, heads: int, head_dim: int, max_local_rows: int):
        if group.fabric is None:
            raise RuntimeError("FusedUlysses needs the peer-memory fabric")
        self.group, self.D, self.H, self.d = group, hidden, heads, head_dim
        Pn = group.size
        self.Hl = heads // Pn
        self.own = self.Hl * head_dim
        if self.own % 128 or hidden % 128:
            raise ValueError("head slices must be multiples of 128 columns")
        self.cap = max_local_rows
        fab: Fabric = group.fabric
        self.qkv = fab.alloc(Pn * max_local_rows * 3 * self.own, torch.bfloat16, zero=False)
        self.o = fab.alloc(max_local_rows * hidden, torch.bfloat16, zero=False)
        # The arrival counters only ever grow (every rank makes the same calls, so every rank knows the value a counter
        # must reach): nothing is cleared between passes and no rank waits for the others before it pushes.  32 bits
        # last for 2^32 tiles, i.e. months of continuous denoising.
        self.qkv_flag = fab.alloc(4, torch.int32)
        self.o_flag = fab.alloc(4, torch.int32)
        self._qkv_ptr, self._qkv_fptr = self.qkv.ptr_array(), self.qkv_flag.ptr_array()
        self._o_ptr, self._o_fptr = self.o.ptr_array(), self.o_flag.ptr_array()
        self.done = torch.zeros(1, device=group.device, dtype=torch.int32)
        self.qkv_expected = 0
        self.o_expected = 0

    def begin_pass(self) -> None:
        """Start of a denoiser forward.  Nothing to do on the device: the counters are cumulative."""

    def qkv_scatter(self, x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None, row0: int, run: int, stride: int,
                    seg: int) -> None:
        """``x w.T + bias`` with ``w`` = ``[3D, D]``, scattered by head owner.  Row ``m`` of ``x`` is row
        ``row0 + (m // run) * stride + m % run`` of this rank's token order (one stream of every sample in one call);
        ``seg`` = this rank's rows per sample."""
        g = self.group
        M, K = x.shape
        lib = _lib.load()
        rc = lib.cs_gemm_bf16_a2a(x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), _ptr(bias), M, 3 * self.D, K, g.size, g.rank,
                                  ctypes.cast(self._qkv_ptr, c_void_p), ctypes.cast(self._qkv_fptr, c_void_p), 3 * self.own,
                                  self.D, self.own, seg, row0, run, stride, _stream())
        if rc != 0:
            raise RuntimeError(f"cs_gemm_bf16_a2a failed with code {rc}")
        _count()
        count_path("ulysses_qkv_alltoall")
        # every rank makes the same calls: each delivers tiles_m x (3 * own / 128) tiles to every destination
        self.qkv_expected = (self.qkv_expected + g.size * (-(-M // 128)) * (3 * self.own // 128)) & 0xFFFFFFFF

    def gathered_qkv(self, rows_total: int) -> torch.Tensor:
        """Waits for all ranks' tiles, then returns ``[rows_total, 3 * own]`` (this rank's heads, every token)."""
        lib = _lib.load()
        lib.cs_wait_flag(self.qkv_flag.local.data_ptr(), self.qkv_expected, _stream())
        _count()
        return self.qkv.local[: rows_total * 3 * self.own].view(rows_total, 3 * self.own)

    def push_heads(self, o_full: torch.Tensor, seg: int) -> torch.Tensor:
        """``o_full`` = ``[world * rows_local, own]`` (every token, this rank's heads) -> ``[rows_local, D]`` with all heads."""
        g = self.group
        rows_total = o_full.shape[0]
        lib = _lib.load()
        rc = lib.cs_a2a_push_heads(o_full.data_ptr(), o_full.stride(0), rows_total, self.own, g.size, g.rank, seg,
                                   ctypes.cast(self._o_ptr, c_void_p), self.D, ctypes.cast(self._o_fptr, c_void_p),
                                   self.done.data_ptr(), _stream())
        if rc != 0:
            raise RuntimeError(f"cs_a2a_push_heads failed with code {rc}")
        self.o_expected = (self.o_expected + g.size) & 0xFFFFFFFF
        lib.cs_wait_flag(self.o_flag.local.data_ptr(), self.o_expected, _stream())
        _count(2)
        count_path("ulysses_head_return")
        rows_local = rows_total // g.size
        return self.o.local[: rows_local * self.D].view(rows_local, self.D)
