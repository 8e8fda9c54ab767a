"""Python front-ends of the fused compute+collective kernels."""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from ..ops import _lib
from ..ops import _ptr, _skinny_workspace, _stream, _count  # noqa: F401  (shared helpers)
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
        return h, normed
