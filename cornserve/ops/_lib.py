"""ctypes loader for ``libcornserve.so``.

The library is built in-tree by ``cornserve.ops.build``.  On a machine with a GPU a missing
library is an error (no silent fallback); on a CPU-only machine the bindings are simply not used.
"""

from __future__ import annotations

import ctypes
import threading
from ctypes import c_float, c_int, c_longlong, c_uint, c_void_p
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "libcornserve.so"
_lock = threading.Lock()
_lib: ctypes.PyDLL | None = None

ERROR_NAMES = {
    0: "ok",
    1: "timeout waiting for a TMA tile",
    2: "timeout waiting for tcgen05.commit",
    3: "timeout waiting for a free pipeline slot",
    4: "timeout waiting for a peer flag",
    5: "bad argument",
    6: "timeout waiting for the epilogue",
}

P, I, L, F, U = c_void_p, c_int, c_longlong, c_float, c_uint

_SIGNATURES = {
    "cs_last_error": ([], I),
    "cs_reset_error": ([], None),
    "cs_sm_count": ([], I),
    "cs_abi_version": ([], I),
    "cs_gemm_bf16": ([P, L, P, L, P, L, P, P, L, P, L, I, I, I, I, I, I, I, I, I, P], I),
    "cs_gemm_skinny": ([P, L, P, L, P, L, P, P, L, I, I, I, I, I, I, I, P, L, P, I, P], I),
    "cs_gemm_skinny_ws_bytes": ([I, I, I, I], L),
    "cs_gemm_skinny_auto_splits": ([I, I, I], I),
    "cs_norm": ([P, L, P, L, P, L, P, P, P, P, L, I, P, L, I, I, F, I, P], I),
    "cs_rope": ([P, L, I, I, I, I, P, P], I),
    "cs_mrope_table": ([P, I, I, F, I, I, P, P], I),
    "cs_rope_kv_write": ([P, L, I, I, I, I, P, P, P, I, P], I),
    "cs_act_mul": ([P, L, P, L, I, I, I, P], I),
    "cs_gather_rows": ([P, L, P, L, P, I, L, I, P], I),
    "cs_push_bytes": ([P, P, L, P], I),
    "cs_apply_penalties": ([P, L, P, L, P, P, I, I, P], I),
    "cs_count_tokens": ([P, L, P, P, I, I, P], I),
    "cs_argmax": ([P, L, I, I, I, P, P, P], I),
    "cs_flow_step": ([P, P, P, I, I, F, F, I, P], I),
    "cs_pcm16": ([P, P, L, P], I),
    "cs_l2_flush": ([P, L, U, P], I),
    "cs_decode_advance": ([P, P, P, P, P, P, I, P, P, I, P, I, I, P], I),
    "cs_attention_decode": ([P, L, P, P, L, P, P, I, I, I, I, I, F, I, P, L, P], I),
    "cs_head_norm_rope": ([P, L, L, I, I, P, F, P, P, I, I, P], I),
    "cs_qk_norm_rope128": ([P, L, L, I, L, P, P, P, P, F, P, I, I, P], I),
    "cs_sample_rows": ([P, L, I, I, P, P, P, P, P, P, P], I),
    "cs_softmax_rows": ([P, L, P, L, I, I, F, P], I),
    "cs_im2col3x3": ([P, P, I, I, I, I, I, I, I, P], I),
    "cs_im2col1d": ([P, P, I, I, I, I, I, I, I, I, I, P, P, P], I),
    "cs_dwconv1d": ([P, P, P, P, I, I, I, I, P], I),
    "cs_bilinear_embed_add": ([P, L, P, L, P, P, L, I, P], I),
    "cs_gemm_fp8_blockscaled": ([P, L, P, L, P, L, P, P, L, P, I, I, I, P], I),
    "cs_quant_fp8_rows": ([P, L, I, I, P, L, P, L, P], I),
    "cs_kv_copy_pages": ([P, P, L, L, L, I, I, I, I, P, P, P], I),
    "cs_enable_peer_access": ([I], I),
    "cs_to_rgb8": ([P, L, P, L, P], I),
    "cs_attention": ([P, L, P, L, P, L, P, L, P, P, P, P, I, I, I, I, I, I, I, I, I, F, I, I, I, P, L, I, P, P, P], I),
}


def lib_path() -> Path:
    return _LIB_PATH


def available() -> bool:
    return _LIB_PATH.exists()


def load() -> ctypes.PyDLL:
    """Load the kernel library (once) and declare the argument types of every entry point.

    Every entry point only enqueues work on a stream, a few microseconds, so calls keep the interpreter lock
    (``PyDLL``): giving it up around each launch would let a busy thread of the same process take it for a whole
    switch interval, once per kernel."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build it with `python -m cornserve.ops.build` "
                "(the CUDA path never falls back to PyTorch kernels)"
            )
        lib = ctypes.PyDLL(str(_LIB_PATH))
        for name, (argtypes, restype) in _SIGNATURES.items():
            if not hasattr(lib, name):
                continue
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = lib
        return lib


def register_signature(name: str, argtypes: list, restype) -> None:
    """Let other modules (e.g. ``parallel``) declare entry points that live in the same library."""
    _SIGNATURES[name] = (argtypes, restype)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


def check_error(where: str = "") -> None:
    """Raise if any kernel recorded an error (bounded wait ran out) since the last reset."""
    lib = load()
    code = lib.cs_last_error()
    if code != 0:
        lib.cs_reset_error()
        raise RuntimeError(f"kernel error {code} ({ERROR_NAMES.get(code, '?')}) {where}")
