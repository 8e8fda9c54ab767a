"""Wire encoding of sidecar payloads (msgpack), reference: python/cornserve/sidecar/serde.py.

Three payload kinds travel in the ``data`` bytes of Send / PrepareReceive / Receive:

* ``obj``    small Python objects (dict, str, int, ...), inline
* ``inline`` a CPU tensor, inline as raw bytes (CPU deployments and tests)
* ``ipc``    a CUDA tensor as a CUDA-IPC reference (the arguments ``torch.multiprocessing.reductions``
             produces), so only a handle crosses the process boundary
* ``slab``   a region of a sidecar's slab: ``(rank, offset, numel, dtype, shape)``; receivers map the
             slab of ``rank`` once and read the region in place
"""

from __future__ import annotations

from typing import Any

import msgpack
import torch

_DTYPES = {str(d).removeprefix("torch."): d for d in (
    torch.float32, torch.float64, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.int16,
    torch.int8, torch.uint8, torch.bool)}


def dtype_name(d: torch.dtype) -> str:
    return str(d).removeprefix("torch.")


def dtype_from_name(s: str) -> torch.dtype:
    return _DTYPES[s.removeprefix("torch.")]


def encode_obj(obj: Any) -> bytes:
    return msgpack.packb({"kind": "obj", "obj": obj}, use_bin_type=True)


def encode_inline_tensor(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    raw = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
    return msgpack.packb({"kind": "inline", "dtype": dtype_name(t.dtype), "shape": list(t.shape), "raw": raw},
                         use_bin_type=True)


def encode_ipc_tensor(t: torch.Tensor) -> bytes:
    """The tensor must stay alive until the receiver has rebuilt (and copied) it."""
    from ..utils.cuda_ipc import export_tensor

    return msgpack.packb({"kind": "ipc", "dtype": dtype_name(t.dtype), "shape": list(t.shape),
                          "handle": export_tensor(t)}, use_bin_type=True)


def encode_slab_ref(rank: int, offset: int, nbytes: int, dtype: torch.dtype, shape: list[int]) -> bytes:
    """``nbytes`` bytes at byte ``offset`` of sidecar ``rank``'s slab hold a tensor of ``dtype`` and ``shape``."""
    return msgpack.packb({"kind": "slab", "rank": rank, "offset": offset, "nbytes": nbytes,
                          "dtype": dtype_name(dtype), "shape": list(shape)}, use_bin_type=True)


def decode(data: bytes) -> dict[str, Any]:
    return msgpack.unpackb(data, raw=False)


def tensor_from_inline(msg: dict[str, Any]) -> torch.Tensor:
    dt = dtype_from_name(msg["dtype"])
    if not msg["raw"]:
        return torch.empty(msg["shape"], dtype=dt)
    return torch.frombuffer(bytearray(msg["raw"]), dtype=torch.uint8).view(dt).view(msg["shape"])


def tensor_from_ipc(msg: dict[str, Any]) -> torch.Tensor:
    from ..utils.cuda_ipc import import_tensor

    return import_tensor(msg["handle"])
