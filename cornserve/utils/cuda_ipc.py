"""CUDA-IPC tensor handles as plain data.

``torch.multiprocessing.reductions.reduce_tensor`` describes a CUDA tensor by a tuple that another process of the
same machine can turn back into a tensor over the same memory.  That tuple holds classes and byte strings, so the
obvious way to ship it is pickle, and unpickling bytes that arrived over HTTP or gRPC runs whatever they say.  Here
the tuple is flattened into JSON-able fields and rebuilt field by field with type checks; nothing is unpickled.
"""

from __future__ import annotations

import base64
import inspect
from typing import Any

import torch

_FIELDS = ("tensor_cls", "tensor_size", "tensor_stride", "tensor_offset", "storage_cls", "dtype", "storage_device",
           "storage_handle", "storage_size_bytes", "storage_offset_bytes", "requires_grad", "ref_counter_handle",
           "ref_counter_offset", "event_handle", "event_sync_required")
_STORAGE_CLASSES = {"UntypedStorage": torch.UntypedStorage, "TypedStorage": torch.storage.TypedStorage}
_BYTES = ("storage_handle", "ref_counter_handle", "event_handle")
_INTS = ("tensor_offset", "storage_device", "storage_size_bytes", "storage_offset_bytes", "ref_counter_offset")


def export_tensor(t: torch.Tensor) -> dict[str, Any]:
    """JSON-able description of the CUDA tensor ``t`` for another process on this machine."""
    from torch.multiprocessing.reductions import rebuild_cuda_tensor, reduce_tensor

    fn, args = reduce_tensor(t.detach())
    names = tuple(inspect.signature(rebuild_cuda_tensor).parameters)
    if fn is not rebuild_cuda_tensor or names != _FIELDS:
        raise RuntimeError("this torch version describes CUDA-IPC tensors differently; update cuda_ipc._FIELDS")
    d = dict(zip(names, args))
    out: dict[str, Any] = {"tensor_size": [int(v) for v in d["tensor_size"]], "tensor_stride": [int(v) for v in d["tensor_stride"]],
                           "storage_cls": d["storage_cls"].__name__, "dtype": str(d["dtype"]).replace("torch.", ""),
                           "event_sync_required": bool(d["event_sync_required"])}
    if out["storage_cls"] not in _STORAGE_CLASSES:
        raise RuntimeError(f"unexpected storage class {out['storage_cls']}")
    for k in _INTS:
        out[k] = int(d[k])
    for k in _BYTES:
        out[k] = base64.b64encode(bytes(d[k])).decode()
    return out


def import_tensor(desc: dict[str, Any], device_index: int | None = None) -> torch.Tensor:
    """The tensor described by :func:`export_tensor`.  ``device_index`` labels the mapping with the GPU of the
    process that opens it (the handle is opened with that GPU current, so its kernels can address the memory)."""
    from torch.multiprocessing.reductions import rebuild_cuda_tensor

    if not isinstance(desc, dict):
        raise TypeError("a CUDA-IPC description is a mapping")
    dtype = getattr(torch, str(desc["dtype"]), None)
    if not isinstance(dtype, torch.dtype):
        raise ValueError(f"unknown dtype {desc['dtype']!r}")
    storage_cls = _STORAGE_CLASSES.get(str(desc["storage_cls"]))
    if storage_cls is None:
        raise ValueError(f"unknown storage class {desc['storage_cls']!r}")
    size = tuple(int(v) for v in desc["tensor_size"])
    stride = tuple(int(v) for v in desc["tensor_stride"])
    if len(size) != len(stride) or any(v < 0 for v in (*size, *stride)):
        raise ValueError("malformed tensor geometry")
    ints = {k: int(desc[k]) for k in _INTS}
    raw = {k: base64.b64decode(desc[k]) for k in _BYTES}
    # the view must lie inside the exported allocation
    last = ints["tensor_offset"] + sum((n - 1) * s for n, s in zip(size, stride) if n > 0)
    if ints["tensor_offset"] < 0 or (all(size) and (last + 1) * dtype.itemsize > ints["storage_size_bytes"]):
        raise ValueError("the described view does not fit its allocation")
    if device_index is not None:
        ints["storage_device"] = int(device_index)
    return rebuild_cuda_tensor(torch.Tensor, size, stride, ints["tensor_offset"], storage_cls, dtype, ints["storage_device"],
                               raw["storage_handle"], ints["storage_size_bytes"], ints["storage_offset_bytes"], False,
                               raw["ref_counter_handle"], ints["ref_counter_offset"], raw["event_handle"],
                               bool(desc["event_sync_required"]))
