"""Sidecar client: what an executor uses to forward tensors and small objects to other executors.

Public surface as in the reference (python/cornserve/sidecar/api.py:62-520): ``send`` (fire and forget on
a worker pool), ``recv`` / ``recv_sync``, ``mark_done`` / ``mark_done_sync``, ``close_stream``,
``shutdown``; plus the file-backed mock mode (``CORNSERVE_MOCK_SIDECAR=1``) for running an executor
without any sidecar server.

A received tensor is a view of the *producer's* slab: on GPUs that is peer memory mapped through CUDA
IPC, so the consumer can hand it to a copy kernel that reads over NVLink and writes directly into its
own buffer; on CPU it is a view of the producer's shared-memory file.  Call ``mark_done`` when the
data has been consumed so that the producer can reuse the slots.
"""

from __future__ import annotations

import asyncio
import json
import os
import threading
from concurrent.futures import Future, ThreadPoolExecutor
from pathlib import Path
from typing import Any

import grpc
import torch

from ..logging import get_logger
from ..services.pb import common_pb2, sidecar_pb2, sidecar_pb2_grpc
from ..tracing import get_tracer
from . import serde
from .constants import grpc_url, slab_handle_path
from .schema import SidecarConfig

logger = get_logger(__name__)
tracer = get_tracer(__name__)

_GRPC_OPTS = [("grpc.max_send_message_length", -1), ("grpc.max_receive_message_length", -1)]


def _is_mocking() -> bool:
    return os.environ.get("CORNSERVE_MOCK_SIDECAR", "0") == "1"


def _mock_mapping() -> dict[str, Path]:
    """``"{id}-{chunk}" -> file`` from ``CORNSERVE_MOCK_SIDECAR_MAPPING`` (JSON)."""
    raw = os.environ.get("CORNSERVE_MOCK_SIDECAR_MAPPING")
    return {k: Path(v) for k, v in json.loads(raw).items()} if raw else {}


def _mock_dir() -> Path:
    d = Path(os.environ.get("CORNSERVE_MOCK_SIDECAR_DIR", "/tmp/cornserve_mock_sidecar"))
    d.mkdir(parents=True, exist_ok=True)
    return d


class Sidecar:
    def __init__(self, config: SidecarConfig) -> None:
        self.config = config
        self.sidecar_rank = config.sidecar_rank
        self.group = list(config.group)
        self.shard_rank = config.shard_rank
        self.worker_pool = ThreadPoolExecutor(max_workers=config.max_workers, thread_name_prefix="sidecar")
        self._stubs: dict[int, Any] = {}
        self._aio_stubs: dict[int, Any] = {}
        self._channels: list[Any] = []
        self._slabs: dict[int, tuple[int, torch.Tensor]] = {}
        self._lock = threading.Lock()
        self._pending: list[Future] = []
        self.local_rank = config.sidecar_rank
        if _is_mocking():
            return
        resp = self._stub(self.sidecar_rank).Register(sidecar_pb2.RegisterRequest(
            rank=self.sidecar_rank, group=self.group,
            send_slot_numel=config.get_send_slot_numel(), recv_slot_numel=config.get_recv_slot_numel(),
            concurrent_copy=config.concurrent_copy,
            send_dtype=serde.dtype_name(config.get_send_dtype()), recv_dtype=serde.dtype_name(config.get_recv_dtype())))
        if resp.status != common_pb2.STATUS_OK:
            raise RuntimeError(f"Failed to register with sidecar {self.sidecar_rank}")
        self.local_rank = resp.local_rank
        logger.info("Registered with sidecar %d (group %s)", self.sidecar_rank, self.group)

    # -- connections --------------------------------------------------------------------------------------
    def _stub(self, rank: int):
        with self._lock:
            if rank not in self._stubs:
                ch = grpc.insecure_channel(grpc_url(rank), options=_GRPC_OPTS)
                self._channels.append(ch)
                self._stubs[rank] = sidecar_pb2_grpc.SidecarStub(ch)
            return self._stubs[rank]

    def _aio_stub(self, rank: int):
        if rank not in self._aio_stubs:
            ch = grpc.aio.insecure_channel(grpc_url(rank), options=_GRPC_OPTS)
            self._channels.append(ch)
            self._aio_stubs[rank] = sidecar_pb2_grpc.SidecarStub(ch)
        return self._aio_stubs[rank]

    def _slab_of(self, rank: int) -> torch.Tensor:
        """Sidecar ``rank``'s slab (bytes), mapped once per allocation: the handle file changes only when that sidecar
        was restarted, and then the mapping is renewed."""
        path = slab_handle_path(rank)
        stamp = os.stat(path).st_mtime_ns
        with self._lock:
            cached = self._slabs.get(rank)
            if cached is not None and cached[0] == stamp:
                return cached[1]
            info = json.loads(Path(path).read_bytes())
            if info["kind"] == "cuda_ipc":
                from ..utils.cuda_ipc import import_tensor

                # Open the handle with THIS process's GPU current (the open enables peer access to the slab's GPU as
                # needed): kernels of this GPU can then read the slab in place, over NVLink when it lives elsewhere.
                slab = import_tensor(info["handle"], torch.cuda.current_device())
            else:
                slab = torch.from_file(info["path"], shared=True, size=info["nbytes"], dtype=torch.uint8)
            self._slabs[rank] = (stamp, slab)
            return slab

    # -- send -------------------------------------------------------------------------------------------------
    def send(self, data: Any, id: str, dst_sidecar_ranks: list[list[int]], chunk_id: int = 0, num_chunks: int = 1,
             stream: bool = False) -> Future | None:
        """Forward ``data`` (tensor or small object) under ``id`` to every destination group.

        Returns immediately; the transfer runs on the worker pool.  With ``stream=True`` the number of
        chunks is open-ended: call :meth:`close_stream` after the last chunk.  Tensors must be contiguous;
        every rank of a tensor-parallel group calls ``send`` with its (identical) tensor.
        """
        if any(r < 0 for g in dst_sidecar_ranks for r in g):
            raise ValueError("Invalid sidecar rank")
        if stream:
            num_chunks = 0
        if _is_mocking():
            path = str(_mock_dir() / f"{id}-{chunk_id}")
            if isinstance(data, torch.Tensor):
                torch.save(data.detach().cpu(), path + ".pt")
            else:
                Path(path + ".json").write_text(json.dumps(data))
            return None
        if isinstance(data, torch.Tensor):
            if not data.is_contiguous():
                raise ValueError("Tensor must be contiguous")
        fut = self.worker_pool.submit(self._send_worker, data, id, dst_sidecar_ranks, chunk_id, num_chunks)
        fut.add_done_callback(self._log_failure)
        self._pending = [f for f in self._pending if not f.done()] + [fut]
        return fut

    @staticmethod
    def _log_failure(f: Future) -> None:
        if f.exception() is not None:
            logger.error("sidecar send failed: %s", f.exception())

    def _send_worker(self, data: Any, id: str, dst: list[list[int]], chunk_id: int, num_chunks: int) -> None:
        with tracer.start_as_current_span("Sidecar._send_worker"):
            if isinstance(data, torch.Tensor):
                if data.is_cuda:
                    torch.cuda.current_stream(data.device).synchronize()  # the data must be complete before it is shared
                    payload = serde.encode_ipc_tensor(data)
                else:
                    payload = serde.encode_inline_tensor(data)
            else:
                payload = serde.encode_obj(data)
            req = sidecar_pb2.SendRequest(id=id, dst_ranks=[sidecar_pb2.RankGroup(ranks=g) for g in dst],
                                          shard_rank=self.shard_rank, data=payload, chunk_id=chunk_id,
                                          num_chunks=num_chunks)
            resp = self._stub(self.config.leader).Send(req)  # the group leader's sidecar stages the data
            if resp.status != common_pb2.STATUS_OK:
                raise RuntimeError(f"Sidecar send of {id} chunk {chunk_id} failed")

    def flush(self, timeout: float | None = None) -> None:
        """Wait for the sends issued so far."""
        for f in list(self._pending):
            f.result(timeout=timeout)
        self._pending.clear()

    def close_stream(self, id: str, num_chunks: int, dst_sidecar_ranks: list[list[int]]) -> None:
        """Tell every destination group how many chunks the stream ``id`` had."""
        if _is_mocking():
            return
        earlier = [f for f in self._pending if not f.done()]
        for leader in (min(g) for g in dst_sidecar_ranks):
            if leader < 0:
                raise ValueError("Invalid sidecar rank")
            fut = self.worker_pool.submit(self._close_stream_worker, id, num_chunks, leader, earlier)
            fut.add_done_callback(self._log_failure)
            self._pending.append(fut)

    def _close_stream_worker(self, id: str, num_chunks: int, rank: int, earlier: list[Future]) -> None:
        # chunks are staged asynchronously: closing must not overtake the sends issued before it
        for f in earlier:
            try:
                f.result(timeout=600)
            except Exception:
                pass
        resp = self._stub(rank).CloseStream(sidecar_pb2.CloseStreamRequest(id=id, num_chunks=num_chunks))
        if resp.status != common_pb2.STATUS_OK:
            raise RuntimeError(f"Failed to close stream {id}")

    # -- receive ---------------------------------------------------------------------------------------------------
    def _decode_received(self, data: bytes) -> Any:
        if not data:
            return None
        msg = serde.decode(data)
        if msg["kind"] == "obj":
            return msg["obj"]
        if msg["kind"] == "slab":
            # the producer pushed the tensor into the slab of this group's leader: a view of those bytes
            slab = self._slab_of(msg["rank"])
            shape = msg["shape"] if -1 not in msg["shape"] else list(self.config.get_recv_tensor_shape())
            return slab[msg["offset"]: msg["offset"] + msg["nbytes"]].view(serde.dtype_from_name(msg["dtype"])).view(shape)
        if msg["kind"] == "inline":
            return serde.tensor_from_inline(msg)
        raise ValueError(f"unknown payload kind {msg['kind']}")

    def _mock_recv(self, id: str, chunk_id: int) -> Any:
        key = f"{id}-{chunk_id}"
        mapping = _mock_mapping()
        base = mapping.get(key, _mock_dir() / key)
        for p in (base, Path(str(base) + ".pt"), Path(str(base) + ".json")):
            if p.exists():
                return json.loads(p.read_text()) if p.suffix == ".json" else torch.load(p)
        return None

    async def recv(self, id: str, chunk_id: int = 0) -> Any:
        """Wait for chunk ``chunk_id`` of ``id``.  Returns ``None`` past the end of a closed stream."""
        if _is_mocking():
            return self._mock_recv(id, chunk_id)
        with tracer.start_as_current_span("Sidecar.recv"):
            resp = await self._aio_stub(self.config.leader).Receive(sidecar_pb2.ReceiveRequest(id=id, chunk_id=chunk_id))
            if resp.status != common_pb2.STATUS_OK:
                raise RuntimeError(f"Failed to receive {id} chunk {chunk_id}")
            return self._decode_received(resp.data)

    def recv_sync(self, id: str, chunk_id: int = 0) -> Any:
        if _is_mocking():
            return self._mock_recv(id, chunk_id)
        resp = self._stub(self.config.leader).Receive(sidecar_pb2.ReceiveRequest(id=id, chunk_id=chunk_id))
        if resp.status != common_pb2.STATUS_OK:
            raise RuntimeError(f"Failed to receive {id} chunk {chunk_id}")
        return self._decode_received(resp.data)

    async def mark_done(self, id: str, chunk_id: int = 0) -> None:
        """The data was consumed: once every member of this group said so the producer frees the slots."""
        if _is_mocking():
            return
        for shard in self._marks():
            resp = await self._aio_stub(self.config.leader).MarkDone(
                sidecar_pb2.MarkDoneRequest(id=id, chunk_id=chunk_id, shard_rank=shard))
            if resp.status != common_pb2.STATUS_OK:
                logger.error("Failed to mark %s chunk %d done", id, chunk_id)
                return

    def mark_done_sync(self, id: str, chunk_id: int = 0) -> None:
        if _is_mocking():
            return
        for shard in self._marks():
            resp = self._stub(self.config.leader).MarkDone(
                sidecar_pb2.MarkDoneRequest(id=id, chunk_id=chunk_id, shard_rank=shard))
            if resp.status != common_pb2.STATUS_OK:
                logger.error("Failed to mark %s chunk %d done", id, chunk_id)
                return

    def _marks(self) -> list[int]:
        """Shard ranks this client reports for: its own, or every member's when it stands for the whole group (the
        producer's slots are freed once every member of the consuming group has said it is done)."""
        return list(range(len(self.group))) if self.config.whole_group else [self.shard_rank]

    # -- lifecycle ---------------------------------------------------------------------------------------------------
    def check_health(self, rank: int | None = None) -> int:
        return self._stub(self.sidecar_rank if rank is None else rank).CheckHealth(sidecar_pb2.CheckHealthRequest()).status

    def shutdown_sync(self) -> None:
        try:
            self.flush(timeout=30)
        except Exception:
            pass
        self.worker_pool.shutdown(wait=False)
        self._slabs.clear()
        for ch in self._channels:
            try:
                res = ch.close()
                if asyncio.iscoroutine(res):
                    res.close()
            except Exception:
                pass
        self._channels.clear()

    async def shutdown(self) -> None:
        await asyncio.to_thread(self.shutdown_sync)

    def __del__(self) -> None:  # pragma: no cover
        try:
            self.worker_pool.shutdown(wait=False)
        except Exception:
            pass
