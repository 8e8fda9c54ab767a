"""Sidecar server: one process per GPU that owns a slab of forwarding memory and the ledgers of what was
sent and what is expected.

Behaviour follows the reference's sidecar (python/cornserve/services/sidecar/{server,sender,receiver}.py):
``Send`` stages a tensor into producer-owned slots and tells the leader of every destination group with
``PrepareReceive``; ``Receive`` blocks until the chunk (or the end of the stream) is known; ``MarkDone``
from every member of the consumer group triggers ``Unlink`` at the producer, which frees the slots once
all destination groups are done.  What differs is where the bytes live: the reference copies GPU -> host
shared memory -> GPU; here the slab is *GPU memory* of the producer's device, published to the other
processes of the box as a CUDA-IPC mapping, and consumers read the region in place over NVLink with a
copy kernel that writes straight into their destination buffer (no host staging, no NCCL).  Without CUDA
the slab is a ``/dev/shm`` file and tensors travel inline, which serves CPU-only deployments and tests.
"""

from __future__ import annotations

import asyncio
import os
import json
import signal
from dataclasses import dataclass, field
from typing import Any

import grpc
import torch

from ...logging import SidecarAdapter, get_logger
from ...sidecar import serde
from ...sidecar.constants import (DEVICE_ENV, RANK_ENV, SHM_SIZE_ENV, WORLD_SIZE_ENV, grpc_port, grpc_url,
                                  shm_slab_path, slab_handle_path)
from ..pb import common_pb2, sidecar_pb2, sidecar_pb2_grpc
from .allocator import OutOfSlots, SlotAllocator

OK = common_pb2.STATUS_OK
ERROR = common_pb2.STATUS_ERROR
MEMORY_PRESSURE_THRESHOLD = 500


@dataclass
class _Sent:
    """A staged chunk waiting for its consumers."""

    offset: int
    pending_groups: int


@dataclass
class _Incoming:
    """What this sidecar knows about data id ``id`` on the receiving side."""

    chunks: dict[int, bytes] = field(default_factory=dict)
    num_chunks: int = 0  # 0 = not known yet (stream still open)
    src_rank: dict[int, int] = field(default_factory=dict)
    done_marks: dict[int, set[int]] = field(default_factory=dict)
    changed: asyncio.Condition = field(default_factory=asyncio.Condition)


class SidecarServicer(sidecar_pb2_grpc.SidecarServicer):
    def __init__(self, rank: int, world_size: int, slab_bytes: int, device: torch.device):
        self.rank, self.world_size = rank, world_size
        self.device = device
        self.slab_bytes = slab_bytes
        self.log = get_logger(__name__, [lambda lg: SidecarAdapter(lg, rank)])
        self.online = False
        self.group: list[int] = [rank]
        self.dtype = torch.bfloat16
        self.slot_numel = 1
        self.concurrent_copy = False
        self.slab: torch.Tensor | None = None
        self.allocator: SlotAllocator | None = None
        self._space = asyncio.Condition()
        self.mem_pressure_count = 0
        self.sent: dict[tuple[str, int], _Sent] = {}
        self.incoming: dict[str, _Incoming] = {}
        self._stubs: dict[int, sidecar_pb2_grpc.SidecarStub] = {}
        self._channels: dict[int, grpc.aio.Channel] = {}
        self._copy_stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self._registered_cfg: tuple | None = None
        self._concurrent: dict[tuple[str, int], dict[str, Any]] = {}

    # -- plumbing -----------------------------------------------------------------------------------------
    def stub(self, rank: int) -> sidecar_pb2_grpc.SidecarStub:
        if rank not in self._stubs:
            ch = grpc.aio.insecure_channel(grpc_url(rank), options=[("grpc.max_send_message_length", -1),
                                                                    ("grpc.max_receive_message_length", -1)])
            self._channels[rank] = ch
            self._stubs[rank] = sidecar_pb2_grpc.SidecarStub(ch)
        return self._stubs[rank]

    def _build_slab(self, dtype: torch.dtype) -> None:
        """(Re)create the slab for ``dtype`` and publish how other processes can map it."""
        numel = self.slab_bytes // dtype.itemsize
        if self.device.type == "cuda":
            self.slab = torch.empty(numel, dtype=dtype, device=self.device)
            from ...utils.cuda_ipc import export_tensor

            blob = json.dumps({"kind": "cuda_ipc", "handle": export_tensor(self.slab), "dtype": serde.dtype_name(dtype),
                               "numel": numel}).encode()
        else:
            path = shm_slab_path(self.rank)
            with open(path, "wb") as f:
                f.truncate(self.slab_bytes)
            self.slab = torch.from_file(path, shared=True, size=numel, dtype=dtype)
            blob = json.dumps({"kind": "shm", "path": path, "dtype": serde.dtype_name(dtype), "numel": numel}).encode()
        tmp = slab_handle_path(self.rank) + ".tmp"
        with open(tmp, "wb") as f:
            f.write(blob)
        os.replace(tmp, slab_handle_path(self.rank))
        self.dtype = dtype

    # -- RPCs ------------------------------------------------------------------------------------------------
    async def Register(self, request, context):
        cfg = (tuple(request.group), request.send_slot_numel, request.recv_slot_numel, request.concurrent_copy,
               request.send_dtype, request.recv_dtype)
        if cfg != self._registered_cfg:
            if self.sent:
                self.log.warning("Re-registering with %d staged chunks outstanding; dropping them", len(self.sent))
            dtype = serde.dtype_from_name(request.send_dtype or request.recv_dtype or "bfloat16")
            self.group = sorted(request.group) or [self.rank]
            self.slot_numel = max(1, request.send_slot_numel or request.recv_slot_numel)
            self.concurrent_copy = request.concurrent_copy
            self._build_slab(dtype)
            self.allocator = SlotAllocator(self.slab.numel(), self.slot_numel)
            self.sent.clear()
            self._registered_cfg = cfg
            self.log.info("Registered group=%s slot=%d dtype=%s slab=%d elems", self.group, self.slot_numel, dtype,
                          self.slab.numel())
        self.online = True
        local_rank = self.device.index if self.device.type == "cuda" and self.device.index is not None else self.rank
        return sidecar_pb2.RegisterResponse(status=OK, shm_size=self.slab.numel(), local_rank=local_rank,
                                            num_local_sidecars=self.world_size)

    async def _allocate(self, numel: int) -> int:
        assert self.allocator is not None
        async with self._space:
            while True:
                try:
                    return self.allocator.allocate(numel)
                except OutOfSlots:
                    self.mem_pressure_count += 1
                    if numel > self.allocator.total:
                        raise
                    await self._space.wait()

    async def _release(self, offset: int) -> None:
        async with self._space:
            self.allocator.free(offset)
            self._space.notify_all()

    async def _stage(self, src: torch.Tensor, shard_rank: int, key: tuple[str, int]) -> tuple[int, int] | None:
        """Copy ``src`` into freshly allocated slots.  Returns ``(offset, numel)`` for the shard that owns
        the notification, ``None`` for shards whose call is absorbed."""
        flat = src.reshape(-1)
        n = flat.numel()
        if not self.concurrent_copy:
            if shard_rank != 0:
                return None  # every shard holds the same tensor; shard 0 stages it
            off = await self._allocate(n)
            await self._copy(self.slab[off: off + n], flat)
            return off, n
        # concurrent copy: the first shard to arrive allocates, every shard copies its 1/TP of the data,
        # the last one to finish reports
        st = self._concurrent.setdefault(key, {"off": None, "done": 0, "lock": asyncio.Lock()})
        async with st["lock"]:
            if st["off"] is None:
                st["off"] = await self._allocate(n)
        tp = len(self.group)
        per = -(-n // tp)
        lo, hi = min(shard_rank * per, n), min((shard_rank + 1) * per, n)
        if hi > lo:
            await self._copy(self.slab[st["off"] + lo: st["off"] + hi], flat[lo:hi])
        st["done"] += 1
        if st["done"] == tp:
            self._concurrent.pop(key, None)
            return st["off"], n
        return None

    async def _copy(self, dst: torch.Tensor, src: torch.Tensor) -> None:
        if self._copy_stream is None:
            dst.copy_(src.to(dst.dtype))
            return
        with torch.cuda.stream(self._copy_stream):
            dst.copy_(src.to(device=dst.device, dtype=dst.dtype, non_blocking=True), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        await asyncio.to_thread(ev.synchronize)

    async def Send(self, request, context):
        if not self.online:
            return sidecar_pb2.SendResponse(status=ERROR)
        msg = serde.decode(request.data)
        key = (request.id, request.chunk_id)
        try:
            if msg["kind"] == "obj":
                if request.shard_rank != 0:
                    return sidecar_pb2.SendResponse(status=OK)
                payload, staged = request.data, None
            else:
                src = serde.tensor_from_ipc(msg) if msg["kind"] == "ipc" else serde.tensor_from_inline(msg)
                if src.dtype != self.dtype:
                    self.log.error("dtype mismatch: got %s, slab holds %s", src.dtype, self.dtype)
                    return sidecar_pb2.SendResponse(status=ERROR)
                staged = await self._stage(src, request.shard_rank, key)
                del src
                if staged is None:
                    return sidecar_pb2.SendResponse(status=OK)
                payload = serde.encode_slab_ref(self.rank, staged[0], staged[1], self.dtype, msg["shape"])
            groups = [sorted(g.ranks) for g in request.dst_ranks if g.ranks]
            if staged is not None:
                self.sent[key] = _Sent(staged[0], max(1, len(groups)))
            await asyncio.gather(*(self.stub(g[0]).PrepareReceive(sidecar_pb2.PrepareReceiveRequest(
                id=request.id, data=payload, src_rank=self.rank, chunk_id=request.chunk_id,
                num_chunks=request.num_chunks)) for g in groups))
            return sidecar_pb2.SendResponse(status=OK)
        except Exception:
            self.log.exception("Send failed for %s", key)
            return sidecar_pb2.SendResponse(status=ERROR)

    def _entry(self, data_id: str) -> _Incoming:
        if data_id not in self.incoming:
            self.incoming[data_id] = _Incoming()
        return self.incoming[data_id]

    async def PrepareReceive(self, request, context):
        e = self._entry(request.id)
        async with e.changed:
            e.chunks[request.chunk_id] = request.data
            e.src_rank[request.chunk_id] = request.src_rank
            if request.num_chunks > 0:
                e.num_chunks = request.num_chunks
            e.changed.notify_all()
        return sidecar_pb2.PrepareReceiveResponse(status=OK)

    async def CloseStream(self, request, context):
        """From a local client: forward to nobody, just close; from a producer: record the final count."""
        e = self._entry(request.id)
        async with e.changed:
            e.num_chunks = max(request.num_chunks, 0) or -1  # -1: closed with zero chunks
            e.changed.notify_all()
        return sidecar_pb2.CloseStreamResponse(status=OK)

    async def Receive(self, request, context):
        """Blocks until the chunk is known.  Empty ``data`` means "past the end of the stream"."""
        e = self._entry(request.id)
        async with e.changed:
            while True:
                if request.chunk_id in e.chunks:
                    return sidecar_pb2.ReceiveResponse(status=OK, data=e.chunks[request.chunk_id])
                if e.num_chunks == -1 or (e.num_chunks > 0 and request.chunk_id >= e.num_chunks):
                    return sidecar_pb2.ReceiveResponse(status=OK, data=b"")
                await e.changed.wait()

    async def MarkDone(self, request, context):
        e = self.incoming.get(request.id)
        if e is None or request.chunk_id not in e.chunks:
            return sidecar_pb2.MarkDoneResponse(status=ERROR)
        marks = e.done_marks.setdefault(request.chunk_id, set())
        marks.add(request.shard_rank)
        if len(marks) >= len(self.group):
            payload = serde.decode(e.chunks.pop(request.chunk_id))
            src = e.src_rank.pop(request.chunk_id, self.rank)
            e.done_marks.pop(request.chunk_id, None)
            if payload.get("kind") == "slab":
                try:
                    await self.stub(src).Unlink(sidecar_pb2.UnlinkRequest(id=request.id, chunk_id=request.chunk_id))
                except Exception:
                    self.log.exception("Unlink to sidecar %d failed", src)
            # the entry stays as a tombstone (its chunk count is still needed to answer a late
            # "is there a next chunk?" query); old tombstones are pruned in insertion order
            if len(self.incoming) > 16384:
                for k in [k for k, v in self.incoming.items() if not v.chunks and v.num_chunks != 0][:4096]:
                    self.incoming.pop(k, None)
        return sidecar_pb2.MarkDoneResponse(status=OK)

    async def Unlink(self, request, context):
        key = (request.id, request.chunk_id)
        s = self.sent.get(key)
        if s is None:
            return sidecar_pb2.UnlinkResponse(status=ERROR)
        s.pending_groups -= 1
        if s.pending_groups <= 0:
            self.sent.pop(key)
            await self._release(s.offset)
        return sidecar_pb2.UnlinkResponse(status=OK)

    async def CheckHealth(self, request, context):
        if not self.online:
            st = sidecar_pb2.HealthStatus.HEALTH_OFFLINE
        elif self.mem_pressure_count > MEMORY_PRESSURE_THRESHOLD:
            st = sidecar_pb2.HealthStatus.HEALTH_MEMORY_PRESSURE
        else:
            st = sidecar_pb2.HealthStatus.HEALTH_ALL_GOOD
        return sidecar_pb2.CheckHealthResponse(status=st)

    async def shutdown(self) -> None:
        for ch in self._channels.values():
            await ch.close()
        for p in (slab_handle_path(self.rank), shm_slab_path(self.rank)):
            try:
                os.unlink(p)
            except OSError:
                pass


def pick_device(rank: int) -> torch.device:
    want = os.environ.get(DEVICE_ENV)
    if want:
        return torch.device(want)
    if torch.cuda.is_available():
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


async def serve(rank: int, world_size: int, slab_bytes: int, device: torch.device | None = None,
                ready: asyncio.Event | None = None) -> None:
    device = device or pick_device(rank)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    servicer = SidecarServicer(rank, world_size, slab_bytes, device)
    server = grpc.aio.server(options=[("grpc.max_send_message_length", -1), ("grpc.max_receive_message_length", -1)])
    sidecar_pb2_grpc.add_SidecarServicer_to_server(servicer, server)
    server.add_insecure_port(f"0.0.0.0:{grpc_port(rank)}")
    await server.start()
    # the slab exists (with the default dtype) before any client registers, so health checks can pass
    servicer._build_slab(torch.bfloat16)
    servicer.allocator = SlotAllocator(servicer.slab.numel(), 1)
    servicer.online = True
    servicer.log.info("Sidecar server up on port %d (%s, %d MiB slab)", grpc_port(rank), device, slab_bytes >> 20)
    if ready is not None:
        ready.set()
    stop = asyncio.Event()
    loop = asyncio.get_running_loop()
    for sig in (signal.SIGTERM, signal.SIGINT):
        try:
            loop.add_signal_handler(sig, stop.set)
        except (NotImplementedError, RuntimeError):
            pass
    try:
        await stop.wait()
    finally:
        await server.stop(1.0)
        await servicer.shutdown()


def main() -> None:
    rank = int(os.environ[RANK_ENV])
    world = int(os.environ.get(WORLD_SIZE_ENV, "1"))
    slab = int(os.environ.get(SHM_SIZE_ENV, str(1 << 30)))
    asyncio.run(serve(rank, world, slab))


if __name__ == "__main__":
    main()
