"""Sidecar server: one process per GPU that owns a slab of forwarding memory and the ledgers of what was
sent and what is expected.

Behaviour follows the reference's sidecar (python/cornserve/services/sidecar/{server,sender,receiver}.py):
``Send`` stages a tensor into producer-owned slots and tells the leader of every destination group with
``PrepareReceive``; ``Receive`` blocks until the chunk (or the end of the stream) is known; ``MarkDone``
from every member of the consumer group triggers ``Unlink`` at the producer, which frees the slots once
all destination groups are done.  What differs is where the bytes live and who moves them: the reference copies
GPU -> host shared memory -> GPU; here every sidecar owns a slab of *GPU memory* on its device, allocated once when the
server starts and published to the other processes of the box as a CUDA-IPC mapping, and a producer **pushes**: its
sidecar writes the tensor straight into the slab of the consuming executor's GPU with a copy kernel that stores over
NVLink, then tells the consumer's sidecar where the rows are.  The consumer reads its own GPU's memory.  No host
staging, no NCCL, one pass over the data.

A push needs space at the destination without asking for it first: each slab is cut into ``world_size`` equal
regions and region ``p`` of every slab is managed by sidecar ``p`` (the only one that writes there), so a producer
allocates in its own ledger, writes, and frees when the consumer's ``MarkDone`` comes back as ``Unlink``.  Without CUDA
the slabs are ``/dev/shm`` files and the same protocol runs on the CPU, which serves CPU-only deployments and tests.
"""

from __future__ import annotations

import asyncio
import json
import os
import signal
import time
import uuid
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
from ...tracing import grpc_server_interceptors

OK = common_pb2.STATUS_OK
ERROR = common_pb2.STATUS_ERROR
MEMORY_PRESSURE_THRESHOLD = 500


@dataclass
class _Sent:
    """A pushed chunk waiting for its consumers: where it was placed (destination sidecar -> offset in this
    sidecar's region of that slab) and how many destination groups still hold it."""

    placed: dict[int, int]
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
        self.slab: torch.Tensor | None = None          # uint8, allocated once in serve(), never replaced
        self.generation = uuid.uuid4().hex             # names this allocation: a restarted sidecar has a new one
        self.region_bytes = (slab_bytes // max(world_size, 1)) // 256 * 256
        self.remote: dict[int, SlotAllocator] = {}     # destination sidecar -> allocator of this sidecar's region there
        self._peer_slabs: dict[int, tuple[str, torch.Tensor]] = {}
        self.send_dtype: torch.dtype | None = None
        self.push_stats = {"pushes": 0, "bytes": 0, "copy_ms": 0.0, "send_ms": 0.0}
        self._probe_repeat = os.environ.get("SIDECAR_PUSH_PROBE") == "1"
        self._space = asyncio.Condition()
        self.mem_pressure_count = 0
        self.sent: dict[tuple[str, int], _Sent] = {}
        self.incoming: dict[str, _Incoming] = {}
        self._stubs: dict[int, sidecar_pb2_grpc.SidecarStub] = {}
        self._channels: dict[int, grpc.aio.Channel] = {}
        self._copy_stream = torch.cuda.Stream(device=device) if device.type == "cuda" else None
        self._registered_cfg: tuple | None = None
        self._concurrent: dict[tuple[str, int], dict[str, Any]] = {}
        self._placed: dict[tuple[str, int], dict[int, int]] = {}

    # -- plumbing -----------------------------------------------------------------------------------------
    def stub(self, rank: int) -> sidecar_pb2_grpc.SidecarStub:
        if rank not in self._stubs:
            ch = grpc.aio.insecure_channel(grpc_url(rank), options=[("grpc.max_send_message_length", -1),
                                                                    ("grpc.max_receive_message_length", -1)])
            self._channels[rank] = ch
            self._stubs[rank] = sidecar_pb2_grpc.SidecarStub(ch)
        return self._stubs[rank]

    def build_slab(self) -> None:
        """Allocate the slab (once) and publish how other processes can map it."""
        if self.device.type == "cuda":
            self.slab = torch.empty(self.slab_bytes, dtype=torch.uint8, device=self.device)
            from ...utils.cuda_ipc import export_tensor

            info = {"kind": "cuda_ipc", "handle": export_tensor(self.slab)}
        else:
            path = shm_slab_path(self.rank)
            with open(path, "wb") as f:
                f.truncate(self.slab_bytes)
            self.slab = torch.from_file(path, shared=True, size=self.slab_bytes, dtype=torch.uint8)
            info = {"kind": "shm", "path": path}
        info.update(nbytes=self.slab_bytes, generation=self.generation, region_bytes=self.region_bytes,
                    world_size=self.world_size)
        tmp = slab_handle_path(self.rank) + ".tmp"
        with open(tmp, "w") as f:
            json.dump(info, f)
        os.replace(tmp, slab_handle_path(self.rank))

    def peer_slab(self, rank: int) -> torch.Tensor:
        """Sidecar ``rank``'s slab as a tensor of this process (own slab: the tensor itself).  Mapped once per
        allocation: when the peer restarted (new generation in its handle file) it is mapped again."""
        if rank == self.rank:
            return self.slab
        info = json.loads(open(slab_handle_path(rank)).read())
        cached = self._peer_slabs.get(rank)
        if cached is not None and cached[0] == info["generation"]:
            return cached[1]
        if info["kind"] == "cuda_ipc":
            from ...utils.cuda_ipc import import_tensor

            # opened with this sidecar's GPU current, so its copy kernel can store there over NVLink
            slab = import_tensor(info["handle"], self.device.index if self.device.type == "cuda" else None)
        else:
            slab = torch.from_file(info["path"], shared=True, size=info["nbytes"], dtype=torch.uint8)
        self._peer_slabs[rank] = (info["generation"], slab)
        self.remote.pop(rank, None)   # a new allocation starts empty
        return slab

    # -- RPCs ------------------------------------------------------------------------------------------------
    async def Register(self, request, context):
        """Records the client's group and dtypes.  The slab is not touched: it was allocated when the server started,
        and every process that mapped it keeps a valid mapping whatever registers later."""
        cfg = (tuple(request.group), request.send_slot_numel, request.recv_slot_numel, request.concurrent_copy,
               request.send_dtype, request.recv_dtype)
        if cfg != self._registered_cfg:
            self.group = sorted(request.group) or [self.rank]
            self.slot_numel = max(1, request.send_slot_numel or request.recv_slot_numel)
            self.concurrent_copy = request.concurrent_copy
            self.send_dtype = serde.dtype_from_name(request.send_dtype) if request.send_dtype else None
            self.dtype = serde.dtype_from_name(request.send_dtype or request.recv_dtype or "bfloat16")
            self._registered_cfg = cfg
            self.log.info("Registered group=%s slot=%d dtype=%s", self.group, self.slot_numel, self.dtype)
        self.online = True
        local_rank = self.device.index if self.device.type == "cuda" and self.device.index is not None else self.rank
        return sidecar_pb2.RegisterResponse(status=OK, shm_size=self.slab_bytes // self.dtype.itemsize, local_rank=local_rank,
                                            num_local_sidecars=self.world_size)

    def _allocator(self, dst: int) -> SlotAllocator:
        if dst not in self.remote:
            self.remote[dst] = SlotAllocator(self.region_bytes, 1, align=256)
        return self.remote[dst]

    async def _allocate(self, dst: int, nbytes: int) -> int:
        """Byte offset (inside this sidecar's region of ``dst``'s slab) of ``nbytes`` free bytes; waits for space."""
        alloc = self._allocator(dst)
        if nbytes > alloc.total:
            raise OutOfSlots(f"{nbytes} bytes do not fit a region of {alloc.total} bytes (raise {SHM_SIZE_ENV})")
        deadline = time.monotonic() + float(os.environ.get("SIDECAR_ALLOC_TIMEOUT_S", "120"))
        async with self._space:
            while True:
                try:
                    return alloc.allocate(nbytes)
                except OutOfSlots:
                    self.mem_pressure_count += 1
                    left = deadline - time.monotonic()
                    if left <= 0:
                        # the consumer does not give space back (it died, or never marks its data done): fail this
                        # send rather than hold the producer for ever
                        raise OutOfSlots(f"no {nbytes} free bytes in the region of sidecar {dst} after waiting") from None
                    try:
                        await asyncio.wait_for(self._space.wait(), timeout=left)
                    except asyncio.TimeoutError:
                        pass

    async def _release(self, placed: dict[int, int]) -> None:
        async with self._space:
            for dst, off in placed.items():
                alloc = self.remote.get(dst)
                if alloc is not None:
                    try:
                        alloc.free(off)
                    except KeyError:
                        pass   # the peer restarted in between: its region started over
            self._space.notify_all()

    def _region(self, dst: int, off: int, nbytes: int) -> tuple[torch.Tensor, int]:
        """The destination bytes and their absolute offset in ``dst``'s slab."""
        base = self.rank * self.region_bytes + off
        return self.peer_slab(dst)[base: base + nbytes], base

    async def _push(self, src: torch.Tensor, shard_rank: int, key: tuple[str, int], leaders: list[int]) -> dict[int, int] | None:
        """Write ``src`` into this sidecar's region of every destination leader's slab.  Returns where it was placed
        (destination -> absolute byte offset) for the shard that owns the notification, ``None`` for shards whose
        call is absorbed."""
        flat = src.reshape(-1)
        nbytes = flat.numel() * flat.element_size()
        if not self.concurrent_copy:
            if shard_rank != 0:
                return None   # every shard holds the same tensor; shard 0 pushes it
            placed, absolute = {}, {}
            for dst in leaders:
                self.peer_slab(dst)   # map (or re-map after the peer restarted) before allocating in its region
                off = await self._allocate(dst, nbytes)
                placed[dst] = off
                view, absolute[dst] = self._region(dst, off, nbytes)
                await self._copy(view, flat)
            self._placed[key] = placed
            return absolute
        # concurrent copy: the first shard to arrive allocates, every shard copies its 1/TP of the bytes, the last one
        # to finish reports
        st = self._concurrent.setdefault(key, {"placed": None, "done": 0, "lock": asyncio.Lock()})
        async with st["lock"]:
            if st["placed"] is None:
                for dst in leaders:
                    self.peer_slab(dst)
                st["placed"] = {dst: await self._allocate(dst, nbytes) for dst in leaders}
        tp = len(self.group)
        n = flat.numel()
        per = -(-n // tp)
        lo, hi = min(shard_rank * per, n), min((shard_rank + 1) * per, n)
        absolute = {}
        for dst, off in st["placed"].items():
            view, absolute[dst] = self._region(dst, off, nbytes)
            if hi > lo:
                es = flat.element_size()
                await self._copy(view[lo * es: hi * es], flat[lo:hi])
        st["done"] += 1
        if st["done"] == tp:
            self._concurrent.pop(key, None)
            self._placed[key] = st["placed"]
            return absolute
        return None

    async def _copy(self, dst_bytes: torch.Tensor, src: torch.Tensor) -> None:
        """``src`` -> ``dst_bytes`` (uint8 view of a slab, possibly on another GPU)."""
        if self._copy_stream is None or not src.is_cuda:
            dst_bytes.copy_(src.contiguous().view(torch.uint8).reshape(-1).to(dst_bytes.device))
            return
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(self._copy_stream):
            t0.record()
            if src.device == self.device:
                from ... import ops

                ops.push_bytes_(dst_bytes, src.contiguous())   # this library's copy kernel: plain stores over NVLink
            else:
                # a shard that lives on another GPU of the group (concurrent copy): the driver's peer copy
                dst_bytes.copy_(src.contiguous().view(torch.uint8).reshape(-1), non_blocking=True)
            t1.record()
            t2 = None
            if self._probe_repeat and src.device == self.device:
                # diagnosis only (SIDECAR_PUSH_PROBE=1): the same copy once more, straight behind the first, tells the
                # kernel's own time apart from what its launch out of an otherwise idle process costs on a shared GPU
                t2 = torch.cuda.Event(enable_timing=True)
                ops.push_bytes_(dst_bytes, src.contiguous())
                t2.record()
        await asyncio.to_thread((t2 or t1).synchronize)
        if t2 is not None:
            self.push_stats["repeat_ms"] = self.push_stats.get("repeat_ms", 0.0) + t1.elapsed_time(t2)
        self.push_stats["copy_ms"] += t0.elapsed_time(t1)
        self.push_stats["bytes"] += dst_bytes.numel()
        self.push_stats["pushes"] += 1
        if self.push_stats["pushes"] % 16 == 0:
            self.write_stats()

    def write_stats(self) -> None:
        """Counters of the push path (device time of the copy kernels, time inside ``Send``) beside the handle file."""
        try:
            with open(slab_handle_path(self.rank) + ".stats", "w") as f:
                json.dump(self.push_stats, f)
        except OSError:
            pass

    async def Send(self, request, context):
        if not self.online:
            return sidecar_pb2.SendResponse(status=ERROR)
        t_begin = time.perf_counter()
        msg = serde.decode(request.data)
        key = (request.id, request.chunk_id)
        groups = [sorted(g.ranks) for g in request.dst_ranks if g.ranks]
        try:
            if msg["kind"] == "obj":
                if request.shard_rank != 0:
                    return sidecar_pb2.SendResponse(status=OK)
                payloads = {g[0]: request.data for g in groups}
            else:
                src = serde.tensor_from_ipc(msg) if msg["kind"] == "ipc" else serde.tensor_from_inline(msg)
                if self.send_dtype is not None and src.dtype != self.send_dtype:
                    self.log.error("dtype mismatch: got %s, registered to send %s", src.dtype, self.send_dtype)
                    return sidecar_pb2.SendResponse(status=ERROR)
                placed = await self._push(src, request.shard_rank, key, [g[0] for g in groups])
                nbytes, dtype = src.numel() * src.element_size(), src.dtype
                del src
                if placed is None:
                    return sidecar_pb2.SendResponse(status=OK)
                self.sent[key] = _Sent(self._placed.pop(key), max(1, len(groups)))
                payloads = {dst: serde.encode_slab_ref(dst, off, nbytes, dtype, msg["shape"]) for dst, off in placed.items()}
            await asyncio.gather(*(self.stub(g[0]).PrepareReceive(sidecar_pb2.PrepareReceiveRequest(
                id=request.id, data=payloads[g[0]], src_rank=self.rank, chunk_id=request.chunk_id,
                num_chunks=request.num_chunks)) for g in groups))
            self.push_stats["send_ms"] += (time.perf_counter() - t_begin) * 1e3
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
            await self._release(s.placed)
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
        if self.push_stats["pushes"]:
            ps = self.push_stats
            self.log.info("pushed %d tensors, %.1f MB, %.2f ms in copy kernels (%.0f GB/s), %.1f ms in Send", ps["pushes"],
                          ps["bytes"] / 1e6, ps["copy_ms"], ps["bytes"] / 1e6 / max(ps["copy_ms"], 1e-9), ps["send_ms"])
        for p in (slab_handle_path(self.rank), slab_handle_path(self.rank) + ".stats", shm_slab_path(self.rank)):
            try:
                os.unlink(p)
            except OSError:
                pass


def pick_device(rank: int) -> torch.device:
    want = os.environ.get(DEVICE_ENV)
    if want:
        dev = torch.device(want)
        if dev.type == "cuda" and dev.index is None:   # "cuda" alone means this sidecar's own GPU
            dev = torch.device("cuda", rank % max(torch.cuda.device_count(), 1))
        return dev
    if torch.cuda.is_available():
        return torch.device("cuda", rank % torch.cuda.device_count())
    return torch.device("cpu")


async def serve(rank: int, world_size: int, slab_bytes: int, device: torch.device | None = None,
                ready: asyncio.Event | None = None) -> None:
    device = device or pick_device(rank)
    if device.type == "cuda":
        torch.cuda.set_device(device)
    servicer = SidecarServicer(rank, world_size, slab_bytes, device)
    server = grpc.aio.server(interceptors=grpc_server_interceptors(), options=[("grpc.max_send_message_length", -1), ("grpc.max_receive_message_length", -1)])
    sidecar_pb2_grpc.add_SidecarServicer_to_server(servicer, server)
    server.add_insecure_port(f"0.0.0.0:{grpc_port(rank)}")
    await server.start()
    # the slab is allocated here, once, before any client registers; nothing ever replaces it
    servicer.build_slab()
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
