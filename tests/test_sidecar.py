"""Sidecar: real server processes on localhost (CPU slabs), clients in this process.  Covers objects,
tensors with 1-4 chunks, tensor-parallel groups on both sides (single and concurrent copy), broadcast to
two consumer groups, out-of-order streaming with ``close_stream``, dtype mismatch, slot reuse after
``mark_done`` and the file-backed mock mode."""

import asyncio
import os
import signal
import socket
import uuid

import pytest
import torch

from cornserve.services.sidecar.allocator import OutOfSlots, SlotAllocator


def _free_port_base(n):
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    base = s.getsockname()[1]
    s.close()
    return base if base + n < 65000 else 20000


@pytest.fixture(scope="module")
def cluster():
    ns = uuid.uuid4().hex[:8]
    base = _free_port_base(8)
    os.environ["CORNSERVE_SIDECAR_BASE_PORT"] = str(base)
    os.environ["SIDECAR_NAMESPACE"] = ns
    import importlib

    import cornserve.constants as c
    import cornserve.sidecar.constants as sc

    importlib.reload(c)
    importlib.reload(sc)
    import cornserve.services.sidecar.launch as launch
    import cornserve.sidecar.api as api

    importlib.reload(launch)
    importlib.reload(api)
    env = {"CORNSERVE_SIDECAR_BASE_PORT": str(base), "SIDECAR_NAMESPACE": ns, "CORNSERVE_LOG_LEVEL": "WARNING"}
    procs = [launch.spawn_sidecar(r, 4, slab_bytes=8 << 20, device="cpu", env=env) for r in range(4)]
    assert launch.wait_all_good(list(range(4)), 60), "sidecar servers did not come up"
    yield api
    for p in procs:
        try:
            os.killpg(p.pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
    for p in procs:
        p.wait(timeout=10)


def _client(api, rank, group=None, shape=(-1, 64), dtype=torch.bfloat16, concurrent=False):
    from cornserve.sidecar.schema import SidecarConfig

    return api.Sidecar(SidecarConfig(sidecar_rank=rank, group=group, send_tensor_dtype=dtype, send_tensor_shape=shape,
                                     recv_tensor_dtype=dtype, recv_tensor_shape=shape, concurrent_copy=concurrent))


def test_allocator():
    a = SlotAllocator(1024, 64, align=128)
    x, y = a.allocate(64), a.allocate(200)
    assert x == 0 and y == 128 and a.used_runs() == 2
    a.free(x)
    assert a.allocate(100) == 0
    with pytest.raises(OutOfSlots):
        a.allocate(4096)
    a.free(y)
    a.free(0)
    assert a.free_numel() == 1024


def test_objects_and_tensors(cluster):
    api = cluster
    prod, cons = _client(api, 0), _client(api, 1)
    try:
        prod.send({"k": [1, 2], "s": "v"}, "obj1", [[1]])
        assert cons.recv_sync("obj1") == {"k": [1, 2], "s": "v"}
        for n_chunks in (1, 4):
            did = uuid.uuid4().hex
            chunks = [torch.randn(5 + i, 64).bfloat16() for i in range(n_chunks)]
            for i, c in enumerate(chunks):
                prod.send(c, did, [[1]], chunk_id=i, num_chunks=n_chunks)
            for i, c in enumerate(chunks):
                got = cons.recv_sync(did, i)
                assert got.shape == c.shape and torch.equal(got, c)
                cons.mark_done_sync(did, i)
            assert cons.recv_sync(did, n_chunks) is None
        # slots are reused after mark_done: far more data than the slab holds in total
        for i in range(40):
            did = uuid.uuid4().hex
            t = torch.full((2000, 64), float(i)).bfloat16()
            prod.send(t, did, [[1]])
            assert torch.equal(cons.recv_sync(did), t)
            cons.mark_done_sync(did)
    finally:
        prod.shutdown_sync()
        cons.shutdown_sync()


@pytest.mark.parametrize("concurrent", [False, True])
def test_tp_groups_and_broadcast(cluster, concurrent):
    api = cluster
    p0, p1 = _client(api, 0, [0, 1], concurrent=concurrent), _client(api, 1, [0, 1], concurrent=concurrent)
    c2, c3 = _client(api, 2), _client(api, 3)
    try:
        did = uuid.uuid4().hex
        t = torch.randn(33, 64).bfloat16()
        for p in (p0, p1):  # every TP rank sends its (identical) tensor
            p.send(t.clone(), did, [[2], [3]])
        for c in (c2, c3):
            assert torch.equal(c.recv_sync(did), t)
            c.mark_done_sync(did)
        # a TP consumer group: data lands at the leader, both members read it, both must mark done
        g2, g3 = _client(api, 2, [2, 3]), _client(api, 3, [2, 3])
        did = uuid.uuid4().hex
        for p in (p0, p1):
            p.send(t.clone(), did, [[2, 3]])
        for c in (g2, g3):
            assert torch.equal(c.recv_sync(did), t)
        g2.mark_done_sync(did)
        g3.mark_done_sync(did)
        g2.shutdown_sync()
        g3.shutdown_sync()
    finally:
        for c in (p0, p1, c2, c3):
            c.shutdown_sync()


def test_group_leader_that_alone_has_a_client_frees_the_producers_space(cluster):
    """A tensor-parallel executor whose leader is its only sidecar client (``whole_group``): its ``mark_done`` counts for
    every rank of the group, so the producer's region of the leader's slab is freed and never fills up.  The region is
    2 MiB (an 8 MiB slab shared by four sidecars); 40 tensors of 256 KiB only fit if space comes back."""
    import concurrent.futures
    import dataclasses

    api = cluster
    from cornserve.sidecar.schema import SidecarConfig

    prod = _client(api, 0)
    cfg = SidecarConfig(sidecar_rank=2, group=[2, 3], recv_tensor_dtype=torch.bfloat16, recv_tensor_shape=(-1, 64), whole_group=True)
    leader = api.Sidecar(cfg)
    try:
        t = torch.randn(2048, 64).bfloat16()   # 256 KiB

        def roundtrip(i: int) -> bool:
            did = uuid.uuid4().hex
            prod.send(t, did, [[2, 3]])
            ok = torch.equal(leader.recv_sync(did), t)
            leader.mark_done_sync(did)
            return ok

        pool = concurrent.futures.ThreadPoolExecutor(max_workers=1)
        try:
            for i in range(40):
                assert pool.submit(roundtrip, i).result(timeout=20), f"tensor {i} did not come back intact"
        finally:
            pool.shutdown(wait=False, cancel_futures=True)
        assert dataclasses.replace(cfg, whole_group=False).whole_group is False
    finally:
        prod.shutdown_sync()
        leader.shutdown_sync()


def test_rows_are_pushed_into_the_consumers_slab_and_survive_new_registrations(cluster):
    """The producer's sidecar writes into the slab of the consumer's sidecar (a view of rank 1's slab comes back, not of
    rank 0's), and the slab is never re-allocated: a client that registers later with another dtype and slot size does
    not invalidate what a consumer has mapped or what is still in flight."""
    api = cluster
    from cornserve.sidecar import serde
    from cornserve.services.pb import sidecar_pb2

    prod, cons = _client(api, 0), _client(api, 1)
    try:
        first, second = uuid.uuid4().hex, uuid.uuid4().hex
        a = torch.randn(40, 64).bfloat16()
        prod.send(a, first, [[1]])
        prod.flush()
        raw = cons._stub(1).Receive(sidecar_pb2.ReceiveRequest(id=first, chunk_id=0)).data
        ref = serde.decode(raw)
        assert ref["kind"] == "slab" and ref["rank"] == 1 and ref["nbytes"] == a.numel() * 2
        got_a = cons.recv_sync(first)
        mapped_before = cons._slab_of(1)
        # another executor shows up on the producer's GPU with a different dtype and slot size
        other = _client(api, 0, shape=(-1, 7), dtype=torch.float32)
        b = torch.randn(9, 7)
        other.send(b, second, [[1]])
        other.flush()
        late = _client(api, 1, shape=(-1, 7), dtype=torch.float32)
        assert torch.equal(late.recv_sync(second), b)
        assert torch.equal(got_a, a)                                 # still the same bytes through the old mapping
        assert cons._slab_of(1) is mapped_before                     # and the mapping was not renewed
        cons.mark_done_sync(first)
        late.mark_done_sync(second)
        other.shutdown_sync()
        late.shutdown_sync()
    finally:
        prod.shutdown_sync()
        cons.shutdown_sync()


def test_streaming_out_of_order_and_close(cluster):
    api = cluster
    prod, cons = _client(api, 0), _client(api, 2)

    async def run():
        did = uuid.uuid4().hex
        chunks = [torch.randn(3, 64).bfloat16() for _ in range(3)]
        waiter = asyncio.create_task(cons.recv(did, 2))  # asks for the last chunk first
        await asyncio.sleep(0.05)
        for i in (1, 0, 2):
            prod.send(chunks[i], did, [[2]], chunk_id=i, stream=True)
        assert torch.equal(await waiter, chunks[2])
        assert torch.equal(await cons.recv(did, 0), chunks[0])
        end = asyncio.create_task(cons.recv(did, 3))
        await asyncio.sleep(0.05)
        assert not end.done()  # the stream is still open
        prod.close_stream(did, 3, [[2]])
        assert await end is None
        for i in range(3):
            await cons.mark_done(did, i)
        # closing before any chunk was sent
        did = uuid.uuid4().hex
        prod.close_stream(did, 0, [[2]])
        assert await cons.recv(did, 0) is None

    try:
        asyncio.run(run())
    finally:
        prod.shutdown_sync()
        cons.shutdown_sync()


def test_dtype_mismatch_is_an_error(cluster):
    api = cluster
    prod = _client(api, 3, dtype=torch.float64)
    try:
        fut = prod.send(torch.randn(4, 64).bfloat16(), uuid.uuid4().hex, [[1]])
        with pytest.raises(RuntimeError):
            fut.result(timeout=10)
    finally:
        prod.shutdown_sync()


def test_mock_sidecar(tmp_path, monkeypatch):
    monkeypatch.setenv("CORNSERVE_MOCK_SIDECAR", "1")
    monkeypatch.setenv("CORNSERVE_MOCK_SIDECAR_DIR", str(tmp_path))
    from cornserve.sidecar.api import Sidecar
    from cornserve.sidecar.schema import SidecarConfig

    sc = Sidecar(SidecarConfig(sidecar_rank=0, send_tensor_dtype=torch.float32, send_tensor_shape=(-1, 8)))
    t = torch.arange(16.0).view(2, 8)
    sc.send(t, "abc", [[1]])
    sc.send({"a": 1}, "obj", [[1]])
    assert torch.equal(sc.recv_sync("abc"), t) and sc.recv_sync("obj") == {"a": 1} and sc.recv_sync("none") is None
    sc.mark_done_sync("abc")
    sc.shutdown_sync()
