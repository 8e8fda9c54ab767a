"""The sidecar's GPU path: a producer's tensor is pushed into the slab of the consumer's GPU by the copy kernel (over
NVLink when the two sidecars sit on different GPUs) and the consumer gets a view of its own GPU's memory."""

import json
import os
import signal
import socket
import time
import uuid

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def gpu_sidecars():
    ns = uuid.uuid4().hex[:8]
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    base = s.getsockname()[1]
    s.close()
    os.environ["CORNSERVE_SIDECAR_BASE_PORT"] = str(base if base + 8 < 65000 else 20000)
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
    env = {"CORNSERVE_SIDECAR_BASE_PORT": os.environ["CORNSERVE_SIDECAR_BASE_PORT"], "SIDECAR_NAMESPACE": ns,
           "CORNSERVE_LOG_LEVEL": "INFO", "SIDECAR_PUSH_PROBE": "1"}
    n = torch.cuda.device_count()
    devices = ["cuda:0", f"cuda:{min(1, n - 1)}"]
    procs = [launch.spawn_sidecar(r, 2, slab_bytes=512 << 20, device=devices[r], env=env) for r in range(2)]
    assert launch.wait_all_good([0, 1], 120), "sidecar servers did not come up"
    yield api, devices, sc
    for p in procs:
        try:
            os.killpg(p.pid, signal.SIGTERM)
        except ProcessLookupError:
            pass
    for p in procs:
        p.wait(timeout=20)


def test_push_lands_in_the_consumers_gpu_memory_and_is_timed(gpu_sidecars):
    api, devices, sc = gpu_sidecars
    from cornserve.sidecar.schema import SidecarConfig

    def client(rank):
        torch.cuda.set_device(devices[rank])
        return api.Sidecar(SidecarConfig(sidecar_rank=rank, group=None, send_tensor_dtype=torch.bfloat16,
                                         send_tensor_shape=(-1, 3584), recv_tensor_dtype=torch.bfloat16,
                                         recv_tensor_shape=(-1, 3584)))

    prod, cons = client(0), client(1)
    try:
        rows = 1196                                         # one 1280x720 image of Qwen2.5-VL: 8.6 MB of bf16 rows
        src = [torch.randn(rows, 3584, device=devices[0]).bfloat16() for _ in range(4)]
        torch.cuda.synchronize()
        lat = []
        for i in range(24):
            did = uuid.uuid4().hex
            t = src[i % 4]
            t0 = time.perf_counter()
            prod.send(t, did, [[1]])
            got = cons.recv_sync(did)
            lat.append((time.perf_counter() - t0) * 1e3)
            assert got.device == torch.device(devices[1]) and got.shape == t.shape
            if i < 4:
                assert torch.equal(got.to(devices[0]), t)
            cons.mark_done_sync(did)
        prod.flush()
        # odd sizes and another dtype through the same slab
        odd = torch.arange(7 * 13, device=devices[0], dtype=torch.float32).view(7, 13)
        o2 = api.Sidecar(SidecarConfig(sidecar_rank=0, group=None, send_tensor_dtype=torch.float32, send_tensor_shape=(-1, 13)))
        o2.send(odd, "odd", [[1]])
        c2 = api.Sidecar(SidecarConfig(sidecar_rank=1, group=None, recv_tensor_dtype=torch.float32, recv_tensor_shape=(-1, 13)))
        assert torch.equal(c2.recv_sync("odd").cpu(), odd.cpu())
        c2.mark_done_sync("odd")
        o2.shutdown_sync()
        c2.shutdown_sync()
        time.sleep(0.2)
        stats = json.loads(open(sc.slab_handle_path(0) + ".stats").read())
        gbs = stats["bytes"] / 1e6 / max(stats["copy_ms"], 1e-9)
        lat = sorted(lat[4:])
        print(f"\\nsidecar push {devices[0]} -> {devices[1]}: {rows}x3584 bf16 = {rows * 3584 * 2 / 1e6:.1f} MB; copy kernel "
              f"{stats['copy_ms'] / stats['pushes'] * 1e3:.1f} us per push = {gbs:.0f} GB/s (the same copy repeated at once: "
              f"{stats.get('repeat_ms', 0.0) / stats['pushes'] * 1e3:.1f} us); send -> rows visible at the "
              f"consumer (client clocks, 3 RPCs): median {lat[len(lat) // 2]:.2f} ms, min {lat[0]:.2f} ms")
        out_dir = os.environ.get("CORNSERVE_TEST_ARTIFACTS", "")   # where to leave the figures, when they are wanted as a file
        with open(os.path.join(out_dir, "sidecar_push.json") if out_dir else os.devnull, "w") as f:
            json.dump({"devices": devices, "rows": rows, "bytes": rows * 3584 * 2, "copy_us": stats["copy_ms"] / stats["pushes"] * 1e3,
                       "repeat_copy_us": stats.get("repeat_ms", 0.0) / stats["pushes"] * 1e3,
                       "copy_gbs": gbs, "send_to_visible_ms_median": lat[len(lat) // 2], "send_to_visible_ms_min": lat[0]}, f)
        assert stats["pushes"] >= 16
    finally:
        prod.shutdown_sync()
        cons.shutdown_sync()
