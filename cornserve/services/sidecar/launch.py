"""Starting and stopping sidecar server processes on the local box (the reference builds pod specs:
python/cornserve/services/sidecar/launch.py:10-116)."""

from __future__ import annotations

import os
import subprocess
import sys
import time

import grpc

from ...sidecar.constants import DEVICE_ENV, RANK_ENV, SHM_SIZE_ENV, WORLD_SIZE_ENV, grpc_url
from ..pb import sidecar_pb2, sidecar_pb2_grpc


def spawn_sidecar(rank: int, world_size: int, slab_bytes: int = 1 << 30, device: str | None = None,
                  env: dict[str, str] | None = None, log_path: str | None = None) -> subprocess.Popen:
    e = dict(os.environ)
    e.update({RANK_ENV: str(rank), WORLD_SIZE_ENV: str(world_size), SHM_SIZE_ENV: str(slab_bytes)})
    if device:
        e[DEVICE_ENV] = device
    e.update(env or {})
    out = open(log_path, "ab") if log_path else subprocess.DEVNULL
    return subprocess.Popen([sys.executable, "-m", "cornserve.services.sidecar.server"], env=e, stdout=out,
                            stderr=subprocess.STDOUT, start_new_session=True)


def check_health(rank: int, timeout_s: float = 1.0) -> int | None:
    """Health status of sidecar ``rank`` or ``None`` when it does not answer."""
    try:
        with grpc.insecure_channel(grpc_url(rank)) as ch:
            return sidecar_pb2_grpc.SidecarStub(ch).CheckHealth(sidecar_pb2.CheckHealthRequest(), timeout=timeout_s).status
    except grpc.RpcError:
        return None


def wait_all_good(ranks: list[int], timeout_s: float = 300.0, procs: list | None = None) -> bool:
    """Wait until every listed sidecar reports ``ALL_GOOD``.  With ``procs`` (the ``Popen`` objects of sidecars started
    for this wait) the wait ends at once when one of them has exited: a sidecar that died will never answer."""
    deadline = time.monotonic() + timeout_s
    pending = set(ranks)
    while pending and time.monotonic() < deadline:
        for r in list(pending):
            if check_health(r) == sidecar_pb2.HealthStatus.HEALTH_ALL_GOOD:
                pending.discard(r)
        if pending and procs and any(p.poll() is not None for p in procs):
            return False
        if pending:
            time.sleep(0.2)
    return not pending
