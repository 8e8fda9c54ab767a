"""Addresses of sidecar servers.  Every GPU has one sidecar server with a fixed rank; rank ``r`` listens
for gRPC on ``SIDECAR_GRPC_BASE_PORT + r`` on the local host (the reference derives Kubernetes service
names instead: python/cornserve/sidecar/constants.py:11-35)."""

from __future__ import annotations

import os

from ..constants import SIDECAR_GRPC_BASE_PORT

RANK_ENV = "SIDECAR_RANK"
WORLD_SIZE_ENV = "SIDECAR_WORLD_SIZE"
SHM_SIZE_ENV = "SIDECAR_SHM_SIZE"
DEVICE_ENV = "SIDECAR_DEVICE"          # "cpu", "cuda" or "cuda:<index>"; default: cuda:<rank> when available
HANDLE_DIR = os.environ.get("SIDECAR_HANDLE_DIR", "/dev/shm")


def grpc_port(rank: int) -> int:
    return SIDECAR_GRPC_BASE_PORT + rank


def grpc_url(rank: int) -> str:
    host = os.environ.get("SIDECAR_HOST", "127.0.0.1")
    return f"{host}:{grpc_port(rank)}"


def slab_handle_path(rank: int) -> str:
    """File in which sidecar ``rank`` publishes how other processes can map its slab."""
    ns = os.environ.get("SIDECAR_NAMESPACE", "default")
    return os.path.join(HANDLE_DIR, f"cornserve_sidecar_{ns}_{rank}.handle")


def shm_slab_path(rank: int) -> str:
    ns = os.environ.get("SIDECAR_NAMESPACE", "default")
    return os.path.join(HANDLE_DIR, f"cornserve_sidecar_{ns}_{rank}.slab")
