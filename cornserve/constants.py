"""Deployment constants.  Kubernetes service names of the reference (python/cornserve/constants.py:61-125)
become localhost endpoints: every service is a local process and ports are handed out dynamically by
the resource manager, except for the well-known entry points below (overridable by environment)."""

from __future__ import annotations

import os

GATEWAY_HOST = os.environ.get("CORNSERVE_GATEWAY_HOST", "127.0.0.1")
GATEWAY_HTTP_PORT = int(os.environ.get("CORNSERVE_GATEWAY_PORT", "8000"))
GATEWAY_URL = os.environ.get("CORNSERVE_GATEWAY_URL", f"http://{GATEWAY_HOST}:{GATEWAY_HTTP_PORT}")

RESOURCE_MANAGER_GRPC_URL = os.environ.get("CORNSERVE_RESOURCE_MANAGER_URL", "127.0.0.1:50051")
TASK_DISPATCHER_HTTP_URL = os.environ.get("CORNSERVE_TASK_DISPATCHER_HTTP_URL", "http://127.0.0.1:8001")
TASK_DISPATCHER_GRPC_URL = os.environ.get("CORNSERVE_TASK_DISPATCHER_GRPC_URL", "127.0.0.1:50052")

STATE_DIR = os.environ.get("CORNSERVE_STATE_DIR", os.path.expanduser("~/.local/state/cornserve"))
LOG_DIR = os.environ.get("CORNSERVE_LOG_DIR", os.path.join(STATE_DIR, "logs"))
TASKLIB_DIR = os.environ.get("CORNSERVE_TASKLIB_DIR", "/tmp/cornserve_tasklib")

TASK_TIMEOUT_S = 30 * 60
EXECUTOR_HEALTHY_TIMEOUT_S = float(os.environ.get("CORNSERVE_EXECUTOR_HEALTHY_TIMEOUT", 20 * 60))
EXECUTOR_HEALTH_POLL_S = 0.5
SIDECAR_HEALTHY_TIMEOUT_S = 5 * 60
SYNC_WATCHERS_TIMEOUT_S = 30.0

SIDECAR_GRPC_BASE_PORT = int(os.environ.get("CORNSERVE_SIDECAR_BASE_PORT", "10000"))

# names of the five object kinds kept by the registry store (custom resources in the reference)
KIND_TASK_DEFINITION = "TaskDefinition"
KIND_EXECUTION_DESCRIPTOR = "ExecutionDescriptor"
KIND_UNIT_TASK_INSTANCE = "UnitTaskInstance"
KIND_UNIT_TASK_PROFILE = "UnitTaskProfile"
KIND_LATEST_TASKLIB_RV = "LatestTasklibRV"
# what is running where, so that a restarted control plane can take its processes over again
KIND_TASK_MANAGER_RECORD = "TaskManagerRecord"
KIND_EXECUTOR_RECORD = "ExecutorRecord"
KIND_SIDECAR_RECORD = "SidecarRecord"
