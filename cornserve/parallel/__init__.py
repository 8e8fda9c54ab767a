"""Parallel runtime: tensor/sequence/expert-parallel groups (one process per GPU), the NVLink
peer-memory fabric and the fused compute+collective kernels built on it."""

from .state import ParallelGroup, get_tp_group, init_distributed, set_tp_group, single_group  # noqa: F401
