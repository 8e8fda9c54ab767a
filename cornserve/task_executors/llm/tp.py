"""Tensor-parallel serving of the LLM executor (``--tensor-parallel-size N``).

Contract (reference: tasklib/cornserve_tasklib/task_executors/descriptor/llm.py launches its vLLM with
``--tensor-parallel-size <number of GPUs>``): one executor, one HTTP endpoint, the model sharded over the GPUs the task
manager granted.

Rank 0 is the process the task manager started: it owns the HTTP server, the sidecar client and the request queue.  It
starts one follower process per further GPU.  Every rank runs the same deterministic engine (scheduler, block manager,
CUDA-graph decode) on the same requests in the same order, so their collectives inside the model line up without any
per-step negotiation: before each engine step the leader publishes the requests that were added since the last one
(prompt ids, sampling parameters with the seed already drawn, and the encoder rows that replace placeholder tokens), the
followers add them and step.  Control messages travel over a gloo group whose waits do not expire while the executor is
idle; encoder rows are broadcast over the ranks' data group (NCCL on GPUs) from a buffer of the leader's own memory.
"""

from __future__ import annotations

import dataclasses
import datetime
import os
import socket
import subprocess
import sys
import time
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from ...logging import get_logger
from ...parallel.state import ParallelGroup, init_distributed
from .engine import LLMEngine, MMItem, SamplingParams, Sequence

logger = get_logger(__name__)

IDLE_BEAT_S = 5.0          # the leader's keep-alive period while it has nothing to run
CONTROL_TIMEOUT_S = 120.0  # a follower gives up when the leader stays silent this long


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


def rank_device_index(rank: int) -> int | None:
    """GPU of tensor-parallel rank ``rank``: the rank-th entry of the GPUs granted to this executor."""
    ids = [int(x) for x in os.environ.get("CORNSERVE_LOCAL_GPUS", "").split(",") if x.strip() != ""]
    return ids[rank] if rank < len(ids) else rank


def join_group(rank: int, world: int, port: int) -> ParallelGroup:
    cpu = not torch.cuda.is_available() or os.environ.get("CORNSERVE_DEVICE") == "cpu"
    return init_distributed(rank, world, master_addr="127.0.0.1", master_port=port, backend="gloo" if cpu else None,
                            local_device=None if cpu else rank_device_index(rank))


def agree_on_min(value: int, group: ParallelGroup) -> int:
    """The smallest ``value`` over the ranks (e.g. KV pages that fit everywhere: the schedulers must decide alike)."""
    if group.size == 1:
        return value
    t = torch.tensor([value], dtype=torch.int64, device=group.device)
    dist.all_reduce(t, op=dist.ReduceOp.MIN)
    return int(t.item())


def _pack(seq: Sequence) -> dict[str, Any]:
    return {"seq_id": seq.seq_id, "prompt_ids": np.asarray(seq.prompt_ids), "params": dataclasses.asdict(seq.params),
            "positions": seq.positions, "next_pos": seq.next_pos,
            "mm": [(it.offset, it.grid_thw, tuple(it.embeds.shape), it.second_per_grid) for it in seq.mm_items]}


class TPControl:
    """The leader's publish / the followers' receive of one engine step."""

    def __init__(self, group: ParallelGroup, dtype: torch.dtype):
        self.group, self.dtype = group, dtype
        # An idle executor publishes nothing, so a follower may wait here for as long as no request comes: the leader
        # sends an empty "keep-alive" step every IDLE_BEAT_S seconds, which lets this wait carry a finite timeout.  A
        # leader that died is then noticed after CONTROL_TIMEOUT_S instead of never.
        self.ctl = dist.new_group(backend="gloo", timeout=datetime.timedelta(seconds=CONTROL_TIMEOUT_S))
        self.publish_ms = 0.0

    # -- rank 0 -------------------------------------------------------------------------------------------
    def publish(self, seqs: list[Sequence], stop: bool = False, beat: bool = False, aborts: list[str] | None = None) -> None:
        t0 = time.perf_counter()
        dist.broadcast_object_list([{"stop": stop, "beat": beat, "aborts": list(aborts or []), "seqs": [_pack(s) for s in seqs]}],
                                   src=0, group=self.ctl)
        for s in seqs:
            for it in s.mm_items:
                # a buffer of this GPU's own memory: the rows may sit in another process's slab
                own = torch.empty(tuple(it.embeds.shape), device=self.group.device, dtype=self.dtype)
                own.copy_(it.embeds)
                dist.broadcast(own, src=0)
        self.publish_ms += (time.perf_counter() - t0) * 1e3

    # -- other ranks -----------------------------------------------------------------------------------------
    def receive(self) -> tuple[bool, list[Sequence], list[str]] | None:
        """``(stop, new sequences, aborted sequence ids)`` of the next engine step, or ``None`` for a keep-alive."""
        box: list[Any] = [None]
        dist.broadcast_object_list(box, src=0, group=self.ctl)
        msg = box[0]
        if msg.get("beat"):
            return None
        seqs = []
        for d in msg["seqs"]:
            items = []
            for offset, grid, shape, spg in d["mm"]:
                rows = torch.empty(shape, device=self.group.device, dtype=self.dtype)
                dist.broadcast(rows, src=0)
                items.append(MMItem(rows, offset, grid, spg))
            s = Sequence(d["seq_id"], d["prompt_ids"], SamplingParams(**d["params"]), mm_items=items)
            s.positions, s.next_pos = d["positions"], d["next_pos"]
            seqs.append(s)
        return bool(msg["stop"]), seqs, list(msg.get("aborts") or [])


def follower_loop(engine: LLMEngine, ctl: TPControl) -> None:
    """Mirror the leader: add what it added, step when it steps, until it says stop."""
    while True:
        got = ctl.receive()
        if got is None:
            continue
        stop, seqs, aborts = got
        if stop:
            return
        for sid in aborts:
            engine.abort(sid)
        for s in seqs:
            try:
                engine.add_request(s)
            except Exception as e:  # noqa: BLE001  (the leader refused the same request for the same reason)
                logger.warning("follower refused %s: %s", s.seq_id, e)
        engine.step()


def spawn_followers(argv: list[str], world: int, port: int) -> list[subprocess.Popen]:
    """One process per further rank, same command line plus its rank and the rendezvous port."""
    procs = []
    for r in range(1, world):
        cmd = [sys.executable, "-m", "cornserve.task_executors.llm.server", *argv, "--tp-rank", str(r), "--tp-port", str(port)]
        procs.append(subprocess.Popen(cmd, env=dict(os.environ)))
    return procs
