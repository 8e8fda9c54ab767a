"""Open-loop rate sweep of a serving deployment: request throughput at a latency bound.

The reference's harness (benchmark/benchmark_cornserve.py:98-209, 399-435; default experiment benchmark/schema.py:178-242)
releases requests on a Poisson schedule, records per request when the first and the last streamed chunk arrived, and
reports request throughput with percentiles of TTFT / TPOT / E2EL.  This module runs that measurement at several arrival
rates in one go and names the best rate whose 99th-percentile end-to-end latency stays under a bound:

* a *step* is ``window_s`` seconds of Poisson arrivals at one rate;
* the ``steps`` timed steps are split into contiguous *segments*, one per rate, lowest rate first; inside a segment
  the arrivals of consecutive steps follow each other without a pause, and a segment ends when every request it sent
  has been answered (the drain belongs to the timed region);
* per segment: requests sent / completed / failed, duration (first send to last answer), request and output-token
  throughput, mean / p50 / p90 / p99 of TTFT, TPOT and E2EL;
* the result value is the highest request throughput among the segments that answered everything with p99 E2EL
  under the bound.

Both arms of ``bench.py`` drive their deployment through this module, so the schedule (a function of the seed only),
the request mix and the arithmetic are the same.
"""

from __future__ import annotations

import asyncio
import time
from collections.abc import Awaitable, Callable
from dataclasses import dataclass, field

import aiohttp
import numpy as np

from .load_generator import RequestRecord, one_request, percentiles


@dataclass
class SweepConfig:
    rates: list[float]                 # requests/s, ascending
    steps: int = 20                    # timed steps in total
    warmup: int = 5                    # untimed steps before them (at the middle rate)
    window_s: float = 8.0              # seconds of arrivals per step
    slo_e2el_s: float = 10.0           # bound on the 99th-percentile end-to-end latency
    output_tokens: int = 256           # tokens every request generates (ignore_eos): used for TPOT
    seed: int = 48105
    request_timeout_s: float = 120.0   # a request that takes longer is a failure (the latency bound is far below)
    deadline_s: float | None = None    # wall-clock budget of warm-up + timed steps; what does not fit is cut (and says so)


@dataclass
class Segment:
    rate: float
    steps: int
    sent: int = 0
    completed: int = 0
    failed: int = 0
    duration_s: float = 0.0
    request_throughput: float = 0.0
    output_token_throughput: float = 0.0
    ttft_ms: dict = field(default_factory=dict)
    tpot_ms: dict = field(default_factory=dict)
    e2el_ms: dict = field(default_factory=dict)
    slo_ok: bool = False
    device_ms: float | None = None     # the same span measured by the deployment's GPUs (max over executors)
    errors: list[str] = field(default_factory=list)


def poisson_schedule(rate: float, span_s: float, seed: int) -> np.ndarray:
    """Send offsets in ``[0, span_s)`` of a Poisson process with ``rate`` arrivals per second, conditioned on its count:
    ``round(rate * span_s)`` arrivals placed independently and uniformly over the span (which is what a Poisson process
    looks like once the number of arrivals is known).  The gaps are exponential in the limit, and the realised rate is
    the nominal one, so a short segment is not mislabelled by an unlucky draw of the count."""
    rng = np.random.default_rng(seed)
    n = max(1, int(round(rate * span_s)))
    return np.sort(rng.uniform(0.0, span_s, size=n))


def split_steps(steps: int, parts: int) -> list[int]:
    """``steps`` divided over ``parts`` segments as evenly as possible (later segments get the remainder)."""
    parts = max(1, min(parts, steps))
    base, extra = divmod(steps, parts)
    return [base + (1 if i >= parts - extra else 0) for i in range(parts)]


def _summarise(seg: Segment, records: list[RequestRecord], t_first: float, cfg: SweepConfig) -> None:
    good = [r for r in records if r.ok and r.chunk_times]
    seg.sent, seg.completed, seg.failed = len(records), len(good), len(records) - len(good)
    seg.errors = sorted({r.error for r in records if r.error})[:3]
    t_last = max((r.chunk_times[-1] for r in good), default=t_first)
    seg.duration_s = max(t_last - t_first, 1e-9)
    seg.request_throughput = seg.completed / seg.duration_s
    seg.output_token_throughput = seg.completed * cfg.output_tokens / seg.duration_s
    ms = lambda xs: {k: round(v, 2) for k, v in percentiles([x * 1e3 for x in xs]).items()}  # noqa: E731
    seg.ttft_ms = ms([r.ttft for r in good])
    seg.e2el_ms = ms([r.e2el for r in good])
    # chunks arrive per decode burst, not per token: time per output token from the known token count
    seg.tpot_ms = ms([(r.e2el - r.ttft) / max(cfg.output_tokens - 1, 1) for r in good])
    seg.slo_ok = bool(good) and seg.failed == 0 and seg.e2el_ms["p99"] <= cfg.slo_e2el_s * 1e3


async def _drive(http: aiohttp.ClientSession, url: str, payload_of: Callable[[int], dict], first_index: int,
                 offsets: np.ndarray, give_up_at: float | None = None) -> tuple[list[RequestRecord], float]:
    """Send one request at every offset (open loop) and wait for all answers; requests that are still unanswered at
    ``give_up_at`` (a ``perf_counter`` value) are cancelled and count as failures."""
    records = [RequestRecord(0.0) for _ in offsets]
    t0 = time.perf_counter()
    tasks = []
    for k, (rec, at) in enumerate(zip(records, offsets)):
        delay = t0 + float(at) - time.perf_counter()
        if delay > 0:
            await asyncio.sleep(delay)
        if give_up_at is not None and time.perf_counter() > give_up_at:
            rec.ok, rec.error = False, "not sent: out of time"
            continue
        tasks.append(asyncio.create_task(one_request(http, url, payload_of(first_index + k), rec)))
    if tasks:
        left = None if give_up_at is None else max(0.0, give_up_at - time.perf_counter())
        _, pending = await asyncio.wait(tasks, timeout=left)
        for t in pending:
            t.cancel()
        if pending:
            await asyncio.gather(*pending, return_exceptions=True)
            for rec in records:
                if not rec.ok and not rec.error:
                    rec.error = "no answer before the deadline"
    return records, t0


Hook = Callable[[str, int], Awaitable[None]]


async def run_sweep(url: str, payload_of: Callable[[int], dict], cfg: SweepConfig, hook: Hook | None = None) -> dict:
    """Warm up, then run the timed steps.  ``hook(phase, segment)`` is awaited with phase ``"begin"`` right before a
    timed segment's first request and ``"end"`` right after its last answer (device-side marks go there).  Returns the
    segments and the wall-clock length of the whole timed region."""
    rates = sorted(cfg.rates)
    per_seg = split_steps(cfg.steps, len(rates))
    rates = rates[len(rates) - len(per_seg):] if len(per_seg) < len(rates) else rates
    timeout = aiohttp.ClientTimeout(total=cfg.request_timeout_s)
    segments: list[Segment] = []
    index = 0
    give_up_at = None if cfg.deadline_s is None else time.perf_counter() + cfg.deadline_s
    truncated = False
    async with aiohttp.ClientSession(timeout=timeout, connector=aiohttp.TCPConnector(limit=0)) as http:
        if cfg.warmup > 0:
            mid = rates[len(rates) // 2]
            off = poisson_schedule(mid, cfg.warmup * cfg.window_s, cfg.seed - 1)
            recs, _ = await _drive(http, url, payload_of, index, off, give_up_at)
            index += len(off)
            bad = [r.error for r in recs if not r.ok]
            if bad and 2 * len(bad) >= len(recs):
                # a deployment that answers a few requests and then stalls is as unusable as one that answers none
                raise RuntimeError(f"{len(bad)} of {len(recs)} warm-up requests failed: {bad[0]}")
        t_begin = time.perf_counter()
        for i, (rate, n_steps) in enumerate(zip(rates, per_seg)):
            if give_up_at is not None and time.perf_counter() + n_steps * cfg.window_s > give_up_at:
                truncated = True   # this segment's arrivals alone would run past the budget
                break
            seg = Segment(rate=rate, steps=n_steps)
            off = poisson_schedule(rate, n_steps * cfg.window_s, cfg.seed + i)
            if hook is not None:
                await hook("begin", i)
            recs, t0 = await _drive(http, url, payload_of, index, off, give_up_at)
            if hook is not None:
                await hook("end", i)
            index += len(off)
            _summarise(seg, recs, t0, cfg)
            segments.append(seg)
        t_end = time.perf_counter()
    return {"segments": segments, "timed_s": t_end - t_begin, "requests": index, "truncated": truncated,
            "steps_run": sum(s.steps for s in segments)}


def best_segment(segments: list[Segment]) -> Segment | None:
    ok = [s for s in segments if s.slo_ok]
    return max(ok, key=lambda s: s.request_throughput) if ok else None
