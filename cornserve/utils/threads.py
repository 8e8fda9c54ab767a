"""Interpreter settings for processes that launch kernels from several threads, and a stack sampler to see what they do.

An executor process has an event loop, an engine thread and (in the no-fission layout) a vision-tower thread.  Each
kernel launch of the tower is a short native call; when such a call gives up the interpreter lock and another thread is
busy, getting the lock back takes up to one *switch interval* (5 ms by default), and a forward pass of some hundred
launches turns into seconds.  ``tune_interpreter`` shortens the interval; the kernel library is loaded so that its
launches keep the lock (``cornserve/ops/_lib.py``).
"""

from __future__ import annotations

import collections
import os
import sys
import threading
import time


def tune_interpreter() -> None:
    """Set the interpreter's thread switch interval (``CORNSERVE_GIL_SWITCH_S``, default 0.1 ms).

    A thread that launches a tower forward makes a few thousand short calls that give the lock up; whenever another
    thread holds it at that moment the launcher waits up to one interval, so the interval bounds what a forward pass
    loses to the other threads of the process (measured: 5 ms -> 480 ms per batch, 0.5 ms -> 180 ms)."""
    try:
        sys.setswitchinterval(max(1e-5, float(os.environ.get("CORNSERVE_GIL_SWITCH_S", "0.0001"))))
    except ValueError:
        pass


class StackSampler:
    """Samples every thread's innermost frames at a fixed period; ``top()`` gives the most frequent ones per thread.

    Enabled in the executors by ``CORNSERVE_SAMPLE_STACKS=1``; the result is part of their ``/stats`` answer.  The
    sampler needs the interpreter lock to look, so it sees a busy thread mostly at the calls where that thread gives
    the lock up (a copy, a wait, a library call): read the counts as "where threads yield", not as CPU time."""

    def __init__(self, period_s: float = 0.005, depth: int = 3):
        self.period_s, self.depth = period_s, depth
        self.counts: dict[str, collections.Counter] = collections.defaultdict(collections.Counter)
        self.samples = 0
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._run, name="stack-sampler", daemon=True)

    def start(self) -> "StackSampler":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()

    def _run(self) -> None:
        me = threading.get_ident()
        while not self._stop.wait(self.period_s):
            names = {t.ident: t.name for t in threading.enumerate()}
            for ident, frame in sys._current_frames().items():
                if ident == me:
                    continue
                where = []
                f = frame
                while f is not None and len(where) < self.depth:
                    where.append(f"{os.path.basename(f.f_code.co_filename)}:{f.f_lineno}:{f.f_code.co_name}")
                    f = f.f_back
                self.counts[names.get(ident, str(ident))][" < ".join(where)] += 1
            self.samples += 1

    def top(self, n: int = 8) -> dict:
        return {"samples": self.samples, "period_s": self.period_s,
                "threads": {name: c.most_common(n) for name, c in self.counts.items()}}


_sampler: StackSampler | None = None


def maybe_start_sampler() -> StackSampler | None:
    global _sampler
    if _sampler is None and os.environ.get("CORNSERVE_SAMPLE_STACKS") == "1":
        _sampler = StackSampler().start()
    return _sampler


def sampler_report() -> dict | None:
    return _sampler.top() if _sampler is not None else None


def wall_ms(t0: float) -> float:
    return (time.perf_counter() - t0) * 1e3
