"""Time spans on an executor's GPU, read through its HTTP API.

A load test that wants its timed region measured by the device (CUDA events) rather than by the client's clock asks
every executor for a mark before the first request and another after the last answer, then for the time between the
two marks; the slowest executor's span is the region.  On a CPU executor the marks are host timestamps."""

from __future__ import annotations

import threading
import time

import torch


class DeviceTimer:
    def __init__(self, device: torch.device | str):
        self.device = torch.device(device)
        self._marks: list = []
        self._lock = threading.Lock()

    def mark(self) -> int:
        """Record "now" on the device's default stream (it completes once the work queued so far has run)."""
        with self._lock:
            if self.device.type == "cuda":
                ev = torch.cuda.Event(enable_timing=True)
                ev.record(torch.cuda.default_stream(self.device))
            else:
                ev = time.perf_counter()
            self._marks.append(ev)
            return len(self._marks) - 1

    def elapsed_ms(self, start: int, end: int) -> float:
        a, b = self._marks[start], self._marks[end]
        if self.device.type == "cuda":
            b.synchronize()
            return float(a.elapsed_time(b))
        return (b - a) * 1e3


def add_timer_routes(app, device: torch.device | str) -> DeviceTimer:
    timer = DeviceTimer(device)

    @app.post("/timer/mark")
    async def timer_mark():
        return {"mark": timer.mark()}

    @app.get("/timer/elapsed")
    async def timer_elapsed(start: int, end: int):
        return {"ms": timer.elapsed_ms(start, end), "device": str(timer.device)}

    return timer
