"""Follows the log files of task executors while an app is being registered (the reference tails the logs of
``te-<task>*`` pods: python/cornserve/cli/log_streamer.py:33-193; here executors are local processes whose output
goes to ``<log dir>/<executor>_<timestamp>.log``)."""

from __future__ import annotations

import itertools
import sys
import threading
import time
from pathlib import Path

from ..constants import LOG_DIR
from ..services.process import to_strict_name

_COLOURS = ["\033[36m", "\033[35m", "\033[33m", "\033[32m", "\033[34m", "\033[91m"]
_RESET = "\033[0m"


class LogStreamer:
    def __init__(self, task_names: list[str], log_dir: str | None = None, out=None, poll_s: float = 0.3) -> None:
        self.prefixes = [to_strict_name(f"te-{n}") for n in task_names]
        self.dir = Path(log_dir or LOG_DIR)
        self.out = out or sys.stderr
        self.poll_s = poll_s
        self._stop = threading.Event()
        self._seen: dict[Path, int] = {}
        self._colours = itertools.cycle(_COLOURS)
        self._colour_of: dict[Path, str] = {}
        self._start_time = time.time()
        self._thread = threading.Thread(target=self._run, name="log-streamer", daemon=True)

    def start(self) -> "LogStreamer":
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        self._thread.join(timeout=2)

    def _matches(self, p: Path) -> bool:
        # executor names embed the descriptor's executor name, which need not equal the task name: follow every
        # executor log that appeared after the streamer started, plus the ones that match a task prefix
        return p.name.startswith("te-") and (p.stat().st_mtime >= self._start_time - 1 or any(p.name.startswith(x) for x in self.prefixes))

    def _run(self) -> None:
        while not self._stop.is_set():
            self.poll_once()
            self._stop.wait(self.poll_s)
        self.poll_once()

    def poll_once(self) -> None:
        if not self.dir.is_dir():
            return
        for p in sorted(self.dir.glob("te-*.log")):
            try:
                if not self._matches(p):
                    continue
                size = p.stat().st_size
                off = self._seen.get(p, 0)
                if size <= off:
                    continue
                with open(p, "rb") as f:
                    f.seek(off)
                    chunk = f.read(size - off)
                self._seen[p] = size
            except OSError:
                continue
            colour = self._colour_of.setdefault(p, next(self._colours))
            tag = p.name.rsplit("_", 1)[0]
            for line in chunk.decode(errors="replace").splitlines():
                self.out.write(f"{colour}[{tag}]{_RESET} {line}\n")
            self.out.flush()
