"""Local process management: what pods and services are in the reference's Kubernetes deployment are
child processes with dynamically assigned localhost ports here."""

from __future__ import annotations

import asyncio
import os
import signal
import socket
import subprocess
import time
from dataclasses import dataclass, field
from pathlib import Path

from ..constants import LOG_DIR
from ..logging import get_logger

logger = get_logger(__name__)


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def to_strict_name(name: str, max_len: int = 63) -> str:
    """Lower-case alphanumerics and dashes, starting and ending with an alphanumeric (DNS-label rules,
    kept so that names stay valid if a deployment is moved back onto Kubernetes)."""
    out = "".join(c if c.isalnum() else "-" for c in name.lower())
    while "--" in out:
        out = out.replace("--", "-")
    out = out.strip("-")[:max_len].rstrip("-")
    return out or "x"


@dataclass
class ManagedProcess:
    name: str
    popen: subprocess.Popen
    log_path: Path
    port: int = 0
    started: float = field(default_factory=time.monotonic)

    @property
    def pid(self) -> int:
        return self.popen.pid

    def alive(self) -> bool:
        return self.popen.poll() is None

    def returncode(self) -> int | None:
        return self.popen.poll()

    def tail(self, lines: int = 100) -> str:
        try:
            return "\n".join(self.log_path.read_text(errors="replace").splitlines()[-lines:])
        except OSError:
            return ""


class _AdoptedPopen:
    """The part of ``subprocess.Popen`` that :class:`ManagedProcess` uses, for a process this one did not start (an
    executor that outlived the control plane that launched it)."""

    def __init__(self, pid: int):
        import psutil

        self.pid = pid
        try:
            self._ps = psutil.Process(pid)
            self._created = self._ps.create_time()
        except psutil.Error:
            self._ps = None
        self.returncode: int | None = None

    def poll(self) -> int | None:
        import psutil

        if self._ps is None:
            self.returncode = self.returncode if self.returncode is not None else -1
            return self.returncode
        try:
            if self._ps.is_running() and self._ps.status() != psutil.STATUS_ZOMBIE:
                return None
        except psutil.Error:
            pass
        self.returncode = self.returncode if self.returncode is not None else -1
        return self.returncode


def adopt(name: str, pid: int, port: int = 0, log_path: str = "") -> ManagedProcess:
    """A :class:`ManagedProcess` around an already running process (same process-group conventions as :func:`spawn`)."""
    return ManagedProcess(name, _AdoptedPopen(pid), Path(log_path or "/dev/null"), port)  # type: ignore[arg-type]


def spawn(name: str, argv: list[str], env: dict[str, str] | None = None, port: int = 0,
          log_dir: str | None = None) -> ManagedProcess:
    """Start ``argv`` in its own process group with stdout/stderr going to a per-process log file."""
    d = Path(log_dir or LOG_DIR)
    d.mkdir(parents=True, exist_ok=True)
    log_path = d / f"{to_strict_name(name)}_{int(time.time() * 1000)}.log"
    full_env = dict(os.environ)
    full_env.update(env or {})
    # the repository root must be importable in children that are started as ``python -m cornserve...``
    root = str(Path(__file__).resolve().parents[2])
    full_env["PYTHONPATH"] = root + os.pathsep + full_env.get("PYTHONPATH", "")
    f = open(log_path, "ab")
    popen = subprocess.Popen(argv, env=full_env, stdout=f, stderr=subprocess.STDOUT, start_new_session=True)
    f.close()
    logger.info("Spawned %s (pid %d, port %d), log: %s", name, popen.pid, port, log_path)
    return ManagedProcess(name, popen, log_path, port)


async def terminate(proc: ManagedProcess, grace_s: float = 10.0) -> None:
    """SIGTERM the process group, escalate to SIGKILL after ``grace_s``."""
    if not proc.alive():
        return
    try:
        os.killpg(proc.pid, signal.SIGTERM)
    except ProcessLookupError:
        return
    deadline = time.monotonic() + grace_s
    while proc.alive() and time.monotonic() < deadline:
        await asyncio.sleep(0.05)
    if proc.alive():
        logger.warning("%s did not exit after SIGTERM; sending SIGKILL", proc.name)
        try:
            os.killpg(proc.pid, signal.SIGKILL)
        except ProcessLookupError:
            pass
        while proc.alive():
            await asyncio.sleep(0.05)
