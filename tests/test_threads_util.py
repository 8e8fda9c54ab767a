"""Interpreter tuning and the stack sampler of the executor processes."""

import sys
import threading
import time

from cornserve.utils import threads


def test_switch_interval_follows_the_environment(monkeypatch):
    before = sys.getswitchinterval()
    try:
        monkeypatch.setenv("CORNSERVE_GIL_SWITCH_S", "0.002")
        threads.tune_interpreter()
        assert abs(sys.getswitchinterval() - 0.002) < 1e-9
        monkeypatch.setenv("CORNSERVE_GIL_SWITCH_S", "not a number")
        threads.tune_interpreter()   # ignored, no exception
        assert abs(sys.getswitchinterval() - 0.002) < 1e-9
    finally:
        sys.setswitchinterval(before)


def test_stack_sampler_names_the_busy_function():
    stop = threading.Event()

    def spin_here():
        while not stop.is_set():
            sum(range(2000))

    t = threading.Thread(target=spin_here, name="spinner", daemon=True)
    t.start()
    s = threads.StackSampler(period_s=0.002).start()
    time.sleep(0.3)
    s.stop()
    stop.set()
    t.join()
    top = s.top()
    assert top["samples"] > 10
    assert any("spin_here" in where for where, _ in top["threads"]["spinner"])


def test_kernel_library_calls_keep_the_interpreter_lock():
    import ctypes

    from cornserve.ops import _lib

    if not _lib.available():
        return
    assert isinstance(_lib.load(), ctypes.PyDLL)
