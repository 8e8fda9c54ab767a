"""Timer routes of the executors: marks and the span between two of them (host clock on a CPU executor)."""

import time

from fastapi import FastAPI
from fastapi.testclient import TestClient

from cornserve.task_executors.device_timer import DeviceTimer, add_timer_routes


def test_marks_are_ordered_and_spans_add_up():
    t = DeviceTimer("cpu")
    a = t.mark()
    time.sleep(0.02)
    b = t.mark()
    time.sleep(0.01)
    c = t.mark()
    assert (a, b, c) == (0, 1, 2)
    ab, bc, ac = t.elapsed_ms(a, b), t.elapsed_ms(b, c), t.elapsed_ms(a, c)
    assert ab >= 19 and bc >= 9 and abs(ab + bc - ac) < 1e-6


def test_timer_routes_answer_over_http():
    app = FastAPI()
    add_timer_routes(app, "cpu")
    with TestClient(app) as http:
        first = http.post("/timer/mark").json()["mark"]
        time.sleep(0.01)
        second = http.post("/timer/mark").json()["mark"]
        got = http.get("/timer/elapsed", params={"start": first, "end": second}).json()
    assert second == first + 1 and got["device"] == "cpu" and got["ms"] >= 9
