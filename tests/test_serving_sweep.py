"""The rate-sweep harness behind ``bench.py``: schedule, step split, latency arithmetic, and the whole benchmark as a
plumbing run (tiny model, CPU ranks) through ``cornserve up`` -> gateway -> dispatcher -> Eric -> sidecar -> LLM."""

import json
import socket
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

ROOT = Path(__file__).resolve().parents[1]


def test_poisson_schedule_is_a_function_of_the_seed_and_has_the_rate():
    from benchmark.serving_sweep import poisson_schedule

    a, b = poisson_schedule(20.0, 50.0, 7), poisson_schedule(20.0, 50.0, 7)
    assert np.array_equal(a, b) and not np.array_equal(a, poisson_schedule(20.0, 50.0, 8))
    assert a[0] > 0 and a[-1] < 50.0 and np.all(np.diff(a) > 0)
    assert len(a) == 1000                                      # rate * span arrivals exactly
    gaps = np.diff(a)
    assert abs(gaps.std() / gaps.mean() - 1.0) < 0.15           # exponential gaps: coefficient of variation 1


def test_steps_are_split_over_rates_without_losing_any():
    from benchmark.serving_sweep import split_steps

    assert split_steps(20, 5) == [4, 4, 4, 4, 4]
    assert split_steps(7, 3) == [2, 2, 3]
    assert split_steps(2, 5) == [1, 1]
    assert sum(split_steps(13, 4)) == 13


def test_segment_summary_and_bound():
    from benchmark.load_generator import RequestRecord
    from benchmark.serving_sweep import Segment, SweepConfig, _summarise, best_segment

    cfg = SweepConfig(rates=[1.0], output_tokens=11, slo_e2el_s=2.0)
    recs = []
    for i in range(10):
        r = RequestRecord(send_time=float(i))
        r.chunk_times = [i + 0.5, i + 1.5]       # first token after 0.5 s, done after 1.5 s
        r.ok = True
        recs.append(r)
    seg = Segment(rate=1.0, steps=1)
    _summarise(seg, recs, 0.0, cfg)
    assert seg.completed == 10 and seg.failed == 0 and abs(seg.duration_s - 10.5) < 1e-9
    assert abs(seg.request_throughput - 10 / 10.5) < 1e-9
    assert seg.ttft_ms["p99"] == 500.0 and seg.e2el_ms["median"] == 1500.0 and seg.tpot_ms["mean"] == 100.0
    assert seg.slo_ok
    slow = Segment(rate=2.0, steps=1)
    recs[3].chunk_times[-1] += 5.0              # one straggler breaks the p99 bound
    _summarise(slow, recs, 0.0, cfg)
    assert not slow.slo_ok
    failed = Segment(rate=3.0, steps=1)
    recs[3].ok = False
    _summarise(failed, recs, 0.0, cfg)
    assert failed.failed == 1 and not failed.slo_ok
    assert best_segment([seg, slow, failed]) is seg and best_segment([slow]) is None


def test_sweep_stops_at_its_deadline_instead_of_waiting_for_a_stalled_server():
    """A server that stops answering: requests in flight at the deadline are cancelled and counted as failures, segments
    whose arrivals no longer fit are dropped, and the result says that it was cut short."""
    import asyncio

    from aiohttp import web

    from benchmark.serving_sweep import SweepConfig, run_sweep

    served = {"n": 0}

    async def invoke(request: web.Request) -> web.StreamResponse:
        served["n"] += 1
        resp = web.StreamResponse()
        await resp.prepare(request)
        if served["n"] > 6:
            await asyncio.sleep(3600)          # the deployment has stalled
        await resp.write(b'{"choices": [{"delta": {"content": "a"}}]}\n')   # the gateway streams one JSON object per line
        await resp.write(b'{"choices": [{"delta": {"content": "b"}}]}\n')
        return resp

    async def main():
        app = web.Application()
        app.router.add_post("/invoke", invoke)
        runner = web.AppRunner(app)
        await runner.setup()
        site = web.TCPSite(runner, "127.0.0.1", 0, shutdown_timeout=0.5)
        await site.start()
        port = site._server.sockets[0].getsockname()[1]
        try:
            cfg = SweepConfig(rates=[4.0, 6.0, 8.0], steps=3, warmup=0, window_s=1.0, output_tokens=2, deadline_s=3.0)
            return await run_sweep(f"http://127.0.0.1:{port}/invoke", lambda i: {"i": i}, cfg)
        finally:
            await runner.cleanup()

    res = asyncio.run(main())
    assert res["truncated"] and 1 <= len(res["segments"]) < 3 and res["steps_run"] == len(res["segments"])
    first, last = res["segments"][0], res["segments"][-1]
    assert first.completed == 4 and first.failed == 0
    assert last.failed > 0 and not last.slo_ok and "deadline" in " ".join(last.errors)


@pytest.mark.timeout(900)
def test_bench_monolithic_layout_encodes_inside_the_llm_executor():
    """One rank: no encoder executor; the LLM executor's own vision tower thread encodes the images (and counts them)."""
    out = subprocess.run([sys.executable, "bench.py", "--small", "--cpu", "--gpus", "1", "--steps", "2", "--warmup", "1",
                          "--window-s", "2", "--rates", "1,2", "--offline-steps", "0", "--output-tokens", "8"],
                         cwd=ROOT, capture_output=True, text=True, timeout=800)
    assert out.returncode == 0, out.stderr[-3000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["config"]["parallelism"].startswith("1 x monolithic")
    (llm,) = line["executors"]
    assert llm["executor"] == "llm" and llm["local_encoder_images"] > 0 and llm["requests"] == sum(s["sent"] for s in line["sweep"])
    assert all(s["failed"] == 0 for s in line["sweep"]) and line["e2e"]["h2d_bytes_per_step"] > 0


@pytest.mark.timeout(900)
def test_bench_runs_end_to_end_on_cpu_ranks():
    out = subprocess.run([sys.executable, "bench.py", "--small", "--cpu", "--gpus", "2", "--steps", "2", "--warmup", "1",
                          "--window-s", "2", "--rates", "1,2", "--offline-steps", "0", "--output-tokens", "8"],
                         cwd=ROOT, capture_output=True, text=True, timeout=800)
    assert out.returncode == 0, out.stderr[-3000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["metric"] == "requests_per_second_at_p99_e2el_slo" and line["n_gpus"] == 2 and line["steps"] == 2
    assert line["config"]["parallelism"] == "eric tp1 x1 + llm tp1 x1"
    assert len(line["sweep"]) == 2 and all(s["failed"] == 0 and s["completed"] == s["sent"] > 0 for s in line["sweep"])
    assert line["value"] > 0 and line["e2e"]["value"] > 0 and line["e2e"]["d2h_bytes_per_step"] > 0
    assert abs(line["ms_per_step"] * 2 / 1e3 - sum(s["duration_s"] for s in line["sweep"])) < 3.0
    assert {e["executor"] for e in line["executors"]} == {"eric", "llm"}


@pytest.mark.timeout(400)
def test_a_killed_bench_leaves_no_process_of_its_deployment_behind():
    """The control plane, executors and sidecars run in sessions of their own; when ``bench.py`` is killed outright they
    must not stay behind holding GPUs for the next run: every process of the tree leaves once its parent is gone."""
    import os
    import signal
    import time

    import psutil

    def members(tag):
        out = []
        for p in psutil.process_iter(["pid"]):
            try:
                if p.environ().get("SIDECAR_NAMESPACE") == tag:
                    out.append(p.pid)
            except (psutil.Error, OSError):
                pass
        return out

    b = subprocess.Popen([sys.executable, "bench.py", "--gpus", "2", "--cpu", "--small", "--steps", "4", "--warmup", "1",
                          "--window-s", "5", "--offline-steps", "0", "--rates", "1", "--output-tokens", "8"],
                         cwd=ROOT, stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL)
    tag = f"bench{b.pid}"
    try:
        deadline = time.time() + 240
        while time.time() < deadline and len(members(tag)) < 5:   # control plane, two sidecars, two executors
            assert b.poll() is None, "bench.py ended before its deployment was up"
            time.sleep(1)
        assert len(members(tag)) >= 5
        os.kill(b.pid, signal.SIGKILL)
        b.wait(timeout=30)
        deadline = time.time() + 30
        while time.time() < deadline and members(tag):
            time.sleep(0.5)
        assert members(tag) == []
    finally:
        if b.poll() is None:
            b.kill()


def test_serving_processes_do_not_inherit_the_launchers_variables(monkeypatch):
    """``torch.distributed.run`` exports its rendezvous and ``TORCHELASTIC_USE_AGENT_STORE`` to its ranks; servers that
    form their own process groups must not see them (rank 0 of such a group would wait for a store nobody hosts)."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_under_test", ROOT / "bench.py")
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    for k, v in {"RANK": "0", "WORLD_SIZE": "4", "LOCAL_RANK": "0", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29500",
                 "TORCHELASTIC_USE_AGENT_STORE": "True", "TORCHELASTIC_RUN_ID": "x", "OMP_NUM_THREADS": "1",
                 "CORNSERVE_KEEP_ME": "1"}.items():
        monkeypatch.setenv(k, v)
    env = bench.server_env(EXTRA="yes")
    assert env["EXTRA"] == "yes" and env["CORNSERVE_KEEP_ME"] == "1" and "PATH" in env
    assert not any(k in env for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS"))
    assert not any(k.startswith("TORCHELASTIC_") for k in env)


@pytest.mark.timeout(1200)
def test_bench_repeats_a_failed_tensor_parallel_layout_with_one_gpu_executors():
    """Four ranks: the TP 2 + TP 2 layout is made to fail after its deployment; the run is repeated as two one-GPU
    encoder executors and two one-GPU LLM executors, and the line names both layouts."""
    out = subprocess.run([sys.executable, "bench.py", "--small", "--cpu", "--gpus", "4", "--steps", "2", "--warmup", "1",
                          "--window-s", "3", "--rates", "2", "--offline-steps", "0", "--output-tokens", "8", "--slab-mib", "8",
                          "--fail-first-layout"], cwd=ROOT, capture_output=True, text=True, timeout=1100)
    assert out.returncode == 0, out.stderr[-3000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["config"]["parallelism"] == "eric tp1 x2 + llm tp1 x2"
    assert line["fallback_from"]["parallelism"] == "eric tp2 x1 + llm tp2 x1" and "made to fail" in line["fallback_from"]["reason"]
    assert sorted(e["executor"] for e in line["executors"]) == ["eric", "eric", "llm", "llm"]
    assert all(s["failed"] == 0 and s["completed"] == s["sent"] > 0 for s in line["sweep"])


@pytest.mark.timeout(1500)
def test_bench_under_the_launcher_with_four_ranks_prints_one_line():
    """``torch.distributed.run`` with four (gloo) ranks: rank 0 deploys the TP 2 + TP 2 layout, whose executors form their
    own process groups although the launcher's rendezvous variables are set around them; standard output carries the one
    result line and nothing else."""
    with socket.socket() as sock:
        sock.bind(("127.0.0.1", 0))
        port = sock.getsockname()[1]
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "4",
                          "--master-addr", "127.0.0.1", "--master-port", str(port), "bench.py", "--gpus", "4", "--cpu", "--small",
                          "--slab-mib", "8", "--steps", "2", "--warmup", "1", "--window-s", "3", "--offline-steps", "0",
                          "--rates", "2", "--output-tokens", "8", "--no-fallback"],
                         cwd=ROOT, capture_output=True, text=True, timeout=1400)
    assert out.returncode == 0, out.stderr[-3000:]
    lines = out.stdout.strip().splitlines()
    assert len(lines) == 1, lines[:5]
    line = json.loads(lines[0])
    assert line["n_gpus"] == 4 and line["config"]["parallelism"] == "eric tp2 x1 + llm tp2 x1" and "fallback_from" not in line
    assert all(s["failed"] == 0 and s["completed"] == s["sent"] > 0 for s in line["sweep"])
    assert sorted((e["executor"], e["tp_size"]) for e in line["executors"]) == [("eric", 2), ("llm", 2)]
