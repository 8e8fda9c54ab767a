#!/usr/bin/env python
"""Headline benchmark: Qwen2.5-VL-7B request throughput at a p99 latency bound, through the served stack.

What is measured (the reference's metric: benchmark/benchmark_cornserve.py:98-209 with the Poisson arrivals of
:399-435): requests arrive as a Poisson process at several rates; each has 1-4 uniform-random 1280x720 RGB images,
128 prompt tokens and 256 greedy output tokens (``ignore_eos``); the client records time to first token, time per
output token and end-to-end latency per request.  ``value`` is the highest request throughput among the swept rates
whose 99th-percentile end-to-end latency stays under ``config.slo_p99_e2el_s``.

What serves the requests (bf16, random-init weights of the real architecture, synthetic data): this repository's own
control plane on the N GPUs of the box - gateway -> task dispatcher -> Eric encoder executors -> sidecars (GPU slabs read
over NVLink) -> LLM executors - started with ``cornserve up`` as a user would, the MLLM app registered through the
gateway, the load sent to ``POST /app/invoke/{app}``.  Layout by N:

  1   one monolithic executor (vision tower inside the LLM executor)
  2   Eric TP=1  +  LLM TP=1
  4   Eric TP=2  +  LLM TP=2
  8   2 x Eric TP=2  +  2 x LLM TP=2

A *step* is ``--window-s`` seconds of arrivals; the K timed steps are split over the rates (lowest first), each rate's
requests are drained before the next rate starts, and the drains belong to the timed region
(``ms_per_step * steps`` = its length).  Every executor brackets each rate's span with CUDA events on its own GPU; the
span used for ``value`` is the maximum over executors.  ``e2e`` is the same requests timed by the client's clock, with
the bytes the executors copied from page-locked host memory to the GPUs (the images) and read back (the tokens).

  python bench.py --gpus N --steps K --warmup W            # N > 1: launched with torch.distributed.run
  python bench.py --impl reference --gpus N ...            # the reference arm: its Eric modules + stock vLLM

Rank 0 drives the deployment; the other ranks of the launcher join an NCCL group with it and wait.

Both arms get the same rates, request mix, bound, encoder batch limit (``--encoder-batch``) and a wall-clock budget
(``--deadline-s``): segments that no longer fit are dropped and the line says ``truncated``.  The serving processes are
started without the launcher's environment variables and leave with this process, also when it is killed.  If a
tensor-parallel layout (N = 4, 8) cannot serve, the run is repeated once with one-GPU executors on the same GPUs and the
line names both layouts (``fallback_from``).
"""

from __future__ import annotations

import argparse
import asyncio
import datetime
import json
import os
import signal
import socket
import statistics
import subprocess
import sys
import tempfile
import time
from dataclasses import asdict
from pathlib import Path

ROOT = Path(__file__).resolve().parent
T_START = time.monotonic()
METRIC = "requests_per_second_at_p99_e2el_slo"
MODEL = "Qwen/Qwen2.5-VL-7B-Instruct"
TINY = "cornserve-b200/tiny-vlm"

# N GPUs -> how the model is cut into executors (the N = 8 row is the layout the reference's benchmark names)
LAYOUTS = {
    1: {"backend": "V", "encoder_tp": 0, "llm_tp": 1, "replicas": 1, "name": "1 x monolithic executor (encoder inside the LLM executor)"},
    2: {"backend": "EV", "encoder_tp": 1, "llm_tp": 1, "replicas": 1, "name": "eric tp1 x1 + llm tp1 x1"},
    4: {"backend": "EV", "encoder_tp": 2, "llm_tp": 2, "replicas": 1, "name": "eric tp2 x1 + llm tp2 x1"},
    8: {"backend": "EV", "encoder_tp": 2, "llm_tp": 2, "replicas": 2, "name": "eric tp2 x2 + llm tp2 x2"},
}
# arrival rates (requests/s) swept at each N, the same for both arms: geometric ladders that start below what either
# arm sustains and end above what both do, so that each arm's best passing rate lies inside its ladder
RATES = {1: [3.0, 4.5, 6.5, 9.0, 12.0], 2: [4.0, 6.0, 9.0, 13.0, 18.0], 4: [6.0, 10.0, 16.0, 23.0, 30.0],
         8: [12.0, 20.0, 32.0, 46.0, 60.0]}


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--window-s", type=float, default=8.0, help="seconds of Poisson arrivals per step")
    ap.add_argument("--slo-s", type=float, default=10.0, help="bound on the p99 end-to-end latency (both arms)")
    ap.add_argument("--deadline-s", type=float, default=540.0,
                    help="wall-clock budget of warm-up + timed steps; segments that do not fit are dropped and the line says so")
    ap.add_argument("--no-fallback", action="store_true", help="do not repeat a failed tensor-parallel layout with one-GPU executors")
    ap.add_argument("--fail-first-layout", action="store_true", help=argparse.SUPPRESS)   # tests of the fallback path
    ap.add_argument("--slab-mib", type=int, default=0,
                    help="size of every sidecar's slab (0: 4096, or 64 with --small); a producer owns 1/N of its consumer's slab")
    ap.add_argument("--encoder-batch", type=int, default=8,
                    help="images per call of the encoder executor at most, for both arms (the reference benchmark's "
                         "eric_max_batch_size; waiting items are batched, nothing waits for a batch to fill)")
    ap.add_argument("--rates", default="", help="comma-separated requests/s (default: the table for N)")
    ap.add_argument("--output-tokens", type=int, default=256)
    ap.add_argument("--prompt-tokens", type=int, default=128)
    ap.add_argument("--offline-steps", type=int, default=2, help="closed-batch steps of the in-process pipeline, reported as offline_batch_req_s (0 = skip)")
    ap.add_argument("--small", action="store_true", help="tiny model and images: a smoke run, not a valid number")
    ap.add_argument("--cpu", action="store_true", help="with --small: run the deployment on CPU ranks")
    ap.add_argument("--keep-logs", default="", help="directory to keep the deployment's logs in")
    return ap.parse_args()


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return int(s.getsockname()[1])


class ClockSampler:
    """Samples SM clocks and throttle reasons of the GPUs in use with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, n_gpus: int = 1) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        rows, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9 or not p[0].isdigit() or int(p[0]) >= n_gpus:
                    continue
                rows.append((float(p[1]), float(p[3]) if p[3].replace(".", "").isdigit() else 0.0))
                mx.append(float(p[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        # under load = samples drawing more than idle power (an open-loop serving run leaves gaps between bursts)
        busy = [c for c, w in rows if w > 300.0] or [c for c, _ in rows]
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(rows), "samples_under_load": len(busy), "reasons": sorted(reasons)}


# ----------------------------------------------------------------------------------------------------------------------
# the deployment under test (this repository's arm)
# ----------------------------------------------------------------------------------------------------------------------
def wait_http(url: str, proc: subprocess.Popen, timeout_s: float, what: str) -> None:
    import urllib.error
    import urllib.request

    deadline = time.time() + timeout_s
    while time.time() < deadline:
        if proc.poll() is not None:
            raise RuntimeError(f"{what} exited with code {proc.returncode}")
        try:
            with urllib.request.urlopen(url, timeout=2) as r:
                if r.status == 200:
                    return
        except urllib.error.HTTPError as e:
            if e.code == 500:   # the service says that it cannot become healthy (a worker of it died)
                raise RuntimeError(f"{what} reports a failure: {e.read().decode(errors='replace')[:300]}") from None
            time.sleep(0.5)
        except Exception:  # noqa: BLE001
            time.sleep(0.5)
    raise TimeoutError(f"{what} did not answer {url} within {timeout_s:.0f} s")


def stop_group(proc: subprocess.Popen, grace_s: float = 30.0) -> None:
    """SIGTERM to the process group this script started, then SIGKILL if it lingers."""
    try:
        if proc.poll() is None:
            os.killpg(proc.pid, signal.SIGTERM)
            proc.wait(timeout=grace_s)
    except Exception:  # noqa: BLE001
        pass
    try:
        os.killpg(proc.pid, signal.SIGKILL)   # members of the group that outlived its leader (no-op when there are none)
    except Exception:  # noqa: BLE001
        pass


def profiles_for(model: str, layout: dict, small: bool, encoder_batch: int = 1) -> list[dict]:
    """Deployment profiles: the executor size (= tensor-parallel degree) of each unit task and its launch arguments."""
    llm_args = ["--max-num-seqs", "256", "--decode-burst", "8", "--max-model-len", "8192" if not small else "2048"]
    if small:
        llm_args += ["--num-kv-pages", "64", "--max-num-batched-tokens", "512"]
    out = [{"task": {"__class__": "LLMUnitTask", "model_id": model, "receive_embeddings": layout["backend"] == "EV",
                     "execution_descriptor_name": None},
            "num_gpus_to_profile": {str(layout["llm_tp"]): {"launch_args": llm_args}}}]
    if layout["backend"] == "EV":
        out.append({"task": {"__class__": "EncoderTask", "modality": "image", "model_ids": [model], "max_batch_size": 1,
                             "execution_descriptor_name": None},
                    "num_gpus_to_profile": {str(layout["encoder_tp"]): {
                        "launch_args": ["--server.max-batch-size", str(max(1, encoder_batch))]}}})
    return out


async def deploy_ours(gateway: str, model: str, layout: dict, small: bool, encoder_batch: int = 1) -> tuple[str, list[dict]]:
    import aiohttp

    from benchmark.experiment import ExperimentConfig, app_source, part_of

    parts = {"llm": 1} if layout["backend"] == "V" else {"encoder": 1, "llm": 1}
    cfg = ExperimentConfig(layout["backend"], model, parts)
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=1800)) as http:
        async with http.post(f"{gateway}/deploy-profiles", json={"profiles": profiles_for(model, layout, small, encoder_batch)}) as r:
            if r.status != 200:
                raise RuntimeError(f"deploying profiles failed: {await r.text()}")
        async with http.post(f"{gateway}/app/register", json={"source_code": app_source(cfg)}) as resp:
            events = [json.loads(line.decode()[6:]) async for line in resp.content if line.startswith(b"data: ")]
        if not events or events[-1]["event"]["type"] != "final":
            raise RuntimeError(f"registration failed: {events[-1] if events else 'no events'}")
        app_id = events[0]["event"]["app_id"]
        if layout["replicas"] > 1:
            async with http.get(f"{gateway}/tasks/list") as resp:
                tasks = await resp.json()
            for task_json, task_id, _ in tasks:
                tp = layout["encoder_tp"] if part_of(task_json) == "encoder" else layout["llm_tp"]
                extra = tp * (layout["replicas"] - 1)
                async with http.post(f"{gateway}/task/scale", json={"task_id": task_id, "num_gpus": extra}) as resp:
                    if resp.status != 200:
                        raise RuntimeError(f"scaling {task_id} by {extra} GPUs failed: {await resp.text()}")
        async with http.get(f"{gateway}/cluster/executors") as resp:
            executors = await resp.json()
    return app_id, executors


class ExecutorProbe:
    """Counters and device-side marks of every executor of a deployment, over their HTTP APIs."""

    def __init__(self, urls: list[str]):
        self.urls = urls
        self.marks: dict[tuple[str, int], list[int]] = {}

    async def _all(self, method: str, path: str) -> list[dict]:
        import aiohttp

        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=60)) as http:
            async def one(u):
                async with http.request(method, u + path) as r:
                    return await r.json()
            return list(await asyncio.gather(*(one(u) for u in self.urls)))

    async def stats(self) -> list[dict]:
        return await self._all("GET", "/stats")

    async def hook(self, phase: str, segment: int) -> None:
        got = await self._all("POST", "/timer/mark")
        self.marks[(phase, segment)] = [g["mark"] for g in got]

    async def device_ms(self, segment: int) -> float:
        import aiohttp

        a, b = self.marks[("begin", segment)], self.marks[("end", segment)]
        async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=60)) as http:
            async def one(u, s, e):
                async with http.get(f"{u}/timer/elapsed", params={"start": s, "end": e}) as r:
                    return float((await r.json())["ms"])
            return max(await asyncio.gather(*(one(u, s, e) for u, s, e in zip(self.urls, a, b))))


def request_payload(i: int, small: bool, prompt_tokens: int, output_tokens: int) -> dict:
    """Request ``i`` of the mix: 1-4 images (mean 2.5), a prompt that renders to ``prompt_tokens`` text tokens with the
    byte-level tokenizer (19 of them are the chat template's), ``output_tokens`` greedy tokens."""
    import random

    hw = "224x224" if small else "720x1280"
    rng = random.Random(i)
    text = "".join(rng.choice("abcdefghijklmnopqrstuvwxyz ") for _ in range(max(1, prompt_tokens - 19)))
    media = [["image", f"synthetic:{hw}:{i * 16 + k}"] for k in range(1 + i % 4)]
    return {"prompt": text, "multimodal_data": media, "max_completion_tokens": output_tokens}


def server_env(**extra: str) -> dict[str, str]:
    """The environment of the serving processes of either arm: this process's, without what a ``torch.distributed.run``
    launcher added for its own ranks.  The servers form their own process groups; with the launcher's variables still set
    (its rendezvous address, ``TORCHELASTIC_USE_AGENT_STORE``: "the agent hosts the store, connect as a client") rank 0 of
    such a group would wait for a store that nobody hosts, and ``OMP_NUM_THREADS=1`` would pin their host-side work to one
    thread."""
    drop = {"RANK", "LOCAL_RANK", "WORLD_SIZE", "LOCAL_WORLD_SIZE", "GROUP_RANK", "GROUP_WORLD_SIZE", "ROLE_RANK",
            "ROLE_WORLD_SIZE", "ROLE_NAME", "MASTER_ADDR", "MASTER_PORT", "OMP_NUM_THREADS", "NCCL_ASYNC_ERROR_HANDLING",
            "TORCH_NCCL_ASYNC_ERROR_HANDLING"}
    env = {k: v for k, v in os.environ.items() if k not in drop and not k.startswith("TORCHELASTIC_")}
    env.update(extra)
    return env


def diff_stats(before: list[dict], after: list[dict]) -> dict:
    out = {"gpu_launches": 0, "paths": {}, "h2d_bytes": 0, "d2h_bytes": 0, "executors": []}
    for b, a in zip(before, after):
        tp = max(1, int(a.get("tp_size", 1)))
        launches = (a["kernel_launches"] - b["kernel_launches"]) * tp   # every rank of a TP group launches the same kernels
        out["gpu_launches"] += launches
        for k, v in a.get("paths", {}).items():
            d = (v - b.get("paths", {}).get(k, 0)) * tp
            if d:
                out["paths"][k] = out["paths"].get(k, 0) + d
        out["h2d_bytes"] += a.get("h2d_bytes", 0) - b.get("h2d_bytes", 0)
        out["d2h_bytes"] += a.get("d2h_bytes", 0) - b.get("d2h_bytes", 0)
        e = {"executor": a.get("executor"), "tp_size": tp, "gpu_launches": launches}
        for k in ("prefill_steps", "decode_bursts", "prefill_ms", "decode_ms", "decode_host_ms", "prefill_tokens",
                  "decode_tokens", "batches", "items", "busy_ms", "broadcast_ms", "tp_publish_ms", "requests", "inputs_ms",
                  "first_token_ms", "local_encoder_images", "local_encoder_batches", "local_encoder_ms", "local_encoder_host_ms",
                  "local_encoder_wait_ms", "alloc_retries", "device_allocs"):
            if k in a:
                e[k] = round(a[k] - b.get(k, 0), 1)
        if e.get("requests") and "inputs_ms" in e:
            e["ms_per_request_waiting_for_inputs"] = round(e["inputs_ms"] / e["requests"], 1)
            e["ms_per_request_queue_and_prefill"] = round(e["first_token_ms"] / e["requests"], 1)
        if e.get("decode_bursts"):
            e["host_ms_per_decode_burst"] = round(e["decode_host_ms"] / e["decode_bursts"], 3)
            e["ms_per_decode_burst"] = round(e["decode_ms"] / e["decode_bursts"], 3)
        if a.get("stack_samples"):
            e["stack_samples"] = a["stack_samples"]
        if e.get("batches"):
            e["ms_per_encoder_batch"] = round(e["busy_ms"] / e["batches"], 3)
            e["broadcast_ms_per_encoder_batch"] = round(e.get("broadcast_ms", 0.0) / e["batches"], 3)
        out["executors"].append(e)
    return out


def sweep_config(args: argparse.Namespace, world: int):
    from benchmark.serving_sweep import SweepConfig

    rates = [float(x) for x in args.rates.split(",") if x] or RATES[max(k for k in RATES if k <= world)]
    deadline = args.deadline_s if args.deadline_s > 0 else None
    if deadline is not None and args.impl == "reference":
        deadline = min(deadline, 480.0)   # its servers may take five minutes to start; both fit the time a run is given
    return SweepConfig(rates=rates, steps=args.steps, warmup=args.warmup, window_s=args.window_s, slo_e2el_s=args.slo_s,
                       output_tokens=args.output_tokens, deadline_s=deadline)


# If the tensor-parallel layout of an N cannot serve (its deployment does not come up, or every warm-up request fails),
# the run is repeated once with one-GPU executors on the same GPUs, and the line says so (`fallback_from`).
FALLBACKS = {
    4: {"backend": "EV", "encoder_tp": 1, "llm_tp": 1, "replicas": 2, "name": "eric tp1 x2 + llm tp1 x2"},
    8: {"backend": "EV", "encoder_tp": 1, "llm_tp": 1, "replicas": 4, "name": "eric tp1 x4 + llm tp1 x4"},
}


def run_ours(args: argparse.Namespace, world: int) -> dict:
    key = max(k for k in LAYOUTS if k <= world)
    try:
        return run_ours_layout(args, world, LAYOUTS[key], "")
    except Exception as e:  # noqa: BLE001
        fallback = FALLBACKS.get(key)
        left = 800.0 - (time.monotonic() - T_START)
        if fallback is None or args.no_fallback or left < 330.0:
            raise
        sys.stderr.write(f"--- layout '{LAYOUTS[key]['name']}' failed ({type(e).__name__}: {str(e)[:300]}); "
                         f"one more run as '{fallback['name']}' with {left:.0f} s left ---\n")
        args.deadline_s = min(args.deadline_s if args.deadline_s > 0 else left, left - 130.0)
        args.offline_steps = 0
        line = run_ours_layout(args, world, fallback, "-fallback")
        line["fallback_from"] = {"parallelism": LAYOUTS[key]["name"], "reason": f"{type(e).__name__}: {e}"[:400]}
        return line


def run_ours_layout(args: argparse.Namespace, world: int, layout: dict, tag: str) -> dict:
    from benchmark.serving_sweep import best_segment, run_sweep

    model = TINY if args.small else MODEL
    tmp = Path((args.keep_logs + tag) if args.keep_logs else tempfile.mkdtemp(prefix="cornserve-bench-")).resolve()
    (tmp / "logs").mkdir(parents=True, exist_ok=True)
    port = free_port()
    env = server_env(CORNSERVE_LOG_DIR=str(tmp / "logs"), CORNSERVE_STORE_PATH=str(tmp / "store.sqlite"),
               CORNSERVE_LOG_LEVEL=os.environ.get("CORNSERVE_LOG_LEVEL", "WARNING"), OTEL_SDK_DISABLED="true",
               CORNSERVE_EXIT_WITH_PARENT="1",
               SIDECAR_SHM_SIZE=str((args.slab_mib << 20) if args.slab_mib > 0 else ((64 << 20) if args.small else (4 << 30))), CORNSERVE_ALLOW_RANDOM_INIT="1",
               CORNSERVE_SIDECAR_BASE_PORT=str(free_port()), SIDECAR_NAMESPACE=f"bench{os.getpid()}{tag}",
               PYTHONPATH=str(ROOT) + os.pathsep + os.environ.get("PYTHONPATH", ""))
    if args.cpu:
        env.update(CORNSERVE_DEVICE="cpu", SIDECAR_DEVICE="cpu")
    cmd = [sys.executable, "-m", "cornserve.cli.main", "up", "--num-gpus", str(world), "--port", str(port)]
    if args.cpu:
        cmd.append("--cpu")
    log = open(tmp / "cluster.log", "w")
    cluster = subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    gateway = f"http://127.0.0.1:{port}"
    sampler = ClockSampler()
    try:
        wait_http(f"{gateway}/health", cluster, 240, "the control plane")
        t0 = time.time()
        app_id, executors = asyncio.run(deploy_ours(gateway, model, layout, args.small, args.encoder_batch))
        deploy_s = time.time() - t0
        if args.fail_first_layout and not tag:
            raise RuntimeError("the first layout was made to fail (--fail-first-layout)")
        probe = ExecutorProbe([e["url"] for e in executors])
        cfg = sweep_config(args, world)
        payload_of = lambda i: request_payload(i, args.small, args.prompt_tokens, args.output_tokens)  # noqa: E731

        async def measure():
            # warm-up happens inside run_sweep; counters are read around the timed steps only
            state = {}

            async def hook(phase, seg):
                if phase == "begin" and seg == 0:
                    state["before"] = await probe.stats()
                    sampler.start()
                await probe.hook(phase, seg)

            res = await run_sweep(f"{gateway}/app/invoke/{app_id}", payload_of, cfg, hook)
            state["after"] = await probe.stats()
            for i, seg in enumerate(res["segments"]):
                seg.device_ms = await probe.device_ms(i)
            return res, state

        res, state = asyncio.run(measure())
        clocks = sampler.stop(world)
        counters = diff_stats(state.get("before", state["after"]), state["after"])
    except Exception:
        sys.stderr.write(f"--- deployment logs under {tmp} ---\n")
        for p in sorted((tmp / "logs").glob("*.log")) + [tmp / "cluster.log"]:
            try:
                sys.stderr.write(f"== {p.name}\n" + "\n".join(p.read_text(errors="replace").splitlines()[-40:]) + "\n")
            except OSError:
                pass
        raise
    finally:
        stop_group(cluster)
        log.close()

    segs = res["segments"]
    best = best_segment(segs)
    timed_s = res["timed_s"]
    value = best.completed / (best.device_ms / 1e3) if best else 0.0
    n_req = sum(s.sent for s in segs)
    line = {
        "metric": METRIC, "value": value, "unit": "req/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": timed_s * 1e3 / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if not args.cpu else "fp32",
        "data": "synthetic (uniform-random images, random prompt bytes, random-init weights)",
        "config": {
            "model": "Qwen2.5-VL-7B" if not args.small else "tiny-smoke", "parallelism": layout["name"],
            "global_batch": "open loop: Poisson arrivals at rates_req_s, requests in flight vary",
            "seq_len": int(2.5 * (1196 + 2) + args.prompt_tokens) + args.output_tokens if not args.small else None,
            "images_per_request": "1-4 (mean 2.5) of 1280x720" if not args.small else "1-4 of 224x224",
            "prompt_tokens": args.prompt_tokens, "output_tokens": args.output_tokens, "rates_req_s": sorted(cfg.rates),
            "window_s": cfg.window_s, "slo_p99_e2el_s": cfg.slo_e2el_s, "encoder_max_batch": args.encoder_batch,
            "serving_path": "client -> gateway -> task dispatcher -> Eric -> sidecar -> LLM executor (HTTP + gRPC, local processes)",
            "l2_policy": "inputs larger than L2: every decode step streams the 15 GB of decoder weights plus the KV cache",
            "timing": "value = requests of the best rate / that rate's span between CUDA events (max over executors); e2e = client clock",
        },
        "clocks": clocks,
        "e2e": {"value": best.request_throughput if best else 0.0, "unit": "req/s",
                "h2d_bytes_per_step": counters["h2d_bytes"] // args.steps, "d2h_bytes_per_step": counters["d2h_bytes"] // args.steps,
                "api": "HTTP POST {gateway}/app/invoke/{app_id} (app registered from source through /app/register)",
                "whole_sweep_req_s": n_req / timed_s},
        "gpu_launches": counters["gpu_launches"], "fused_path_launches": counters["paths"],
        "steps_run": res.get("steps_run", args.steps), "truncated": bool(res.get("truncated", False)),
        "best_rate_req_s": best.rate if best else None,
        "latency_at_best_rate_ms": {"ttft": best.ttft_ms, "tpot": best.tpot_ms, "e2el": best.e2el_ms} if best else None,
        "sweep": [asdict(s) for s in segs], "executors": counters["executors"], "deploy_s": round(deploy_s, 1),
        "output_tokens_per_second": best.output_token_throughput if best else 0.0,
    }
    if args.offline_steps > 0 and not args.cpu and time.monotonic() - T_START > 620:
        line["offline_batch_req_s"] = {"skipped": "the served sweep used up the time of this run"}
    elif args.offline_steps > 0 and not args.cpu:
        try:
            line["offline_batch_req_s"] = offline_batch(args)
        except Exception as e:  # noqa: BLE001  (an extra: it must not cost the headline)
            line["offline_batch_req_s"] = {"error": f"{type(e).__name__}: {e}"}
    return line


def offline_batch(args: argparse.Namespace) -> dict:
    """Closed-batch throughput of the in-process pipeline on one GPU (no arrival process, no latency bound): 128
    requests of the same mix run to completion per step through ``MLLMPipeline.generate``.  Extra figure, 1 GPU."""
    import numpy as np
    import torch

    from cornserve import ops
    from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer
    from cornserve.models.qwen_llm import LLMConfig, QwenLLM
    from cornserve.pipelines import MLLMPipeline, MLLMRequest
    from cornserve.task_executors.llm.engine import EngineConfig

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    R, out_tok, prompt_tok = (128, args.output_tokens, args.prompt_tokens) if not args.small else (8, 8, 32)
    if args.small:
        vcfg = Qwen25VisionConfig(depth=2, hidden_size=256, num_heads=4, intermediate_size=512, out_hidden_size=512, fullatt_block_indexes=[1])
        lcfg = LLMConfig(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                         intermediate_size=1024, vocab_size=152064)
        img_hw, tokens_per_img = (224, 224), 64
    else:
        vcfg, lcfg, img_hw, tokens_per_img = Qwen25VisionConfig(), LLMConfig(), (720, 1280), 1196
    torch.manual_seed(1234)
    pages = R * (-(-(4 * (tokens_per_img + 2) + prompt_tok + out_tok + 2) // 128) + 1) + 8
    pipe = MLLMPipeline(Qwen25VisionTransformer(vcfg, device=dev), QwenLLM(lcfg, device=dev),
                        EngineConfig(num_pages=pages, max_batched_tokens=18944, max_num_seqs=R, decode_burst=16, max_model_len=8192),
                        max_patches_per_encode=34000)
    rng = np.random.default_rng(0)
    imgs = [[torch.from_numpy(rng.integers(0, 256, (*img_hw, 3), dtype=np.uint8)).pin_memory() for _ in range(1 + i % 4)] for i in range(R)]
    prompts = [rng.integers(1000, 100000, prompt_tok).astype(np.int32) for _ in range(R)]

    def step(tag):
        res = pipe.generate([MLLMRequest(f"{tag}-{i}", prompts[i], imgs[i], max_tokens=out_tok, ignore_eos=True) for i in range(R)])
        assert all(len(v) == out_tok for v in res.values())

    for w in range(3):
        step(f"w{w}")
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for s in range(args.offline_steps):
        step(f"t{s}")
    e1.record()
    torch.cuda.synchronize()
    ops.check_error("offline batch")
    ms = e0.elapsed_time(e1)
    return {"value": R * args.offline_steps / (ms / 1e3), "unit": "req/s", "n_gpus": 1, "requests_per_step": R,
            "steps": args.offline_steps, "warmup": 3, "ms_per_step": ms / args.offline_steps,
            "api": "cornserve.pipelines.MLLMPipeline.generate (images copied from pinned host memory every step)"}


# ----------------------------------------------------------------------------------------------------------------------
# the reference arm
# ----------------------------------------------------------------------------------------------------------------------
def run_reference(args: argparse.Namespace, world: int) -> dict:
    """The reference's own encoder modules (``baseline/_ref``, unmodified) feeding stock vLLM started with the flags
    the reference's descriptor passes, in a server process that never imports this repository's package; the same
    sweep, the same request mix, the same bound."""
    from benchmark.serving_sweep import best_segment, run_sweep

    ref_root = ROOT / "baseline" / "_ref"
    server = ROOT / "baseline" / "reference_server.py"
    if not (ref_root / "cornserve").is_dir():
        return {"impl": "reference", "unavailable": "the reference package is not installed under baseline/_ref"}
    layout = LAYOUTS[max(k for k in LAYOUTS if k <= world)]
    tmp = Path(args.keep_logs or tempfile.mkdtemp(prefix="cornserve-refbench-")).resolve()
    tmp.mkdir(parents=True, exist_ok=True)
    port = free_port()
    # the server's import path holds the reference package and never this repository (both packages are called cornserve)
    keep = [p for p in os.environ.get("PYTHONPATH", "").split(os.pathsep) if p and Path(p).resolve() != ROOT]
    env = server_env(PYTHONPATH=os.pathsep.join([str(ref_root), *keep]), OTEL_SDK_DISABLED="true", REF_EXIT_WITH_PARENT="1",
               VLLM_LOGGING_LEVEL=os.environ.get("VLLM_LOGGING_LEVEL", "WARNING"), HF_HUB_OFFLINE="1", TRANSFORMERS_OFFLINE="1")
    cmd = [sys.executable, "-P", str(server), "--port", str(port), "--gpus", str(world), "--encoder-tp", str(max(1, layout["encoder_tp"])),
           "--llm-tp", str(layout["llm_tp"]), "--replicas", str(layout["replicas"]), "--workdir", str(tmp),
           "--max-tokens", str(args.output_tokens), "--prompt-tokens", str(args.prompt_tokens),
           "--encoder-batch", str(args.encoder_batch)]
    if layout["backend"] == "V":
        cmd.append("--share-gpu")
    if args.small:
        cmd.append("--small")
    log = open(tmp / "reference_server.log", "w")
    proc = subprocess.Popen(cmd, env=env, cwd=tmp, stdout=log, stderr=subprocess.STDOUT, start_new_session=True)
    base = f"http://127.0.0.1:{port}"
    sampler = ClockSampler()

    def tail() -> str:
        out = []
        for p in [tmp / "reference_server.log", *sorted(tmp.glob("llm_*.log")), *sorted(tmp.glob("encoder_*.log"))]:
            try:
                lines = [ln for ln in p.read_text(errors="replace").splitlines() if ln.strip()]
                out.append(f"{p.name}: " + " | ".join(lines[-4:])[-400:])
            except OSError:
                pass
        return " || ".join(out)[-1500:]

    try:
        try:
            wait_http(f"{base}/health", proc, float(os.environ.get("REF_START_WAIT_S", "330")), "the reference server")
        except Exception as e:  # noqa: BLE001
            return {"impl": "reference", "unavailable": f"the reference arm did not start: {e}; log tail: {tail()}"}
        probe = ExecutorProbe([base])
        cfg = sweep_config(args, world)
        payload_of = lambda i: request_payload(i, args.small, args.prompt_tokens, args.output_tokens)  # noqa: E731

        async def measure():
            state = {}

            async def hook(phase, seg):
                if phase == "begin" and seg == 0:
                    state["before"] = await probe.stats()
                    sampler.start()
                await probe.hook(phase, seg)

            res = await run_sweep(f"{base}/app/invoke/reference", payload_of, cfg, hook)
            state["after"] = await probe.stats()
            for i, seg in enumerate(res["segments"]):
                seg.device_ms = await probe.device_ms(i)
            return res, state

        try:
            res, state = asyncio.run(measure())
        except Exception as e:  # noqa: BLE001
            return {"impl": "reference", "unavailable": f"the reference arm failed under load: {type(e).__name__}: {e}; log tail: {tail()}"}
        clocks = sampler.stop(world)
    finally:
        stop_group(proc)
        log.close()
    segs = res["segments"]
    best = best_segment(segs)
    b, a = state.get("before", state["after"])[0], state["after"][0]
    return {
        "impl": "reference", "steps_run": res.get("steps_run", args.steps), "truncated": bool(res.get("truncated", False)),
        "metric": METRIC, "value": best.completed / (best.device_ms / 1e3) if best else 0.0, "unit": "req/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["timed_s"] * 1e3 / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic (uniform-random images, random prompt tokens, random-init weights)",
        "config": {"model": "Qwen2.5-VL-7B" if not args.small else "tiny-smoke",
                   "parallelism": layout["name"].replace("monolithic executor (encoder inside the LLM executor)", "reference encoder + vLLM sharing the GPU"),
                   "images_per_request": "1-4 (mean 2.5) of 1280x720", "prompt_tokens": args.prompt_tokens,
                   "output_tokens": args.output_tokens, "rates_req_s": sorted(cfg.rates), "window_s": cfg.window_s,
                   "slo_p99_e2el_s": cfg.slo_e2el_s, "encoder_max_batch": args.encoder_batch,
                   "reference_class": a.get("reference_class", "cornserve.task_executors.eric Qwen2_5_VisionTransformer + its ModalityProcessor -> pinned shared memory -> stock vLLM (prompt embeddings)"),
                   "vllm_flags": a.get("vllm_flags")},
        "clocks": clocks,
        "e2e": {"value": best.request_throughput if best else 0.0, "unit": "req/s",
                "h2d_bytes_per_step": (a.get("h2d_bytes", 0) - b.get("h2d_bytes", 0)) // args.steps,
                "d2h_bytes_per_step": (a.get("d2h_bytes", 0) - b.get("d2h_bytes", 0)) // args.steps,
                "api": "HTTP POST to the reference arm's front process (the reference's own gateway needs Kubernetes)",
                "whole_sweep_req_s": sum(s.sent for s in segs) / res["timed_s"]},
        "steps_run": res.get("steps_run", args.steps), "truncated": bool(res.get("truncated", False)),
        "best_rate_req_s": best.rate if best else None,
        "latency_at_best_rate_ms": {"ttft": best.ttft_ms, "tpot": best.tpot_ms, "e2el": best.e2el_ms} if best else None,
        "sweep": [asdict(s) for s in segs],
    }


def _raise_on_signal(signum, _frame) -> None:
    raise SystemExit(f"signal {signum}")


def main() -> None:
    args = parse_args()
    # a launcher that gives up sends SIGTERM: unwind (the deployment is stopped in `finally` blocks) instead of dying on the spot
    for sig in (signal.SIGTERM, signal.SIGHUP):
        signal.signal(sig, _raise_on_signal)
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    sys.path.insert(0, str(ROOT))
    # Standard output carries the one result line and nothing else: libraries that write there (NCCL's version banner at
    # the first collective, for one) are pointed at standard error for the life of the process.
    sys.stdout.flush()
    result_out = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if args.cpu or not torch.cuda.is_available():
            dist.init_process_group("gloo", timeout=datetime.timedelta(hours=2))
        else:
            # the launcher's ranks meet once over NCCL (one rank per GPU); after that the GPUs belong to the executors
            # the control plane starts, and the ranks wait for rank 0 on the host (gloo), not in a GPU kernel
            torch.cuda.set_device(local_rank)
            dist.init_process_group("cpu:gloo,cuda:nccl", timeout=datetime.timedelta(hours=2),
                                    device_id=torch.device("cuda", local_rank))
            t = torch.ones(1, device="cuda")
            dist.all_reduce(t)
            torch.cuda.synchronize()
            assert int(t.item()) == world
            del t
            torch.cuda.empty_cache()
        gate = torch.zeros(1)
        dist.all_reduce(gate)   # host-side barrier before the deployment starts
    n = world if world > 1 else args.gpus   # a plain launch may still name several GPUs: rank 0 drives them all
    failure: BaseException | None = None
    if rank == 0:
        try:
            if not args.cpu and args.impl == "ours":
                import torch

                if not torch.cuda.is_available():
                    raise SystemExit("bench.py needs a CUDA device (use --small --cpu for a plumbing run)")
                if torch.cuda.device_count() < n:
                    raise SystemExit(f"{n} GPUs asked for, {torch.cuda.device_count()} visible")
            try:
                line = run_ours(args, n) if args.impl == "ours" else run_reference(args, n)
            except Exception as e:  # noqa: BLE001
                if args.impl != "reference":
                    raise
                line = {"impl": "reference", "unavailable": f"{type(e).__name__}: {e}"[:600]}
            print(json.dumps(line, default=str), file=result_out, flush=True)
        except BaseException as e:  # noqa: BLE001  (the other ranks are released first, then it is raised again)
            failure = e
    if dist is not None:
        import torch

        done = torch.zeros(1)
        dist.all_reduce(done)   # the other ranks wait here, on the host, while rank 0 runs the benchmark
        dist.destroy_process_group()
    if failure is not None:
        raise failure


if __name__ == "__main__":
    main()
