"""Open-loop serving benchmark against a registered app (reference harness: benchmark/benchmark_cornserve.py:66-619).

Requests are released on an arrival schedule that does not depend on completions (Poisson, Gamma with a burstiness
factor, or a duty cycle of bursts), each request is an HTTP invocation of an app that streams OpenAI-style chunks, and
for every request the client records when the first and every later chunk arrived.  From those timestamps:

  TTFT  time to first token     first chunk - send time
  ITL   inter-token latencies   gaps between consecutive chunks
  TPOT  time per output token   (last chunk - first chunk) / (chunks - 1)
  E2EL  end-to-end latency      last chunk - send time

and per run: request throughput, output-token throughput, mean / median / p90 / p95 / p99 of each metric.

    python -m benchmark.load_generator --app mllm --rate 10 --num-prompts 200 --image 1280x720 --input-len 128 --output-len 256
"""

from __future__ import annotations

import argparse
import asyncio
import json
import random
import time
from dataclasses import asdict, dataclass, field

import aiohttp
import numpy as np


@dataclass
class RequestRecord:
    send_time: float
    chunk_times: list[float] = field(default_factory=list)
    output_tokens: int = 0
    ok: bool = False
    error: str = ""

    @property
    def ttft(self) -> float:
        return self.chunk_times[0] - self.send_time

    @property
    def e2el(self) -> float:
        return self.chunk_times[-1] - self.send_time

    @property
    def itl(self) -> list[float]:
        return list(np.diff(self.chunk_times)) if len(self.chunk_times) > 1 else []

    @property
    def tpot(self) -> float | None:
        n = len(self.chunk_times)
        return (self.chunk_times[-1] - self.chunk_times[0]) / (n - 1) if n > 1 else None


def arrival_times(n: int, rate: float, burstiness: float = 1.0, seed: int = 0) -> np.ndarray:
    """Send offsets (seconds) of ``n`` requests at ``rate`` requests/s.  Inter-arrival gaps are Gamma distributed with
    shape ``burstiness`` (1 = Poisson process, < 1 burstier, > 1 more regular); ``rate = inf`` sends everything at once."""
    if not np.isfinite(rate):
        return np.zeros(n)
    rng = np.random.default_rng(seed)
    gaps = rng.gamma(shape=burstiness, scale=1.0 / (rate * burstiness), size=n)
    gaps[0] = 0.0
    return np.cumsum(gaps)


def duty_cycle_times(n: int, rate_on: float, on_s: float, off_s: float, seed: int = 0) -> np.ndarray:
    """Poisson arrivals at ``rate_on`` during ``on_s``-second windows separated by ``off_s`` seconds of silence."""
    t = arrival_times(n, rate_on, 1.0, seed)
    return t + np.floor(t / on_s) * off_s


def percentiles(values: list[float]) -> dict[str, float]:
    if not values:
        return {k: float("nan") for k in ("mean", "median", "p90", "p95", "p99")}
    a = np.asarray(values, dtype=np.float64)
    return {"mean": float(a.mean()), "median": float(np.median(a)), "p90": float(np.percentile(a, 90)),
            "p95": float(np.percentile(a, 95)), "p99": float(np.percentile(a, 99))}


@dataclass
class Summary:
    completed: int
    failed: int
    duration_s: float
    request_throughput: float
    output_token_throughput: float
    ttft_ms: dict[str, float]
    tpot_ms: dict[str, float]
    itl_ms: dict[str, float]
    e2el_ms: dict[str, float]


def summarise(records: list[RequestRecord], duration_s: float) -> Summary:
    good = [r for r in records if r.ok and r.chunk_times]
    ms = lambda xs: percentiles([x * 1e3 for x in xs])  # noqa: E731
    return Summary(
        completed=len(good), failed=len(records) - len(good), duration_s=duration_s,
        request_throughput=len(good) / duration_s if duration_s > 0 else 0.0,
        output_token_throughput=sum(r.output_tokens for r in good) / duration_s if duration_s > 0 else 0.0,
        ttft_ms=ms([r.ttft for r in good]), tpot_ms=ms([r.tpot for r in good if r.tpot is not None]),
        itl_ms=ms([g for r in good for g in r.itl]), e2el_ms=ms([r.e2el for r in good]))


def synthetic_prompt(length: int, rng: random.Random) -> str:
    """About ``length`` tokens of filler text (common English words are one token each in most vocabularies)."""
    words = ("the", "of", "and", "to", "in", "is", "that", "for", "it", "as", "with", "was", "on", "be", "at", "by")
    return " ".join(rng.choice(words) for _ in range(max(1, length)))


def build_request(i: int, args: argparse.Namespace, rng: random.Random) -> dict:
    h, w = (int(v) for v in args.image.split("x")[::-1]) if args.image else (0, 0)
    media = [["image", f"synthetic:{h}x{w}:{i * 16 + k}"] for k in range(args.images_per_request)] if args.image else []
    return {"prompt": synthetic_prompt(args.input_len, rng), "multimodal_data": media, "max_completion_tokens": args.output_len}


async def one_request(http: aiohttp.ClientSession, url: str, payload: dict, rec: RequestRecord) -> None:
    rec.send_time = time.perf_counter()
    try:
        async with http.post(url, json={"request_data": payload}) as resp:
            if resp.status != 200:
                rec.error = f"{resp.status}: {(await resp.text())[:200]}"
                return
            async for line in resp.content:
                if not line.strip():
                    continue
                now = time.perf_counter()
                chunk = json.loads(line)
                if isinstance(chunk, dict) and set(chunk) == {"error"}:
                    rec.error = str(chunk["error"])
                    return
                choices = chunk.get("choices") if isinstance(chunk, dict) else None
                if choices:
                    # every streamed chunk is an arrival; it counts as a token when it carries text or audio (a
                    # chunk may be empty, e.g. while the bytes of a multi-byte character are still incomplete)
                    delta = choices[0].get("delta") or {}
                    rec.chunk_times.append(now)
                    rec.output_tokens += 1 if (delta.get("content") or delta.get("audio")) else 0
                elif not (isinstance(chunk, dict) and chunk.get("usage")):
                    rec.chunk_times.append(now)  # apps with their own chunk type: every line counts as one token
                    rec.output_tokens += 1
            rec.ok = bool(rec.chunk_times)
    except Exception as e:  # noqa: BLE001
        rec.error = repr(e)


async def run(args: argparse.Namespace) -> Summary:
    rng = random.Random(args.seed)
    url = f"{args.gateway.rstrip('/')}/app/invoke/{args.app}"
    payloads = [build_request(i, args, rng) for i in range(args.num_prompts + args.warmup)]
    timeout = aiohttp.ClientTimeout(total=args.timeout)
    async with aiohttp.ClientSession(timeout=timeout, connector=aiohttp.TCPConnector(limit=0)) as http:
        for p in payloads[: args.warmup]:
            await one_request(http, url, p, RequestRecord(0.0))
        sched = (duty_cycle_times(args.num_prompts, args.rate, args.duty_on, args.duty_off, args.seed) if args.duty_on
                 else arrival_times(args.num_prompts, args.rate, args.burstiness, args.seed))
        records = [RequestRecord(0.0) for _ in range(args.num_prompts)]
        t0 = time.perf_counter()
        tasks = []
        for rec, p, at in zip(records, payloads[args.warmup:], sched):
            delay = t0 + at - time.perf_counter()
            if delay > 0:
                await asyncio.sleep(delay)
            tasks.append(asyncio.create_task(one_request(http, url, p, rec)))
        await asyncio.gather(*tasks)
        duration = time.perf_counter() - t0
    return summarise(records, duration)


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gateway", default="http://127.0.0.1:8000")
    ap.add_argument("--app", required=True, help="app id (or alias resolved by the CLI)")
    ap.add_argument("--rate", type=float, default=float("inf"), help="requests per second (inf = all at once)")
    ap.add_argument("--burstiness", type=float, default=1.0)
    ap.add_argument("--duty-on", type=float, default=0.0, help="seconds of traffic per cycle (0 = no duty cycle)")
    ap.add_argument("--duty-off", type=float, default=0.0)
    ap.add_argument("--num-prompts", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--input-len", type=int, default=128)
    ap.add_argument("--output-len", type=int, default=256)
    ap.add_argument("--image", default="1280x720", help="WIDTHxHEIGHT of synthetic images ('' = text only)")
    ap.add_argument("--images-per-request", type=int, default=1)
    ap.add_argument("--timeout", type=float, default=3600.0)
    ap.add_argument("--seed", type=int, default=48105)
    ap.add_argument("--output", default="")
    return ap.parse_args(argv)


def main(argv: list[str] | None = None) -> None:
    args = parse_args(argv)
    summary = asyncio.run(run(args))
    out = {"config": {k: v for k, v in vars(args).items()}, "result": asdict(summary)}
    text = json.dumps(out, indent=1, default=str)
    print(text)
    if args.output:
        with open(args.output, "w") as f:
            f.write(text)


if __name__ == "__main__":
    main()
