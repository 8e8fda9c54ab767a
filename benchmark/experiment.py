"""Experiments on deployment shapes (reference: benchmark/schema.py:16-295, cornserve_utils.py:32-284, run_compare.py).

An experiment = a model, a workload (prompt / output lengths, images per request, arrival rate and burstiness) and a
*backend configuration* that says how the model is cut into executors and how many GPUs each part gets:

  V     one monolithic LLM executor per replica; images are encoded inside it       {"llm": gpus}
  E     the encoder executor alone (outputs dropped): the encoder's own capacity     {"encoder": gpus}
  EV    encoder fission: Eric executors feed LLM executors through the sidecars      {"encoder": g1, "llm": g2}
  PD    prefill / decode disaggregation, encoder inside the prefill executor         {"prefill": g1, "decode": g2}
  EPD   all three separated                                                          {"encoder": g1, "prefill": g2, "decode": g3}

`run_experiment` registers the matching app at the gateway, scales every unit task to its GPU count
(``POST /task/scale``), drives the open-loop load generator and writes a result file whose name is derived from the
whole configuration, so repeated sweeps never overwrite or silently reuse each other's results.

    python -m benchmark.experiment --backend EV --gpus encoder=2,llm=6 --rate 10 --num-prompts 2000
"""

from __future__ import annotations

import argparse
import asyncio
import hashlib
import json
from dataclasses import asdict, dataclass, field
from pathlib import Path

import aiohttp

from . import load_generator

BACKENDS = ("V", "E", "EV", "PD", "EPD")
PARTS = {"V": ("llm",), "E": ("encoder",), "EV": ("encoder", "llm"), "PD": ("prefill", "decode"), "EPD": ("encoder", "prefill", "decode")}


@dataclass
class Workload:
    input_len: int = 500
    output_len: int = 500
    num_prompts: int = 2000
    num_warmups: int = 50
    request_rate: float = 10.0
    burstiness: float = 1.0
    image_width: int = 1920
    image_height: int = 1080
    image_count: int = 1
    seed: int = 48105


@dataclass
class ExperimentConfig:
    backend: str = "EV"
    model_id: str = "Qwen/Qwen2.5-VL-7B-Instruct"
    gpus: dict[str, int] = field(default_factory=lambda: {"encoder": 1, "llm": 1})
    workload: Workload = field(default_factory=Workload)
    gpu_type: str = "B200"

    def __post_init__(self) -> None:
        if self.backend not in BACKENDS:
            raise ValueError(f"backend must be one of {BACKENDS}")
        if set(self.gpus) != set(PARTS[self.backend]):
            raise ValueError(f"backend {self.backend} takes GPU counts for {PARTS[self.backend]}, got {sorted(self.gpus)}")
        if any(n < 1 for n in self.gpus.values()):
            raise ValueError("every part needs at least one GPU")

    @property
    def total_gpus(self) -> int:
        return sum(self.gpus.values())

    def key(self) -> str:
        """Stable name of this configuration: readable prefix + digest of every field."""
        blob = json.dumps(asdict(self), sort_keys=True).encode()
        parts = "-".join(f"{k[0]}{v}" for k, v in sorted(self.gpus.items()))
        w = self.workload
        return (f"{self.model_id.split('/')[-1].lower()}_{self.backend}_{parts}_in{w.input_len}_out{w.output_len}"
                f"_img{w.image_count}x{w.image_width}x{w.image_height}_r{w.request_rate:g}_{hashlib.sha1(blob).hexdigest()[:8]}")

    def result_path(self, root: str | Path = "benchmark/data") -> Path:
        return Path(root) / f"{self.key()}.json"


def app_source(cfg: ExperimentConfig) -> str:
    """Source of the app that realises ``cfg.backend`` (one streaming ``serve`` over the matching composite task)."""
    head = '''from collections.abc import AsyncIterator
from cornserve.app.base import AppConfig, AppRequest, AppResponse
from cornserve_tasklib import (DisaggregatedMLLMTask, MLLMTask, Modality, OpenAIChatCompletionChunk,
                                    OpenAIChatCompletionRequest)
from cornserve_tasklib.task.unit.encoder import DummyEncoderTask, EncoderInput

class Request(AppRequest):
    prompt: str
    multimodal_data: list[tuple[str, str]] = []
    max_completion_tokens: int = 256

def _messages(request):
    content = [{"type": f"{kind}_url", f"{kind}_url": {"url": url}} for kind, url in request.multimodal_data]
    return [{"role": "user", "content": [*content, {"type": "text", "text": request.prompt}]}]
'''
    m = cfg.model_id
    if cfg.backend == "E":
        return head + f'''
task = DummyEncoderTask(modality=Modality.IMAGE, model_ids={{"{m}"}})

class Config(AppConfig):
    tasks = {{"encoder": task}}

class Response(AppResponse):
    ok: bool

async def serve(request: Request) -> Response:
    await task(EncoderInput(model_id="{m}", data_urls=[url for _, url in request.multimodal_data]))
    return Response(ok=True)
'''
    cls = "MLLMTask" if cfg.backend in ("V", "EV") else "DisaggregatedMLLMTask"
    fission = cfg.backend in ("EV", "EPD")
    return head + f'''
task = {cls}(model_id="{m}", modalities=[Modality.IMAGE], encoder_fission={fission})

class Config(AppConfig):
    tasks = {{"mllm": task}}

async def serve(request: Request) -> AsyncIterator[OpenAIChatCompletionChunk]:
    return await task(OpenAIChatCompletionRequest(model="{m}", messages=_messages(request), ignore_eos=True, temperature=0.0,
                                                  max_completion_tokens=request.max_completion_tokens))
'''


def part_of(task_json: str) -> str | None:
    """Which part of a backend configuration a deployed unit task is."""
    cls = json.loads(task_json).get("class_name", "")
    low = (cls or task_json).lower()
    for key, part in (("prefill", "prefill"), ("decode", "decode"), ("encoder", "encoder"), ("llm", "llm")):
        if key in low:
            return part
    return None


async def deploy(cfg: ExperimentConfig, gateway: str) -> str:
    """Register the app, then grow every unit task from its single GPU to the configured count."""
    async with aiohttp.ClientSession(timeout=aiohttp.ClientTimeout(total=3600)) as http:
        async with http.post(f"{gateway}/app/register", json={"source_code": app_source(cfg)}) as resp:
            events = [json.loads(line.decode()[6:]) async for line in resp.content if line.startswith(b"data: ")]
        if not events or events[-1]["event"]["type"] != "final":
            raise RuntimeError(f"registration failed: {events[-1] if events else 'no events'}")
        app_id = events[0]["event"]["app_id"]
        async with http.get(f"{gateway}/tasks/list") as resp:
            tasks = await resp.json()
        for task_json, task_id, _state in tasks:
            extra = cfg.gpus.get(part_of(task_json) or "", 1) - 1
            if extra > 0:
                async with http.post(f"{gateway}/task/scale", json={"task_id": task_id, "num_gpus": extra}) as resp:
                    if resp.status != 200:
                        raise RuntimeError(f"scaling {task_id} by {extra} GPUs failed: {await resp.text()}")
    return app_id


async def run_experiment(cfg: ExperimentConfig, gateway: str = "http://127.0.0.1:8000", out_root: str = "benchmark/data",
                         keep_app: bool = False) -> dict:
    path = cfg.result_path(out_root)
    if path.exists():
        return json.loads(path.read_text())
    app_id = await deploy(cfg, gateway)
    w = cfg.workload
    args = load_generator.parse_args([
        "--gateway", gateway, "--app", app_id, "--rate", str(w.request_rate), "--burstiness", str(w.burstiness),
        "--num-prompts", str(w.num_prompts), "--warmup", str(w.num_warmups), "--input-len", str(w.input_len),
        "--output-len", str(w.output_len), "--image", f"{w.image_width}x{w.image_height}" if w.image_count else "",
        "--images-per-request", str(max(w.image_count, 1)), "--seed", str(w.seed)])
    try:
        summary = await load_generator.run(args)
    finally:
        if not keep_app:
            async with aiohttp.ClientSession() as http:
                await http.post(f"{gateway}/app/unregister/{app_id}")
    result = {"config": asdict(cfg), "key": cfg.key(), "result": asdict(summary)}
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(json.dumps(result, indent=1))
    return result


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gateway", default="http://127.0.0.1:8000")
    ap.add_argument("--backend", choices=BACKENDS, default="EV")
    ap.add_argument("--model", default="Qwen/Qwen2.5-VL-7B-Instruct")
    ap.add_argument("--gpus", default="encoder=1,llm=1", help="comma-separated part=count")
    ap.add_argument("--rate", type=float, default=10.0)
    ap.add_argument("--burstiness", type=float, default=1.0)
    ap.add_argument("--num-prompts", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--input-len", type=int, default=500)
    ap.add_argument("--output-len", type=int, default=500)
    ap.add_argument("--image", default="1920x1080")
    ap.add_argument("--image-count", type=int, default=1)
    ap.add_argument("--out", default="benchmark/data")
    a = ap.parse_args(argv)
    iw, ih = (int(v) for v in a.image.split("x")) if a.image else (0, 0)
    cfg = ExperimentConfig(a.backend, a.model, {k: int(v) for k, v in (kv.split("=") for kv in a.gpus.split(","))},
                           Workload(a.input_len, a.output_len, a.num_prompts, a.warmup, a.rate, a.burstiness, iw, ih,
                                    a.image_count if a.image else 0))
    print(json.dumps(asyncio.run(run_experiment(cfg, a.gateway, a.out)), indent=1))


if __name__ == "__main__":
    main()
