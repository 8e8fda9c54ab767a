"""LLM executor: OpenAI-compatible chat-completions server on top of :class:`LLMEngine`.

This process plays the role the reference gives to its vLLM fork (contract in
tasklib/cornserve_tasklib/task_executors/descriptor/llm.py:68-563 and docker/vllm.Dockerfile):

* ``POST /v1/chat/completions`` (server-sent events when ``stream`` is true, one JSON otherwise), ``GET /health``.
* Multimodal parts whose URL is ``data:{modality}/uuid;data_id={id};url={original},`` are not decoded here:
  the embeddings with that id are received from the sidecar (a view of the producer's GPU slab) and placed
  into the prompt embeddings by a copy kernel.  Plain URLs are encoded locally by an in-process vision tower
  (the monolithic, no-fission deployment).
* ``vllm_xargs`` carries forwarding instructions: ``cornserve_hidden_states_forward_id/_ranks`` sends the
  prompt's final hidden states to another executor instead of generating text.
* Prefill/decode disaggregation (``--kv-transfer-config {"kv_role": "kv_producer" | "kv_consumer"}``; the reference
  delegates this to vLLM's NIXL connector, descriptor/llm.py:213-563).  A producer answers a request after one token,
  keeps the prompt's KV pages and forwards ``kv_transfer_params`` (page numbers, first token, how to reach the cache)
  under ``cornserve_kv_transfer_params_forward_id``.  A consumer that gets ``cornserve_kv_transfer_params_recv_id``
  maps the producer's cache (CUDA IPC, once per producer), pulls the pages with one copy kernel over NVLink and
  decodes; when the producer's GPU is not reachable it fetches the pages over HTTP instead.  Either way it then tells
  the producer to free the pages (``POST /kv/release``).

The command line accepts the flags the descriptors pass (vLLM-style names); flags that only make sense for
vLLM are accepted and ignored.
"""

from __future__ import annotations

import argparse
import ast
import asyncio
import base64
import concurrent.futures
import contextlib
import dataclasses
import io
import json
import os
import random
import re
import sys
import socket
import threading
import time
import uuid
from dataclasses import dataclass, field
from typing import Any

import numpy as np
import torch
import uvicorn
from fastapi import FastAPI, Request, Response
from fastapi.responses import JSONResponse, StreamingResponse

from ... import ops
from ...logging import get_logger
from ...models.qwen_llm import LLMConfig, QwenLLM
from ...parallel.state import ParallelGroup
from ...tracing import configure_otel
from ...utils.hub import load_config, load_model_weights
from ...utils.threads import maybe_start_sampler, sampler_report, tune_interpreter
from ..eric.preprocess import smart_resize
from ..eric.processor import fetch_bytes
from .engine import EngineConfig, LLMEngine, MMItem, PrefilledKV, SamplingParams, Sequence, StepOutput
from .tokenizer import load_tokenizer

logger = get_logger(__name__)

_SIDECAR_URI = re.compile(r"^data:(?P<modality>\w+)/uuid;data_id=(?P<id>[0-9a-f]+);url=(?P<url>.*),$", re.S)


def parse_args(argv: list[str] | None = None) -> argparse.Namespace:
    ap = argparse.ArgumentParser("cornserve-b200 LLM executor")
    ap.add_argument("model")
    ap.add_argument("--tensor-parallel-size", type=int, default=1)
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--host", default="127.0.0.1")
    ap.add_argument("--cornserve-sidecar-ranks", type=int, nargs="*", default=[])
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-model-len", type=int, default=32768)
    ap.add_argument("--max-num-batched-tokens", type=int, default=18944)
    ap.add_argument("--quantization", default=None, choices=[None, "fp8"],
                    help="fp8: attention and MLP projections as e4m3 with 128x128 block scales (also chosen when the "
                         "checkpoint's quantization_config says fp8)")
    ap.add_argument("--gpu-memory-utilization", type=float, default=0.9)
    ap.add_argument("--num-kv-pages", type=int, default=0, help="0 = size the cache from free memory")
    ap.add_argument("--decode-burst", type=int, default=4)
    ap.add_argument("--kv-transfer-config", default=None)
    ap.add_argument("--tp-rank", type=int, default=0, help="set by the executor itself for its follower ranks")
    ap.add_argument("--tp-port", type=int, default=0, help="rendezvous port of the tensor-parallel ranks")
    ap.add_argument("--run-talker", action="store_true")
    ap.add_argument("--run-vocoder", action="store_true")
    for flag in ("--trust-remote-code", "--enforce-eager", "--no-enable-prefix-caching", "--disable-mm-preprocessor-cache",
                 "--no-enable-chunked-prefill", "--disable-chunked-mm-input"):
        ap.add_argument(flag, action="store_true", help="accepted for compatibility")
    return ap.parse_args(argv)


def pick_device() -> torch.device:
    if not torch.cuda.is_available() or os.environ.get("CORNSERVE_DEVICE") == "cpu":
        return torch.device("cpu")
    ids = [int(x) for x in os.environ.get("CORNSERVE_LOCAL_GPUS", "").split(",") if x.strip() != ""]
    return torch.device("cuda", ids[0] if ids else 0)


@dataclass
class _Pending:
    queue: asyncio.Queue
    loop: asyncio.AbstractEventLoop
    recv_ids: list[str] = field(default_factory=list)


class AsyncLLM:
    """Runs the synchronous engine on its own thread and fans step outputs out to per-request queues."""

    def __init__(self, engine: LLMEngine, tp=None):
        self.engine = engine
        self.tp = tp   # tensor-parallel control channel: every step is announced to the follower ranks first
        self.pending: dict[str, _Pending] = {}
        self.inbox: list[Sequence] = []
        self.aborts: list[str] = []
        self.calls: list[tuple[Any, concurrent.futures.Future]] = []
        self.cv = threading.Condition()
        self.alive = True
        self.thread = threading.Thread(target=self._run, name="llm-engine", daemon=True)
        self.thread.start()

    def submit(self, seq: Sequence) -> asyncio.Queue:
        q: asyncio.Queue = asyncio.Queue()
        self.pending[seq.seq_id] = _Pending(q, asyncio.get_running_loop())
        with self.cv:
            self.inbox.append(seq)
            self.cv.notify()
        return q

    def abort(self, seq_id: str) -> None:
        """Take a sequence out of the engine (a stop string matched, the client disconnected).  Runs on the engine
        thread, and on every follower rank of a tensor-parallel executor at the same point of the step sequence."""
        self.pending.pop(seq_id, None)
        with self.cv:
            self.aborts.append(seq_id)
            self.cv.notify()

    def call(self, fn) -> concurrent.futures.Future:
        """Run ``fn()`` on the engine thread (the engine's state is not shared between threads)."""
        fut: concurrent.futures.Future = concurrent.futures.Future()
        with self.cv:
            self.calls.append((fn, fut))
            self.cv.notify()
        return fut

    def _deliver(self, out: StepOutput) -> None:
        p = self.pending.get(out.seq_id)
        if p is None:
            return
        if out.finished:
            self.pending.pop(out.seq_id, None)
        p.loop.call_soon_threadsafe(p.queue.put_nowait, out)

    def _run(self) -> None:
        ops.bind_thread(self.engine.device)  # a new thread starts on CUDA device 0
        from .tp import IDLE_BEAT_S

        last_beat = time.monotonic()
        try:
            while self.alive:
                with self.cv:
                    while self.alive and not self.inbox and not self.calls and not self.aborts and not self.engine.has_work():
                        self.cv.wait(timeout=0.5)
                        if self.engine.held or (self.tp is not None and time.monotonic() - last_beat > IDLE_BEAT_S):
                            break
                    new, self.inbox = self.inbox, []
                    calls, self.calls = self.calls, []
                    aborts, self.aborts = self.aborts, []
                for fn, fut in calls:
                    try:
                        fut.set_result(fn())
                    except Exception as e:
                        fut.set_exception(e)
                if self.engine.held:
                    for sid in self.engine.expire_held(float(os.environ.get("CORNSERVE_KV_HOLD_SECONDS", "600"))):
                        logger.warning("Freed the KV pages of %s: nobody fetched them", sid)
                if self.tp is not None:
                    if not new and not self.engine.has_work():
                        # nothing to run: the followers only get a keep-alive now and then, so that their wait on the
                        # control group can have a finite timeout
                        if time.monotonic() - last_beat > IDLE_BEAT_S:
                            self.tp.publish([], beat=True)
                            last_beat = time.monotonic()
                        continue
                    last_beat = time.monotonic()
                    for s in new:
                        if s.params.samples and s.params.seed is None:
                            s.params.seed = random.getrandbits(62)   # drawn here so that every rank gets the same stream
                    self.tp.publish(new, aborts=aborts)
                for sid in aborts:
                    self.engine.abort(sid)
                for s in new:
                    try:
                        self.engine.add_request(s)
                    except Exception as e:
                        self._deliver(StepOutput(s.seq_id, [], True, f"error: {e}"))
                outs = self.engine.step()
                for out in outs:
                    self._deliver(out)
                if not outs and not new and not self.engine.running:
                    # work is queued but nothing could be scheduled (pages held for a remote reader, say): wait for
                    # a new request, a call or the next poll instead of spinning
                    with self.cv:
                        if not self.inbox and not self.calls:
                            self.cv.wait(timeout=0.005)
        except Exception:
            logger.exception("LLM engine thread died")
        finally:
            self.alive = False
            if self.tp is not None:
                try:
                    self.tp.publish([], stop=True)
                except Exception:  # noqa: BLE001
                    logger.exception("could not tell the follower ranks to stop")
            for sid in list(self.pending):
                self._deliver(StepOutput(sid, [], True, "error: engine stopped"))

    def shutdown(self) -> None:
        self.alive = False
        with self.cv:
            self.cv.notify_all()
        self.thread.join(timeout=10)


def build_engine(args: argparse.Namespace, group: ParallelGroup | None = None) -> tuple[LLMEngine, dict[str, Any]]:
    hf_cfg = load_config(args.model)
    # any-to-any checkpoints keep their language model under "thinker"
    cfg = LLMConfig.from_hf(hf_cfg.get("thinker_config") or hf_cfg)
    device = group.device if group is not None else pick_device()
    if device.type == "cuda":
        torch.cuda.set_device(device)
    torch.manual_seed(int(os.environ.get("CORNSERVE_SEED", "0")))  # reproducible random-weight runs
    model = QwenLLM(cfg, group=group, device=device)
    if device.type == "cpu":
        model = model.float()  # the CUDA kernels are bf16; fp32 is the CPU restatement's precision
    load_model_weights(model, args.model, ["thinker.model.", "thinker.", "model.language_model.", "language_model.", "model.", ""],
                       strict=False, ignored_prefixes=["visual.", "model.visual.", "vision_tower.", "thinker.visual.", "thinker.audio_tower.",
                                                       "talker.", "code2wav."])
    model.eval()
    qcfg = hf_cfg.get("quantization_config") or (hf_cfg.get("thinker_config") or {}).get("quantization_config") or {}
    if getattr(args, "quantization", None) == "fp8" or qcfg.get("quant_method") == "fp8":
        model.quantize_fp8_()
        logger.info("serving the attention and MLP projections in block-scaled fp8")
    pages = args.num_kv_pages
    if pages <= 0:
        if device.type == "cuda":
            free, _ = torch.cuda.mem_get_info(device)
            budget = int(free * args.gpu_memory_utilization) - (4 << 30)
            pages = max(64, budget // model.kv_bytes_per_page())
        else:
            pages = 64
    if group is not None and group.size > 1:
        from .tp import agree_on_min

        pages = agree_on_min(int(pages), group)
    ecfg = EngineConfig(num_pages=int(pages), max_batched_tokens=args.max_num_batched_tokens, max_num_seqs=args.max_num_seqs,
                        decode_burst=args.decode_burst, max_model_len=args.max_model_len,
                        use_cuda_graph=device.type == "cuda")
    engine = LLMEngine(model, ecfg)
    if os.environ.get("CORNSERVE_LLM_PRECAPTURE", "1") == "1":
        t0 = time.perf_counter()
        n = engine.capture_decode_graphs()
        if n:
            logger.info("captured %d decode graphs in %.1f s", n, time.perf_counter() - t0)
    return engine, hf_cfg


class LocalEncoder:
    """The vision tower inside the LLM executor (the monolithic, no-fission deployment).

    Images of waiting requests are encoded by a thread of their own on a high-priority CUDA stream, in batches of up to
    ``MAX_PATCHES`` patches, so that the tower's kernels run beside the decode graphs of the engine thread instead of
    queueing behind them, and so that the event loop never waits for the GPU.  Raw pixels go to the GPU through one
    page-locked staging buffer."""

    MAX_PATCHES = 34000      # seven 1280x720 images: whole tile waves on 148 SMs for the tower's GEMMs
    STAGING_BYTES = 128 << 20

    def __init__(self, server: "LLMServer"):
        import queue

        from ...models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer

        self.device = server.engine.device
        v = Qwen25VisionTransformer(Qwen25VisionConfig.from_hf(server.hf_cfg), device=self.device)
        if next(server.engine.model.parameters()).dtype == torch.float32:
            v = v.float()
        load_model_weights(v, server.args.model, ["visual.", "model.visual."], strict=False)
        self.vision = v.eval()
        self.inbox: queue.Queue = queue.Queue()
        self.h2d_bytes = 0
        self.images = 0
        self.batches = 0
        self.busy_ms = 0.0
        self.host_ms = 0.0
        self.wait_ms = 0.0
        self.stream = torch.cuda.Stream(device=self.device, priority=-1) if self.device.type == "cuda" else None
        self.stage = torch.empty(self.STAGING_BYTES, dtype=torch.uint8, pin_memory=True) if self.stream is not None else None
        self.thread = threading.Thread(target=self._run, name="llm-local-encoder", daemon=True)
        self.thread.start()

    async def encode(self, url: str) -> tuple[torch.Tensor, tuple[int, int, int]]:
        from ..eric.processor import load_image

        pixels = torch.from_numpy(await asyncio.to_thread(load_image, url))
        loop = asyncio.get_running_loop()
        fut: asyncio.Future = loop.create_future()
        self.inbox.put((pixels, loop, fut))
        return await fut

    def _run(self) -> None:
        import queue

        from ..eric.preprocess import patchify_frames

        ops.bind_thread(self.device)
        vc = self.vision.cfg
        per_image_guess = 0
        while True:
            batch = [self.inbox.get()]
            while True:   # whatever else is waiting, up to the patch budget
                if per_image_guess and (len(batch) + 1) * per_image_guess > self.MAX_PATCHES:
                    break
                try:
                    batch.append(self.inbox.get_nowait())
                except queue.Empty:
                    break
            t0 = time.perf_counter()
            try:
                ctx = torch.cuda.stream(self.stream) if self.stream is not None else contextlib.nullcontext()
                with torch.inference_mode(), ctx:
                    pix, grids, used = [], [], 0
                    for img, _, _ in batch:
                        n = img.numel()
                        if self.stage is not None and used + n <= self.stage.numel():
                            view = self.stage[used: used + n].view(img.shape)
                            view.copy_(img)
                            used += -(-n // 256) * 256
                            dev_img = view.to(self.device, non_blocking=True)
                        else:
                            dev_img = img.to(self.device)
                        self.h2d_bytes += n
                        pv, grid = patchify_frames(dev_img, vc.patch_size, vc.temporal_patch_size, vc.spatial_merge_size,
                                                   out_dtype=self.vision.dtype)
                        pix.append(pv)
                        grids.append(grid)
                    per_image_guess = max(per_image_guess, max(p.shape[0] for p in pix))
                    embs = self.vision("image", None, {"pixel_values": pix, "image_grid_thw": [list(g) for g in grids]})
                    embs = [e.contiguous() for e in embs]
                    if self.stream is not None:
                        for e in embs:   # consumed later by the engine thread's kernels on the default stream
                            e.record_stream(torch.cuda.default_stream(self.device))
                        t_issued = time.perf_counter()
                        self.stream.synchronize()
                        self.host_ms += (t_issued - t0) * 1e3   # staging, preprocessing and launching the tower
                        self.wait_ms += (time.perf_counter() - t_issued) * 1e3   # the GPU finishing it
                self.images += len(batch)
                self.batches += 1
                self.busy_ms += (time.perf_counter() - t0) * 1e3
                for (_, loop, fut), emb, grid in zip(batch, embs, grids):
                    loop.call_soon_threadsafe(lambda f=fut, r=(emb, grid): f.done() or f.set_result(r))
            except Exception as e:  # noqa: BLE001
                logger.exception("local encoding failed")
                for _, loop, fut in batch:
                    loop.call_soon_threadsafe(lambda f=fut, err=e: f.done() or f.set_exception(err))


class LLMServer:
    def __init__(self, args: argparse.Namespace):
        self.args = args
        self.followers: list = []
        tp = int(args.tensor_parallel_size)
        if tp > 1:
            from . import tp as tpmod

            if args.kv_transfer_config:
                raise ValueError("prefill/decode disaggregation is not available with --tensor-parallel-size > 1")
            port = tpmod.free_port()
            self.followers = tpmod.spawn_followers(getattr(args, "argv", None) or sys.argv[1:], tp, port)
            group = tpmod.join_group(0, tp, port)
            self.engine, self.hf_cfg = build_engine(args, group)
            control = tpmod.TPControl(group, next(self.engine.model.parameters()).dtype)
            self.llm = AsyncLLM(self.engine, tp=control)
        else:
            self.engine, self.hf_cfg = build_engine(args)
            self.llm = AsyncLLM(self.engine)
        self.cfg = self.engine.mcfg
        self.tokenizer = load_tokenizer(args.model, {**(self.hf_cfg.get("thinker_config") or {}), **self.hf_cfg}, self.cfg.vocab_size)
        self.omni_cfg = self.hf_cfg if "talker_config" in self.hf_cfg else None
        self.default_temperature = self._default_temperature()
        self.receive_embeddings = os.environ.get("CORNSERVE_VLLM_DISABLE_MULTIMODAL") == "1"
        self.sidecar = None
        if args.cornserve_sidecar_ranks:
            from ...sidecar.api import Sidecar
            from ...sidecar.schema import SidecarConfig

            dtype = next(self.engine.model.parameters()).dtype
            # the leader alone talks to the sidecars: it answers for the follower ranks too
            self.sidecar = Sidecar(SidecarConfig(sidecar_rank=args.cornserve_sidecar_ranks[0],
                                                 group=list(args.cornserve_sidecar_ranks), whole_group=True,
                                                 send_tensor_dtype=dtype, send_tensor_shape=(-1, self.cfg.hidden_size),
                                                 recv_tensor_dtype=dtype, recv_tensor_shape=(-1, self.cfg.hidden_size)))
        self.local_encoder: LocalEncoder | None = None  # built lazily for requests that carry raw URLs (no fission)
        self.timing = {"requests": 0, "inputs_ms": 0.0, "first_token_ms": 0.0}
        kv_cfg = json.loads(args.kv_transfer_config) if args.kv_transfer_config else {}
        self.kv_role = kv_cfg.get("kv_role")
        self.engine_id = uuid.uuid4().hex
        self._kv_export: dict[str, Any] | None = None
        self._kv_maps: dict[str, torch.Tensor] = {}   # producer engine id -> its cache mapped into this process

    def _default_temperature(self) -> float:
        """What a request without ``temperature`` gets: the model's ``generation_config.json`` when it names one
        (greedy when it says ``do_sample: false``), else the OpenAI default 1.0."""
        from ...utils.hub import resolve_model_dir

        d = resolve_model_dir(self.args.model)
        try:
            if d is not None and (d / "generation_config.json").is_file():
                g = json.loads((d / "generation_config.json").read_text())
                if g.get("do_sample") is False:
                    return 0.0
                if g.get("temperature") is not None:
                    return float(g["temperature"])
        except (OSError, ValueError):
            pass
        return 1.0

    @staticmethod
    def _stops(body: dict[str, Any]) -> list[str]:
        stop = body.get("stop")
        if stop is None:
            return []
        return [stop] if isinstance(stop, str) else [str(x) for x in stop if x]

    # -- multimodal inputs ----------------------------------------------------------------------------------
    def _grid_of(self, modality: str, url: str, n_rows: int) -> tuple[int, int, int] | None:
        """Patch grid of the item behind ``url`` (needed for M-RoPE): read the image size, not the pixels."""
        merge = self.cfg.spatial_merge_size
        try:
            if url.startswith("synthetic:"):
                h, w = (int(v) for v in url.split(":")[1].split("x"))
            else:
                from PIL import Image

                data, _ = fetch_bytes(url)
                w, h = Image.open(io.BytesIO(data)).size
            rh, rw = smart_resize(h, w, 14 * merge)
            gh, gw = rh // 14, rw // 14
            per_frame = (gh // merge) * (gw // merge)
            t = max(1, n_rows // per_frame)
            if t * per_frame == n_rows:
                return (t, gh, gw)
        except Exception as e:
            logger.warning("Could not determine the grid of %s (%s); using sequential positions", url[:60], e)
        return None

    async def _local_encode(self, modality: str, url: str) -> tuple[torch.Tensor, tuple[int, int, int]]:
        if self.local_encoder is None:
            self.local_encoder = LocalEncoder(self)
        return await self.local_encoder.encode(url)

    async def build_sequence(self, body: dict[str, Any]) -> tuple[Sequence, list[str]]:
        messages = body["messages"]
        ids, marks = self.tokenizer.render_chat(messages)
        parts = [p for m in messages if not isinstance(m["content"], str) for p in m["content"]
                 if p.get("type", "text") != "text"]
        if len(parts) != len(marks):
            raise ValueError("placeholder count does not match the multimodal parts")
        async def one(p) -> tuple[torch.Tensor, tuple[int, int, int] | None, list[str]]:
            modality = p["type"].split("_")[0]
            url = p[p["type"]]["url"]
            m = _SIDECAR_URI.match(url)
            if m is None:
                emb, grid = await self._local_encode(modality, url)
                return emb, grid, []
            if self.sidecar is None:
                raise ValueError("request refers to forwarded embeddings but this executor has no sidecar")
            chunks, k = [], 0
            while True:
                t = await self.sidecar.recv(m["id"], k)
                if t is None:
                    break
                chunks.append(t)
                k += 1
            rows = chunks[0] if len(chunks) == 1 else torch.cat(chunks, dim=0)
            return rows, self._grid_of(modality, m["url"], rows.shape[0]), [f"{m['id']}:{i}" for i in range(k)]

        # all parts of a request at once: forwarded embeddings arrive in any order, and locally encoded images of one
        # request share a tower pass
        got = await asyncio.gather(*(one(p) for p in parts))
        embeds = [(rows, grid) for rows, grid, _ in got]
        recv_ids = [r for _, _, ids_ in got for r in ids_]
        # expand each single placeholder into as many pad tokens as there are embedding rows
        out: list[int] = []
        items: list[MMItem] = []
        prev = 0
        for (pos, modality), (rows, grid), part in zip(marks, embeds, parts):
            out += ids[prev:pos]
            spg = None
            if modality == "video":
                # seconds per temporal grid step = frames merged per step / sampling rate (Hugging Face: fps 2 -> 1.0 s)
                fps = float((part.get(part["type"]) or {}).get("fps") or body.get("video_fps") or 2.0)
                spg = float((self.hf_cfg.get("vision_config") or {}).get("temporal_patch_size", 2)) / fps
            items.append(MMItem(rows, len(out), grid, spg))
            out += [ids[pos]] * rows.shape[0]
            prev = pos + 1
        out += ids[prev:]
        params = SamplingParams.from_request(body, self.default_temperature,
                                             max_tokens=int(body.get("max_completion_tokens") or body.get("max_tokens") or 256),
                                             ignore_eos=bool(body.get("ignore_eos", False)))
        # without grids M-RoPE degrades to sequential positions (text-only layout)
        if any(it.grid_thw is None for it in items):
            for it in items:
                it.grid_thw = None
        xargs = body.get("vllm_xargs") or {}
        seq = Sequence(body.get("request_id") or uuid.uuid4().hex, np.asarray(out, dtype=np.int32), params, mm_items=items,
                       return_hidden="cornserve_hidden_states_forward_id" in xargs)
        return seq, recv_ids

    async def _release(self, recv_ids: list[str]) -> None:
        for rid in recv_ids:
            data_id, chunk = rid.split(":")
            try:
                await self.sidecar.mark_done(data_id, int(chunk))
            except Exception:
                logger.exception("mark_done failed for %s", rid)

    # -- prefill/decode disaggregation ---------------------------------------------------------------------
    def kv_export(self) -> dict[str, Any]:
        """How another executor reaches this engine's KV cache (a CUDA-IPC handle of the one cache allocation when the
        cache is on a GPU, and the URL that serves pages to executors that cannot map it)."""
        if self._kv_export is None:
            eng = self.engine
            info: dict[str, Any] = {"engine_id": self.engine_id, "base_url": f"http://{self.args.host}:{self.args.port}",
                                    "hostname": socket.gethostname(), **eng.kv_geometry()}
            if eng.on_gpu:
                from ...utils.cuda_ipc import export_tensor

                info["ipc"] = export_tensor(eng.kv_backing)   # plain fields: the consumer rebuilds them with type checks
                info["gpu_uuid"] = str(torch.cuda.get_device_properties(eng.device).uuid)
            self._kv_export = info
        return self._kv_export

    def _map_producer_cache(self, params: dict[str, Any]) -> torch.Tensor | None:
        """The producer's cache as a tensor of this process, or ``None`` when it cannot be mapped (other host, GPU not
        visible here, CPU engines).  Mapped once per producer."""
        eid = params.get("engine_id")
        if eid == self.engine_id:
            return self.engine.kv_backing
        if not self.engine.on_gpu or "ipc" not in params or params.get("hostname") != socket.gethostname():
            return None
        if eid in self._kv_maps:
            return self._kv_maps[eid]
        mine = self.engine.device.index
        theirs = next((i for i in range(torch.cuda.device_count())
                       if str(torch.cuda.get_device_properties(i).uuid) == params.get("gpu_uuid")), None)
        if theirs is None or (theirs != mine and not torch.cuda.can_device_access_peer(mine, theirs)):
            return None
        from ...utils.cuda_ipc import import_tensor

        try:
            # The handle is opened with THIS executor's GPU current (the open then enables peer access between the two
            # GPUs as needed), so the mapping is addressable by kernels of this GPU; the tensor is labelled accordingly.
            mapped = import_tensor(params["ipc"], mine)
            if list(mapped.shape) != [int(v) for v in params["shape"]]:
                raise ValueError("the exported tensor does not have the advertised cache shape")
            # reach it once through the driver's copy path (which reports an error instead of faulting) before any
            # kernel reads it
            probe = torch.empty(8, dtype=mapped.dtype, device=self.engine.device)
            probe.copy_(mapped.reshape(-1)[:8])
            torch.cuda.synchronize(self.engine.device)
        except Exception:
            logger.exception("Could not map the KV cache of engine %s; falling back to the network path", eid)
            return None
        self._kv_maps[eid] = mapped
        return mapped

    async def _fetch_pages(self, params: dict[str, Any]) -> torch.Tensor:
        import aiohttp

        async with aiohttp.ClientSession() as sess:
            async with sess.post(f"{params['base_url']}/kv/pages", json={"request_id": params["request_id"]}) as r:
                r.raise_for_status()
                data = await r.read()
        shape = list(params["shape"])
        shape[1] = len(params["pages"])
        return torch.frombuffer(bytearray(data), dtype=getattr(torch, params["dtype"])).view(shape)

    async def _release_at_producer(self, params: dict[str, Any]) -> None:
        if params.get("engine_id") == self.engine_id:
            await asyncio.wrap_future(self.llm.call(lambda: self.engine.release_held(params["request_id"])))
            return
        import aiohttp

        try:
            async with aiohttp.ClientSession() as sess:
                async with sess.post(f"{params['base_url']}/kv/release", json={"request_id": params["request_id"]}) as r:
                    await r.read()
        except Exception:
            logger.exception("Could not tell %s to free the pages of %s", params.get("base_url"), params.get("request_id"))

    async def _sidecar_parts(self, body: dict[str, Any]) -> list[str]:
        """Forwarded embeddings named by a request that does not need them (its prompt is already prefilled): receive
        them so that they can be marked done."""
        recv_ids: list[str] = []
        for m in body["messages"]:
            if isinstance(m["content"], str):
                continue
            for p in m["content"]:
                if p.get("type", "text") == "text":
                    continue
                hit = _SIDECAR_URI.match(p[p["type"]]["url"])
                if hit is None or self.sidecar is None:
                    continue
                k = 0
                while await self.sidecar.recv(hit["id"], k) is not None:
                    k += 1
                recv_ids.extend(f"{hit['id']}:{i}" for i in range(k))
        return recv_ids

    def _check_transfer(self, params: dict[str, Any]) -> None:
        """The producer's cache must have this engine's geometry (layers, heads, page size, head width, dtype): the
        copy kernel and the page assignment assume it, and a mismatch would otherwise surface inside an engine step."""
        mine = self.engine.kv_geometry()
        shape = [int(v) for v in params.get("shape") or []]
        if len(shape) != len(mine["shape"]) or shape[0] != mine["shape"][0] or shape[2:] != mine["shape"][2:]:
            raise ValueError(f"KV transfer from a cache of shape {shape}; this executor's cache is {mine['shape']}")
        if str(params.get("dtype")) != mine["dtype"]:
            raise ValueError(f"KV transfer of dtype {params.get('dtype')}; this executor's cache is {mine['dtype']}")
        pages = params.get("pages")
        if not isinstance(pages, list) or not pages or any(int(p) < 0 or int(p) >= shape[1] for p in pages):
            raise ValueError("KV transfer names pages outside the producer's cache")
        for k in ("first_token", "next_pos", "num_tokens", "request_id"):
            if k not in params:
                raise ValueError(f"KV transfer parameters lack {k!r}")

    async def build_prefilled_sequence(self, body: dict[str, Any], params: dict[str, Any]) -> tuple[Sequence, list[str]]:
        self._check_transfer(params)
        src = self._map_producer_cache(params)
        raw = None if src is not None else await self._fetch_pages(params)
        pf = PrefilledKV(int(params["first_token"]), int(params["next_pos"]), [int(p) for p in params["pages"]], src_cache=src, raw=raw)
        sp = SamplingParams.from_request(body, self.default_temperature,
                                         max_tokens=int(body.get("max_completion_tokens") or body.get("max_tokens") or 256),
                                         ignore_eos=bool(body.get("ignore_eos", False)))
        seq = Sequence(body.get("request_id") or uuid.uuid4().hex, np.zeros(int(params["num_tokens"]), dtype=np.int32), sp,
                       prefilled=pf)
        return seq, await self._sidecar_parts(body)

    async def _omni_thinker_forward(self, seq: Sequence, queue: asyncio.Queue, xargs: dict[str, Any], rid: str, created: int, model: str):
        """Thinker half of a spoken answer: generate the text, then run the whole conversation (prompt + answer) once more
        to capture what the talker conditions on (token embeddings and the hidden states of the accepted layer), and forward
        that view together with the embeddings of the TTS control tokens (:func:`models.omni_talker.pack_thinker_view`)."""
        from ...models.omni_talker import pack_thinker_view

        tokens: list[int] = []
        while True:
            out: StepOutput = await queue.get()
            tokens.extend(out.new_token_ids)
            if out.finished:
                break
        if (out.finish_reason or "").startswith("error"):
            return JSONResponse({"error": {"message": out.finish_reason}}, status_code=500)
        tc = self.omni_cfg["talker_config"]
        full = np.concatenate([seq.prompt_ids, np.asarray(tokens, dtype=np.int32)])
        view_seq = Sequence(seq.seq_id + "-view", full, SamplingParams(max_tokens=1, ignore_eos=True), mm_items=seq.mm_items,
                            capture_layers=(0, int(tc.get("accept_hidden_layer", 18))))
        q2 = self.llm.submit(view_seq)
        while True:
            out2: StepOutput = await q2.get()
            if out2.finished:
                break
        if out2.hidden is None:
            return JSONResponse({"error": {"message": out2.finish_reason or "no hidden states"}}, status_code=500)
        H = self.cfg.hidden_size
        tts_ids = [int(self.omni_cfg.get(k, d)) for k, d in (("tts_bos_token_id", 151672), ("tts_eos_token_id", 151673),
                                                            ("tts_pad_token_id", 151671))]
        dev = self.engine.device
        tts = await asyncio.wrap_future(self.llm.call(
            lambda: self.engine.model.embed_tokens(torch.tensor(tts_ids, dtype=torch.int32, device=dev))))
        rows = pack_thinker_view(full, out2.hidden[:, :H], out2.hidden[:, H:], tts)
        ranks = ast.literal_eval(xargs.get("cornserve_hidden_states_forward_ranks", "[]")) or []
        if ranks and self.sidecar is not None:
            self.sidecar.send(rows.contiguous(), id=xargs["cornserve_hidden_states_forward_id"], dst_sidecar_ranks=ranks)
            await asyncio.to_thread(self.sidecar.flush)
        return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model,
                             "choices": [{"index": 0, "message": {"role": "assistant", "content": self.tokenizer.decode(tokens)},
                                          "finish_reason": out.finish_reason}],
                             "cornserve": {"hidden_states_rows": int(rows.shape[0])}})

    # -- request handling ---------------------------------------------------------------------------------------
    async def chat(self, body: dict[str, Any]):
        xargs = body.get("vllm_xargs") or {}
        kv_in: dict[str, Any] | None = None
        t_arrival = time.perf_counter()
        try:
            recv_kv = xargs.get("cornserve_kv_transfer_params_recv_id")
            if recv_kv is not None:
                if self.sidecar is None:
                    raise ValueError("request refers to forwarded KV parameters but this executor has no sidecar")
                kv_in = await self.sidecar.recv(recv_kv)
                await self.sidecar.mark_done(recv_kv)
            elif isinstance(body.get("kv_transfer_params"), dict) and "pages" in body["kv_transfer_params"]:
                kv_in = body["kv_transfer_params"]
            if kv_in is not None:
                seq, recv_ids = await self.build_prefilled_sequence(body, kv_in)
            else:
                seq, recv_ids = await self.build_sequence(body)
        except Exception as e:
            logger.exception("Bad request")
            return JSONResponse({"error": {"message": str(e), "type": "invalid_request_error"}}, status_code=400)
        producer = kv_in is None and "cornserve_hidden_states_forward_id" not in xargs and (
            self.kv_role == "kv_producer" or bool((body.get("kv_transfer_params") or {}).get("do_remote_decode")))
        if producer:
            seq.hold_kv = True
            seq.params.max_tokens = 1
        created, rid, model = int(time.time()), f"chatcmpl-{seq.seq_id}", body.get("model", self.args.model)
        omni_view = "cornserve_hidden_states_forward_id" in xargs and self.omni_cfg is not None and kv_in is None
        if omni_view:
            seq.return_hidden = False   # the answer is generated first; the talker's view is captured in a second pass
            held_ids, recv_ids = recv_ids, []   # the encoder rows are needed again by that pass: release them afterwards
        n_choices = max(1, int(body.get("n") or 1))
        if n_choices > 1 and (omni_view or producer or kv_in is not None or "cornserve_hidden_states_forward_id" in xargs):
            await self._release(recv_ids)
            return JSONResponse({"error": {"message": "n > 1 is available for plain chat completions only",
                                           "type": "invalid_request_error"}}, status_code=400)
        t_built = time.perf_counter()
        self.timing["requests"] += 1
        self.timing["inputs_ms"] += (t_built - t_arrival) * 1e3   # tokenising + encoding or receiving the embeddings
        # ``n`` choices are n sequences over the same prompt (and the same encoder rows), each with its own random stream
        seqs = [seq] + [Sequence(f"{seq.seq_id}-{i}", seq.prompt_ids,
                                 dataclasses.replace(seq.params, seed=None if seq.params.seed is None else seq.params.seed + i),
                                 mm_items=seq.mm_items) for i in range(1, n_choices)]
        queues = [self.llm.submit(s) for s in seqs]
        queue = queues[0]
        if omni_view:
            try:
                return await self._omni_thinker_forward(seq, queue, xargs, rid, created, model)
            finally:
                await self._release(held_ids)
        include_usage = bool((body.get("stream_options") or {}).get("include_usage", False))
        want_logprobs = seq.params.logprobs >= 0

        def chunk(delta: dict[str, Any], finish: str | None = None, usage: dict | None = None, index: int = 0,
                  logprobs: dict | None = None) -> str:
            choice = {"index": index, "delta": delta, "finish_reason": finish}
            if logprobs is not None:
                choice["logprobs"] = logprobs
            payload = {"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                       "choices": [choice] if usage is None else []}
            if usage is not None:
                payload["usage"] = usage
            return f"data: {json.dumps(payload)}\n\n"

        def logprob_content(out: StepOutput) -> list[dict]:
            """OpenAI's ``logprobs.content`` entries of the tokens of one engine output."""
            def entry(tid: int, lp: float) -> dict:
                t = self.tokenizer.decode([tid])
                return {"token": t, "logprob": lp, "bytes": list(t.encode("utf-8"))}
            return [{**entry(tid, lp), "top_logprobs": [entry(i, v) for i, v in top]}
                    for tid, (lp, top) in zip(out.new_token_ids, out.logprobs or [])]

        stops = self._stops(body)
        hold = max((len(x) for x in stops), default=1) - 1   # characters that may still turn out to start a stop string
        first_left = [n_choices]   # choices that have not produced their first token yet (they all read the encoder rows)

        async def consume(idx: int = 0):
            """Yields (text_delta, engine output, tokens so far) per engine output of choice ``idx``.  With ``stop`` strings
            the text is cut before the first match, the request ends with reason ``stop`` and the sequence is taken out of
            the engine; the last ``hold`` characters are kept back until it is clear that they do not begin a stop string."""
            all_ids: list[int] = []
            emitted = ""
            stable_text, stable_ids = "", 0
            first = True
            finished = False
            my_seq, my_queue = seqs[idx], queues[idx]
            try:
                while True:
                    out: StepOutput = await my_queue.get()
                    if first:
                        first = False
                        first_left[0] -= 1
                        if idx == 0:
                            self.timing["first_token_ms"] += (time.perf_counter() - t_built) * 1e3   # queue + prefill
                        if first_left[0] == 0:
                            if recv_ids:
                                await self._release(recv_ids)  # the prompt embeddings were consumed by the prefill
                            if kv_in is not None:
                                await self._release_at_producer(kv_in)  # the pages were pulled before the first output
                    all_ids.extend(out.new_token_ids)
                    # detokenise only the tail: the text of ids[:stable_ids] is final; a few tokens before it give the
                    # tokenizer the context it needs (leading spaces, merges across the boundary)
                    ctx = max(0, stable_ids - 6)
                    lead = self.tokenizer.decode(all_ids[ctx:stable_ids]) if stable_ids else ""
                    tail = self.tokenizer.decode(all_ids[ctx:])[len(lead):]
                    text = stable_text + tail
                    if not tail.endswith("\ufffd"):
                        stable_text, stable_ids = text, len(all_ids)
                    if stops:
                        cut = min((i for i in (text.find(x, max(0, len(emitted) - hold)) for x in stops) if i >= 0), default=-1)
                        if cut >= 0:
                            finished = True
                            self.llm.abort(my_seq.seq_id)
                            yield text[len(emitted):cut], StepOutput(out.seq_id, out.new_token_ids, True, "stop",
                                                                     logprobs=out.logprobs), len(all_ids)
                            return
                    if text.endswith("\ufffd") and not out.finished:
                        delta = ""  # an incomplete multi-byte character: wait for the next token
                    elif stops and not out.finished:
                        safe = max(len(emitted), len(text) - hold)
                        delta, emitted = text[len(emitted):safe], text[:safe]
                    else:
                        delta, emitted = text[len(emitted):], text
                    yield delta, out, len(all_ids)
                    if out.finished:
                        finished = True
                        return
            finally:
                if not finished:
                    self.llm.abort(my_seq.seq_id)   # the client went away: free the sequence's pages
                if first:   # never produced a token: it no longer holds the release of the encoder rows back
                    first_left[0] -= 1
                    if first_left[0] == 0 and recv_ids:
                        await self._release(recv_ids)

        async def merged():
            """(choice index, text delta, engine output, tokens so far) of every choice, as they arrive."""
            if n_choices == 1:
                async for delta, out, cnt in consume(0):
                    yield 0, delta, out, cnt
                return
            sink: asyncio.Queue = asyncio.Queue()

            async def pump(i: int) -> None:
                try:
                    async for delta, out, cnt in consume(i):
                        await sink.put((i, delta, out, cnt))
                finally:
                    sink.put_nowait((i, None, None, 0))

            tasks = [asyncio.create_task(pump(i)) for i in range(n_choices)]
            live = n_choices
            try:
                while live:
                    i, delta, out, cnt = await sink.get()
                    if out is None:
                        live -= 1
                        continue
                    yield i, delta, out, cnt
            finally:
                for t in tasks:
                    t.cancel()

        if "cornserve_hidden_states_forward_id" in xargs:
            hidden = None
            async for _, out, _ in consume():
                hidden = out.hidden if out.finished else hidden
            if hidden is not None and self.sidecar is not None:
                ranks = ast.literal_eval(xargs.get("cornserve_hidden_states_forward_ranks", "[]")) or []
                if ranks:
                    self.sidecar.send(hidden.contiguous(), id=xargs["cornserve_hidden_states_forward_id"],
                                      dst_sidecar_ranks=ranks)
                    await asyncio.to_thread(self.sidecar.flush)
            return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model,
                                 "choices": [], "cornserve": {"hidden_states_rows": 0 if hidden is None else hidden.shape[0]}})

        if producer:
            text, last = "", None
            async for delta, last, _ in consume():
                text += delta
            if last is None or (last.finish_reason or "").startswith("error"):
                return JSONResponse({"error": {"message": getattr(last, "finish_reason", "no output")}}, status_code=500)
            held = await asyncio.wrap_future(self.llm.call(lambda: self.engine.kv_transfer_params(seq.seq_id)))
            params = {**self.kv_export(), **held}
            fid = xargs.get("cornserve_kv_transfer_params_forward_id")
            if fid and self.sidecar is not None:
                ranks = ast.literal_eval(xargs.get("cornserve_kv_transfer_params_forward_ranks", "[]")) or []
                if ranks:
                    self.sidecar.send(params, id=fid, dst_sidecar_ranks=ranks)
                    await asyncio.to_thread(self.sidecar.flush)
            return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model,
                                 "choices": [{"index": 0, "message": {"role": "assistant", "content": text},
                                              "finish_reason": "length"}],
                                 "usage": {"prompt_tokens": seq.prompt_len, "completion_tokens": 1,
                                           "total_tokens": seq.prompt_len + 1},
                                 "kv_transfer_params": params})

        if body.get("stream"):
            async def sse():
                # The role chunk goes out with the first generated token, so the arrival of the first chunk is the time
                # to first token; after that one chunk per engine output (a decode burst), even when its bytes do not yet
                # form a printable character, so clients see every step.
                counts, started = [0] * n_choices, set()
                async for i, delta, out, cnt in merged():
                    if out.finish_reason and out.finish_reason.startswith("error"):
                        yield f"data: {json.dumps({'error': out.finish_reason})}\n\n"
                        break
                    counts[i] = cnt
                    if i not in started:
                        started.add(i)
                        yield chunk({"role": "assistant", "content": ""}, index=i)
                    yield chunk({"content": delta}, out.finish_reason if out.finished else None, index=i,
                                logprobs={"content": logprob_content(out)} if want_logprobs else None)
                if include_usage:
                    yield chunk({}, usage={"prompt_tokens": seq.prompt_len, "completion_tokens": sum(counts),
                                           "total_tokens": seq.prompt_len + sum(counts)})
                yield "data: [DONE]\n\n"

            return StreamingResponse(sse(), media_type="text/event-stream")

        texts, reasons, counts = [""] * n_choices, [None] * n_choices, [0] * n_choices
        lps: list[list[dict]] = [[] for _ in range(n_choices)]
        async for i, delta, out, cnt in merged():
            texts[i] += delta
            reasons[i], counts[i] = out.finish_reason, cnt
            if want_logprobs:
                lps[i].extend(logprob_content(out))
        bad = next((r for r in reasons if r and r.startswith("error")), None)
        if bad:
            return JSONResponse({"error": {"message": bad}}, status_code=500)
        choices = [{"index": i, "message": {"role": "assistant", "content": texts[i]}, "finish_reason": reasons[i],
                    **({"logprobs": {"content": lps[i]}} if want_logprobs else {})} for i in range(n_choices)]
        return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model,
                             "choices": choices,
                             "usage": {"prompt_tokens": seq.prompt_len, "completion_tokens": sum(counts),
                                       "total_tokens": seq.prompt_len + sum(counts)},
                             **({"cornserve": {"kv_source": seq.kv_source}} if kv_in is not None else {})})

    def create_app(self) -> FastAPI:
        app = FastAPI(title="cornserve-b200 LLM executor")
        from ...tracing import instrument_fastapi

        instrument_fastapi(app, "cornserve.llm")

        @app.get("/health")
        async def health():
            return Response(status_code=200 if self.llm.alive else 503)

        @app.get("/stats")
        async def stats():
            """Counters of this executor since it started (rank 0 of a tensor-parallel group; the other ranks launch
            the same kernels): this library's kernel launches, launches per fused path, engine steps and their time."""
            eng = self.engine
            return {"executor": "llm", "tp_size": int(self.args.tensor_parallel_size), "kernel_launches": ops.kernel_launches(),
                    "paths": ops.path_counts(), **eng.stats, "running": len(eng.running), "waiting": len(eng.waiting),
                    "kv_pages": eng.cfg.num_pages, "kv_pages_free": eng.blocks.num_free,
                    "d2h_bytes": 4 * (eng.stats["decode_tokens"] + eng.stats["prefill_steps"]),
                    "tp_publish_ms": getattr(self.llm.tp, "publish_ms", 0.0) if self.llm.tp is not None else 0.0,
                    **self.timing,
                    "h2d_bytes": self.local_encoder.h2d_bytes if self.local_encoder is not None else 0,
                    "local_encoder_ms": self.local_encoder.busy_ms if self.local_encoder is not None else 0.0,
                    "local_encoder_host_ms": self.local_encoder.host_ms if self.local_encoder is not None else 0.0,
                    "local_encoder_wait_ms": self.local_encoder.wait_ms if self.local_encoder is not None else 0.0,
                    "alloc_retries": int(torch.cuda.memory_stats(eng.device).get("num_alloc_retries", 0)) if eng.on_gpu else 0,
                    "device_allocs": int(torch.cuda.memory_stats(eng.device).get("num_device_alloc", 0)) if eng.on_gpu else 0,
                    "local_encoder_images": self.local_encoder.images if self.local_encoder is not None else 0,
                    "local_encoder_batches": self.local_encoder.batches if self.local_encoder is not None else 0,
                    "stack_samples": sampler_report()}

        @app.get("/v1/models")
        async def models():
            return {"object": "list", "data": [{"id": self.args.model, "object": "model"}]}

        @app.post("/v1/chat/completions")
        async def chat(raw: Request):
            return await self.chat(await raw.json())

        from ..device_timer import add_timer_routes

        add_timer_routes(app, self.engine.device)

        @app.post("/kv/release")
        async def kv_release(raw: Request):
            rid = (await raw.json())["request_id"]
            ok = await asyncio.wrap_future(self.llm.call(lambda: self.engine.release_held(rid)))
            return {"released": bool(ok)}

        @app.post("/kv/pages")
        async def kv_pages(raw: Request):
            rid = (await raw.json())["request_id"]

            def read() -> bytes | None:
                if rid not in self.engine.held:
                    return None
                pages = self.engine.kv_transfer_params(rid)["pages"]
                return self.engine.read_pages(pages).contiguous().view(torch.uint8).numpy().tobytes()

            data = await asyncio.wrap_future(self.llm.call(read))
            if data is None:
                return JSONResponse({"error": {"message": f"no held pages for {rid}"}}, status_code=404)
            return Response(content=data, media_type="application/octet-stream")

        return app

    def shutdown(self) -> None:
        self.llm.shutdown()
        for p in self.followers:
            try:
                p.wait(timeout=10)
            except Exception:  # noqa: BLE001
                p.kill()
        if self.sidecar is not None:
            self.sidecar.shutdown_sync()


def follower_main(args: argparse.Namespace) -> None:
    """A further tensor-parallel rank: no HTTP server, no sidecar; it mirrors rank 0's engine steps."""
    from . import tp as tpmod

    group = tpmod.join_group(args.tp_rank, int(args.tensor_parallel_size), args.tp_port)
    engine, _ = build_engine(args, group)
    ops.bind_thread(engine.device)
    control = tpmod.TPControl(group, next(engine.model.parameters()).dtype)
    logger.info("tensor-parallel rank %d of %d is ready", args.tp_rank, group.size)
    tpmod.follower_loop(engine, control)


def main(argv: list[str] | None = None) -> None:
    args = parse_args(argv)
    args.argv = list(argv) if argv is not None else sys.argv[1:]
    tune_interpreter()
    if args.tp_rank > 0:
        follower_main(args)
        return
    configure_otel("llm")
    maybe_start_sampler()
    if args.run_talker:
        from .talker_server import TalkerServer

        server = TalkerServer(args)
    else:
        server = LLMServer(args)
    try:
        uvicorn.run(server.create_app(), host=args.host, port=args.port, log_level="warning")
    finally:
        server.shutdown()


if __name__ == "__main__":
    main()
