#!/usr/bin/env python
"""Reference arm of ``bench.py``: the reference's own encoder code in front of stock vLLM, as one small server.

Nothing here imports this repository's package: the interpreter is started with ``-P`` and a ``PYTHONPATH`` that holds
the reference (installed unmodified under ``baseline/_ref``), so ``import cornserve`` below is the reference.

Why a server of its own: the reference's control plane needs a Kubernetes API server and its executor processes
import gRPC bindings that its build generates with ``grpc_tools`` (not available offline), so its gateway, task
dispatcher, sidecar servers and ``eric.executor`` worker wrappers cannot start here.  What does run unmodified is the
code those wrappers call:

* encoder: ``cornserve.task_executors.eric.models.qwen2_5_vl`` - ``ModalityProcessor`` (the Hugging Face image
  processor on CPU threads, as its router does) and ``Qwen2_5_VisionTransformer`` with its own tensor-parallel layers
  over NCCL (``eric.distributed.parallel``), one item per forward pass (the reference's default ``max_batch_size``);
* hand-over: the embeddings are copied GPU -> a ``torch.from_file(shared=True)`` buffer on a side stream and the
  consumer reads that buffer, which is what its sidecar does on one node (services/sidecar/sender.py:498-575,
  sidecar/utils.py:28-65);
* LLM: stock vLLM (the reference's fork is an empty submodule) started with the flags of the reference's descriptor
  (``--tensor-parallel-size N --enforce-eager --no-enable-prefix-caching --gpu-memory-utilization 0.93``,
  ``--max-num-seqs 256`` from its profile), random (``dummy``) weights of the Qwen2.5-VL-7B decoder, prompts given as
  embeddings (encoder rows + text rows), greedy, ``ignore_eos``.

Processes: this front (HTTP, round robin over replicas), per encoder replica ``tp`` worker processes, per LLM replica
one process that hosts vLLM's ``AsyncLLM`` (which starts its own engine and worker processes).  The front speaks the
request / chunk format of the load generator, so both arms are driven by the same client.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import subprocess
import sys
import threading
import time
import uuid
from concurrent.futures import ThreadPoolExecutor
from multiprocessing.connection import Client, Listener
from pathlib import Path

AUTH = b"cornserve-reference-arm"
HIDDEN = 3584
VISION_7B = dict(depth=32, hidden_size=1280, num_heads=16, intermediate_size=3420, out_hidden_size=HIDDEN,
                 fullatt_block_indexes=[7, 15, 23, 31], window_size=112, patch_size=14, spatial_merge_size=2,
                 temporal_patch_size=2, hidden_act="silu", in_channels=3)
DECODER_7B = {"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": HIDDEN, "intermediate_size": 18944,
              "num_attention_heads": 28, "num_key_value_heads": 4, "num_hidden_layers": 28, "vocab_size": 152064,
              "max_position_embeddings": 32768, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "tie_word_embeddings": False,
              "torch_dtype": "bfloat16", "hidden_act": "silu", "bos_token_id": 151643, "eos_token_id": 151645,
              "use_sliding_window": False, "sliding_window": None, "attention_dropout": 0.0, "initializer_range": 0.02,
              "use_cache": True}
PREPROCESSOR = {"image_processor_type": "Qwen2VLImageProcessor", "min_pixels": 3136, "max_pixels": 12845056, "patch_size": 14,
                "temporal_patch_size": 2, "merge_size": 2, "image_mean": [0.48145466, 0.4578275, 0.40821073],
                "image_std": [0.26862954, 0.26130258, 0.27577711], "do_resize": True, "do_rescale": True, "do_normalize": True,
                "do_convert_rgb": True}
VLLM_FLAGS = "--tensor-parallel-size {tp} --trust-remote-code --enforce-eager --no-enable-prefix-caching --gpu-memory-utilization {util} --max-num-seqs 256 --load-format dummy --enable-prompt-embeds"


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", default="front", choices=["front", "encoder", "llm"])
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--encoder-tp", type=int, default=1)
    ap.add_argument("--llm-tp", type=int, default=1)
    ap.add_argument("--replicas", type=int, default=1)
    ap.add_argument("--share-gpu", action="store_true", help="one GPU: encoder and vLLM share it")
    ap.add_argument("--workdir", default=".")
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--prompt-tokens", type=int, default=128)
    ap.add_argument("--small", action="store_true", help="tiny decoder and tower: a plumbing run")
    ap.add_argument("--encoder-batch", type=int, default=1,
                    help="images per tower call at most (the reference's EncoderTask.max_batch_size; its default is 1)")
    # worker roles
    ap.add_argument("--replica", type=int, default=0)
    ap.add_argument("--rank", type=int, default=0)
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("--init-port", type=int, default=0)
    ap.add_argument("--front-port", type=int, default=0)
    ap.add_argument("--slab", default="")
    ap.add_argument("--slab-bytes", type=int, default=0)
    ap.add_argument("--gpu-util", type=float, default=0.93)
    return ap.parse_args()


def synthetic_image(url: str):
    """``synthetic:<H>x<W>[:seed]`` -> uniform random RGB uint8 (the same generator as the other arm's loader)."""
    import numpy as np

    spec = url.split(":")
    h, w = (int(v) for v in spec[1].split("x"))
    rng = np.random.default_rng(int(spec[2]) if len(spec) > 2 else 0)
    return rng.integers(0, 256, (h, w, 3), dtype=np.uint8)


# ----------------------------------------------------------------------------------------------------------------------
# encoder worker: the reference's processor + vision tower
# ----------------------------------------------------------------------------------------------------------------------
def encoder_main(a: argparse.Namespace) -> None:
    import queue

    import torch
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLConfig

    from cornserve.task_executors.eric.distributed import parallel   # the reference package
    from cornserve.task_executors.eric.models import qwen2_5_vl as ref

    parallel.init_distributed(world_size=a.world, rank=a.rank, init_method=f"tcp://127.0.0.1:{a.init_port}")
    vision = dict(VISION_7B)
    if a.small:
        vision.update(depth=2, hidden_size=128, num_heads=4, intermediate_size=256, fullatt_block_indexes=[1], out_hidden_size=256)
    torch.manual_seed(0)
    tower = ref.Qwen2_5_VisionTransformer(Qwen2_5_VLConfig(vision_config=vision)).to(device="cuda", dtype=torch.bfloat16).eval()
    Modality = ref.Modality

    def forward(pixel_values: list, grids: list) -> list:
        """One call of the reference's tower on a batch of images (lists, as its scheduler hands them over)."""
        with torch.inference_mode():
            return tower(Modality.IMAGE, "", {"pixel_values": list(pixel_values), "image_grid_thw": list(grids)})

    def share(pixel_values: list, grids: list) -> list:
        """Rank 0 of a tensor-parallel group: hand the batch to the other ranks.  Shapes go as a small pickled message,
        the pixels as device tensors over NCCL (the reference moves them through a shared-memory ring; pickling 20 MB
        per image through ``broadcast_object_list`` would make this arm slower than what it stands for)."""
        meta = [(tuple(pv.shape), str(pv.dtype).split(".")[-1], g.tolist()) for pv, g in zip(pixel_values, grids)]
        torch.distributed.broadcast_object_list([meta], src=0)
        on_device = [pv.to("cuda") for pv in pixel_values]
        for t in on_device:
            torch.distributed.broadcast(t, src=0)
        return on_device

    if a.rank > 0:   # follower of a tensor-parallel group: replay what rank 0 broadcasts
        while True:
            box = [None]
            torch.distributed.broadcast_object_list(box, src=0)
            if box[0] is None:
                return
            pvs, grids = [], []
            for shape, dtype, grid in box[0]:
                t = torch.empty(shape, dtype=getattr(torch, dtype), device="cuda")
                torch.distributed.broadcast(t, src=0)
                pvs.append(t)
                grids.append(torch.tensor(grid))
            forward(pvs, grids)

    print(f"encoder replica {a.replica} rank {a.rank}: tower on {torch.cuda.get_device_name()}", flush=True)
    processor = ref.ModalityProcessor(str(Path(a.workdir) / "encoder_model"))
    slab = torch.from_file(a.slab, shared=True, size=a.slab_bytes, dtype=torch.uint8)
    copy_stream = torch.cuda.Stream()
    conn = Client(("127.0.0.1", a.front_port), authkey=AUTH)
    send_lock = threading.Lock()
    ready: queue.Queue = queue.Queue()
    pool = ThreadPoolExecutor(max_workers=12)   # the reference's ModalityConfig.num_workers
    free_list = [(0, a.slab_bytes)]             # first-fit allocator over the shared buffer: (offset, bytes)
    held: dict[str, tuple[int, int]] = {}
    alloc_lock = threading.Lock()
    stats = {"h2d_bytes": 0, "d2h_bytes": 0, "items": 0, "busy_ms": 0.0}

    def allocate(n: int) -> int | None:
        with alloc_lock:
            for i, (off, size) in enumerate(free_list):
                if size >= n:
                    free_list[i] = (off + n, size - n)
                    return off
        return None

    def release(item_id: str) -> None:
        with alloc_lock:
            blk = held.pop(item_id, None)
            if blk is None:
                return
            free_list.append(blk)
            free_list.sort()
            merged = [free_list[0]]
            for off, size in free_list[1:]:
                lo, sz = merged[-1]
                if lo + sz == off:
                    merged[-1] = (lo, sz + size)
                else:
                    merged.append((off, size))
            free_list[:] = merged

    def load(item_id: str, url: str) -> None:
        try:
            ready.put((item_id, processor.process(Modality.IMAGE, synthetic_image(url))))
        except Exception as e:  # noqa: BLE001
            ready.put((item_id, e))

    def reader() -> None:
        while True:
            try:
                msg = conn.recv()
            except (EOFError, OSError):
                ready.put(None)
                return
            if msg[0] == "enc":
                pool.submit(load, msg[1], msg[2])
            elif msg[0] == "free":
                for item_id in msg[1]:
                    release(item_id)
            elif msg[0] == "stats":
                with send_lock:
                    conn.send(("stats", dict(stats)))
            elif msg[0] == "stop":
                ready.put(None)
                return

    threading.Thread(target=reader, daemon=True).start()
    with send_lock:
        conn.send(("hello", "encoder", a.replica))
    stop = False
    while not stop:
        item = ready.get()
        if item is None:
            break
        batch = [item]
        while len(batch) < max(1, a.encoder_batch):   # whatever else is ready, up to the batch limit (first come, first served)
            try:
                more = ready.get_nowait()
            except queue.Empty:
                break
            if more is None:
                stop = True
                break
            batch.append(more)
        good = []
        for item_id, data in batch:
            if isinstance(data, Exception):
                with send_lock:
                    conn.send(("error", item_id, repr(data)))
            else:
                good.append((item_id, data))
        if not good:
            continue
        t0 = time.perf_counter()
        pvs = [d["pixel_values"] for _, d in good]
        grids = [d["image_grid_thw"] for _, d in good]
        stats["h2d_bytes"] += sum(pv.numel() * pv.element_size() for pv in pvs)
        if a.world > 1:
            pvs = share(pvs, grids)
        outs = forward(pvs, grids)
        for (item_id, _), out in zip(good, outs):
            out = out.contiguous()
            nbytes = out.numel() * out.element_size()
            off = allocate(nbytes)
            while off is None:   # back-pressure: wait for the consumer to release rows
                time.sleep(0.002)
                off = allocate(nbytes)
            held[item_id] = (off, nbytes)
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_stream(torch.cuda.current_stream())
                slab[off: off + nbytes].view(torch.bfloat16).view(out.shape).copy_(out, non_blocking=True)
            copy_stream.synchronize()
            stats["d2h_bytes"] += nbytes
            stats["items"] += 1
            with send_lock:
                conn.send(("done", item_id, off, int(out.shape[0])))
        stats["busy_ms"] += (time.perf_counter() - t0) * 1e3
        stats["batches"] = stats.get("batches", 0) + 1
    if a.world > 1:
        torch.distributed.broadcast_object_list([None], src=0)


# ----------------------------------------------------------------------------------------------------------------------
# LLM worker: stock vLLM
# ----------------------------------------------------------------------------------------------------------------------
def llm_main(a: argparse.Namespace) -> None:
    import torch
    from vllm import SamplingParams
    from vllm.engine.arg_utils import AsyncEngineArgs
    from vllm.sampling_params import RequestOutputKind
    from vllm.v1.engine.async_llm import AsyncLLM

    hidden = 256 if a.small else HIDDEN
    # Attention backend: vLLM's own choice first ("auto": FlashInfer on sm_100).  FlashInfer compiles helper kernels
    # with nvcc at the first start; if that takes longer than REF_VLLM_START_TIMEOUT_S on a box without its cache, the
    # next entries of vLLM's own priority list are tried: FLASH_ATTN (precompiled in the wheel), then Triton attention.
    wanted = os.environ.get("REF_VLLM_ATTENTION_BACKEND", "auto,FLASH_ATTN,TRITON_ATTN").split(",")
    start_limit = float(os.environ.get("REF_VLLM_START_TIMEOUT_S", "150"))
    engine, last = None, None

    def give_up_on_children(done: threading.Event, backend: str) -> None:
        """An engine process that has not come up in time is asked to abort (with PYTHONFAULTHANDLER set it leaves the
        stacks of its threads in this log), so that the next backend can be tried."""
        if done.wait(start_limit):
            return
        import signal

        import psutil

        print(f"llm replica {a.replica}: vLLM with attention backend {backend} is not up after {start_limit:.0f} s; aborting its processes",
              flush=True)
        for child in psutil.Process().children(recursive=True):
            try:
                child.send_signal(signal.SIGABRT)
            except psutil.Error:
                pass

    for backend in wanted:
        kw = {} if backend == "auto" else {"attention_backend": backend}
        done = threading.Event()
        threading.Thread(target=give_up_on_children, args=(done, backend), daemon=True).start()
        try:
            engine = AsyncLLM.from_engine_args(AsyncEngineArgs(
                model=str(Path(a.workdir) / "decoder_model"), tensor_parallel_size=a.world, enforce_eager=True,
                enable_prefix_caching=False, gpu_memory_utilization=a.gpu_util, max_num_seqs=256, load_format="dummy",
                enable_prompt_embeds=True, skip_tokenizer_init=True, trust_remote_code=True, dtype="bfloat16",
                generation_config="vllm", max_model_len=8192, disable_log_stats=True, enable_flashinfer_autotune=False, **kw))
            done.set()
            print(f"llm replica {a.replica}: vLLM started with attention backend {backend}", flush=True)
            break
        except BaseException as e:  # noqa: BLE001
            done.set()
            last = e
            print(f"llm replica {a.replica}: attention backend {backend} did not start: {type(e).__name__}: {e}", flush=True)
    if engine is None:
        raise RuntimeError(f"vLLM did not start with any of {wanted}: {last}")
    # (after the engine: vLLM may fork its engine process, and a forked child of a process that has already run
    # multi-threaded CPU kernels of torch deadlocks in its first one)
    slabs = {i: torch.from_file(p, shared=True, size=a.slab_bytes, dtype=torch.uint8) for i, p in enumerate(a.slab.split(","))}
    text_rows = (torch.randn(4096, hidden, generator=torch.Generator().manual_seed(1)) * 0.02).to(torch.bfloat16)
    print(f"llm replica {a.replica}: engine ready", flush=True)
    conn = Client(("127.0.0.1", a.front_port), authkey=AUTH)
    send_lock = threading.Lock()
    stats = {"h2d_bytes": 0, "d2h_bytes": 0, "requests": 0}

    def send(msg) -> None:
        with send_lock:
            conn.send(msg)

    async def handle(req_id: str, refs: list[tuple[int, int, int]], n_text: int, max_tokens: int) -> None:
        try:
            rows = [slabs[s][off: off + n * hidden * 2].view(torch.bfloat16).view(n, hidden) for s, off, n in refs]
            embeds = torch.cat([*rows, text_rows[:n_text]])   # the consumer's copy out of the shared buffer
            send(("consumed", req_id))
            stats["h2d_bytes"] += embeds.numel() * 2
            stats["requests"] += 1
            sp = SamplingParams(max_tokens=max_tokens, ignore_eos=True, temperature=0.0, detokenize=False,
                                output_kind=RequestOutputKind.DELTA)
            async for out in engine.generate({"prompt_embeds": embeds}, sp, req_id):
                n = sum(len(c.token_ids) for c in out.outputs)
                stats["d2h_bytes"] += 4 * n
                send(("tok", req_id, n, bool(out.finished)))
        except Exception as e:  # noqa: BLE001
            send(("error", req_id, repr(e)))

    async def main() -> None:
        loop = asyncio.get_running_loop()
        stop = asyncio.Event()

        def reader() -> None:
            while True:
                try:
                    msg = conn.recv()
                except (EOFError, OSError):
                    loop.call_soon_threadsafe(stop.set)
                    return
                if msg[0] == "gen":
                    asyncio.run_coroutine_threadsafe(handle(*msg[1:]), loop)
                elif msg[0] == "stats":
                    send(("stats", dict(stats)))
                elif msg[0] == "stop":
                    loop.call_soon_threadsafe(stop.set)
                    return

        threading.Thread(target=reader, daemon=True).start()
        send(("hello", "llm", a.replica))
        await stop.wait()

    asyncio.run(main())
    engine.shutdown()


# ----------------------------------------------------------------------------------------------------------------------
# front: HTTP, routing, bookkeeping
# ----------------------------------------------------------------------------------------------------------------------
class Worker:
    def __init__(self, conn, role: str, replica: int, loop: asyncio.AbstractEventLoop, front: "Front"):
        self.conn, self.role, self.replica, self.loop, self.front = conn, role, replica, loop, front
        self.lock = threading.Lock()
        threading.Thread(target=self._read, daemon=True).start()

    def send(self, msg) -> None:
        with self.lock:
            self.conn.send(msg)

    def _read(self) -> None:
        while True:
            try:
                msg = self.conn.recv()
            except (EOFError, OSError):
                return
            self.loop.call_soon_threadsafe(self.front.on_message, self, msg)


class Front:
    def __init__(self, a: argparse.Namespace):
        self.a = a
        self.encoders: dict[int, Worker] = {}
        self.llms: dict[int, Worker] = {}
        self.item_futures: dict[str, asyncio.Future] = {}
        self.token_queues: dict[str, asyncio.Queue] = {}
        self.stats_futures: list[asyncio.Future] = []
        self.rr = 0
        self.procs: list[subprocess.Popen] = []
        self.marks: list = []
        self.counters = {"requests": 0}

    def on_message(self, w: Worker, msg) -> None:
        kind = msg[0]
        if kind == "done":
            fut = self.item_futures.pop(msg[1], None)
            if fut is not None and not fut.done():
                fut.set_result((w.replica, msg[2], msg[3]))
        elif kind in ("tok", "consumed"):
            q = self.token_queues.get(msg[1])
            if q is not None:
                q.put_nowait(msg)
        elif kind == "error":
            fut = self.item_futures.pop(msg[1], None)
            if fut is not None and not fut.done():
                fut.set_exception(RuntimeError(msg[2]))
            q = self.token_queues.get(msg[1])
            if q is not None:
                q.put_nowait(msg)
        elif kind == "stats":
            for f in self.stats_futures:
                if not f.done() and getattr(f, "worker", None) is w:
                    f.set_result(msg[1])
                    break

    def spawn(self, listener_port: int) -> None:
        a = self.a
        work = Path(a.workdir)
        (work / "encoder_model").mkdir(parents=True, exist_ok=True)
        (work / "encoder_model" / "preprocessor_config.json").write_text(json.dumps(PREPROCESSOR))
        (work / "decoder_model").mkdir(parents=True, exist_ok=True)
        dec = dict(DECODER_7B)
        if a.small:
            dec.update(hidden_size=256, intermediate_size=512, num_attention_heads=4, num_key_value_heads=2, num_hidden_layers=2, vocab_size=1024)
        (work / "decoder_model" / "config.json").write_text(json.dumps(dec))
        shm_root = Path("/dev/shm") if Path("/dev/shm").is_dir() else work
        slab_bytes = (256 << 20) if a.small else (4 << 30)
        slabs = []
        for r in range(a.replicas):
            p = shm_root / f"cornserve_ref_{os.getpid()}_{r}"
            with open(p, "wb") as f:
                f.truncate(slab_bytes)
            slabs.append(str(p))
        self.slab_paths = slabs
        base = [sys.executable, "-P", str(Path(__file__).resolve()), "--workdir", a.workdir, "--front-port", str(listener_port),
                "--slab-bytes", str(slab_bytes), "--encoder-batch", str(a.encoder_batch)] + (["--small"] if a.small else [])
        et, lt, R = a.encoder_tp, a.llm_tp, a.replicas
        import socket

        for r in range(R):
            with socket.socket() as s:
                s.bind(("127.0.0.1", 0))
                init_port = s.getsockname()[1]
            gpus = "0" if a.share_gpu else ",".join(str(r * et + i) for i in range(et))
            for k in range(et):
                env = dict(os.environ, CUDA_VISIBLE_DEVICES=gpus, GLOO_SOCKET_IFNAME="lo", NCCL_SOCKET_IFNAME="lo")
                log = open(work / f"encoder_{r}_{k}.log", "w")
                self.procs.append(subprocess.Popen(base + ["--role", "encoder", "--replica", str(r), "--rank", str(k), "--world", str(et),
                                                           "--init-port", str(init_port), "--slab", slabs[r]], env=env, stdout=log, stderr=subprocess.STDOUT))
        for r in range(R):
            gpus = "0" if a.share_gpu else ",".join(str(R * et + r * lt + i) for i in range(lt))
            # no network here: vLLM must not look for its address through a route to the outside or a host name that
            # does not resolve (its torch.distributed rendezvous then waits for ever)
            env = dict(os.environ, CUDA_VISIBLE_DEVICES=gpus, VLLM_HOST_IP="127.0.0.1", GLOO_SOCKET_IFNAME="lo", NCCL_SOCKET_IFNAME="lo",
                       VLLM_LOGGING_LEVEL="INFO", MASTER_ADDR="127.0.0.1", VLLM_USE_FLASHINFER_SAMPLER="0", PYTHONFAULTHANDLER="1",
                       VLLM_WORKER_MULTIPROC_METHOD="spawn")
            log = open(work / f"llm_{r}.log", "w")
            util = 0.80 if a.share_gpu else 0.93
            self.procs.append(subprocess.Popen(base + ["--role", "llm", "--replica", str(r), "--world", str(lt), "--slab", ",".join(slabs),
                                                       "--gpu-util", str(util)], env=env, stdout=log, stderr=subprocess.STDOUT))
        self.vllm_flags = VLLM_FLAGS.format(tp=lt, util=0.80 if a.share_gpu else 0.93)

    def ready(self) -> bool:
        return len(self.encoders) == self.a.replicas and len(self.llms) == self.a.replicas

    def dead(self) -> str | None:
        for p in self.procs:
            if p.poll() is not None:
                return f"a worker exited with code {p.returncode}"
        return None

    async def worker_stats(self) -> dict:
        total = {"h2d_bytes": 0, "d2h_bytes": 0}
        for w in [*self.encoders.values(), *self.llms.values()]:
            f = asyncio.get_running_loop().create_future()
            f.worker = w
            self.stats_futures.append(f)
            w.send(("stats",))
            s = await asyncio.wait_for(f, 30)
            self.stats_futures.remove(f)
            for k in total:
                total[k] += s.get(k, 0)
        return total

    async def invoke(self, request):
        from aiohttp import web

        body = await request.json()
        data = body.get("request_data", body)
        urls = [u for kind, u in data.get("multimodal_data", []) if kind == "image"]
        max_tokens = int(data.get("max_completion_tokens", self.a.max_tokens))
        req_id = uuid.uuid4().hex
        self.rr += 1
        enc = self.encoders[self.rr % len(self.encoders)]
        llm = self.llms[self.rr % len(self.llms)]
        loop = asyncio.get_running_loop()
        items = []
        for k, url in enumerate(urls):
            item_id = f"{req_id}-{k}"
            self.item_futures[item_id] = loop.create_future()
            items.append((item_id, self.item_futures[item_id]))
            enc.send(("enc", item_id, url))
        q: asyncio.Queue = asyncio.Queue()
        self.token_queues[req_id] = q
        resp = web.StreamResponse(headers={"Content-Type": "text/plain"})
        await resp.prepare(request)
        try:
            refs = [await f for _, f in items]
            llm.send(("gen", req_id, refs, self.a.prompt_tokens, max_tokens))
            sent = 0
            while True:
                msg = await q.get()
                if msg[0] == "consumed":
                    enc.send(("free", [i for i, _ in items]))
                    continue
                if msg[0] == "error":
                    await resp.write((json.dumps({"error": msg[2]}) + "\n").encode())
                    break
                _, _, n, finished = msg
                sent += n
                chunk = {"object": "chat.completion.chunk", "choices": [{"index": 0, "delta": {"content": ""},
                                                                       "finish_reason": "length" if finished else None}]}
                await resp.write((json.dumps(chunk) + "\n").encode())
                if finished:
                    break
            self.counters["requests"] += 1
        except Exception as e:  # noqa: BLE001
            await resp.write((json.dumps({"error": repr(e)}) + "\n").encode())
        finally:
            self.token_queues.pop(req_id, None)
        await resp.write_eof()
        return resp


def front_main(a: argparse.Namespace) -> None:
    import torch
    from aiohttp import web

    front = Front(a)
    listener = Listener(("127.0.0.1", 0), authkey=AUTH)
    front.spawn(listener.address[1])

    async def main() -> None:
        loop = asyncio.get_running_loop()

        def accept() -> None:
            while True:
                try:
                    conn = listener.accept()
                    hello = conn.recv()
                except Exception:  # noqa: BLE001
                    return
                w = Worker(conn, hello[1], hello[2], loop, front)
                (front.encoders if hello[1] == "encoder" else front.llms)[hello[2]] = w

        threading.Thread(target=accept, daemon=True).start()

        async def health(_):
            why = front.dead()
            if why:
                return web.Response(status=500, text=why)
            return web.Response(status=200 if front.ready() else 503)

        async def stats(_):
            s = await front.worker_stats()
            return web.json_response({"executor": "reference", "tp_size": 1, "kernel_launches": 0, "paths": {}, **s,
                                      "requests": front.counters["requests"], "vllm_flags": front.vllm_flags,
                                      "reference_class": "cornserve.task_executors.eric.models.qwen2_5_vl.{ModalityProcessor,Qwen2_5_VisionTransformer} "
                                                         "-> shared-memory buffer -> stock vLLM " + _vllm_version()})

        async def mark(_):
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.default_stream())
            front.marks.append(ev)
            return web.json_response({"mark": len(front.marks) - 1})

        async def elapsed(request):
            s, e = int(request.query["start"]), int(request.query["end"])
            front.marks[e].synchronize()
            return web.json_response({"ms": float(front.marks[s].elapsed_time(front.marks[e])), "device": "cuda:0"})

        app = web.Application(client_max_size=1 << 26)
        app.add_routes([web.get("/health", health), web.get("/stats", stats), web.post("/timer/mark", mark),
                        web.get("/timer/elapsed", elapsed), web.post("/app/invoke/reference", front.invoke)])
        runner = web.AppRunner(app, access_log=None)
        await runner.setup()
        await web.TCPSite(runner, "127.0.0.1", a.port).start()
        stop = asyncio.Event()
        import signal

        for s in (signal.SIGINT, signal.SIGTERM):
            loop.add_signal_handler(s, stop.set)
        await stop.wait()
        await runner.cleanup()

    try:
        torch.cuda.init()   # the front's own context on GPU 0 only records the timing events
        asyncio.run(main())
    finally:
        for w in [*front.encoders.values(), *front.llms.values()]:
            try:
                w.send(("stop",))
            except Exception:  # noqa: BLE001
                pass
        deadline = time.time() + 20
        for p in front.procs:
            try:
                p.wait(timeout=max(0.1, deadline - time.time()))
            except Exception:  # noqa: BLE001
                p.kill()
        for p in getattr(front, "slab_paths", []):
            try:
                os.unlink(p)
            except OSError:
                pass


def _vllm_version() -> str:
    try:
        from importlib.metadata import version

        return version("vllm")
    except Exception:  # noqa: BLE001
        return "?"


def exit_with_parent() -> None:
    """REF_EXIT_WITH_PARENT=1 (set by bench.py, inherited by the workers): leave when the starting process is gone, so
    that a run that was killed does not leave vLLM holding its GPUs."""
    if os.environ.get("REF_EXIT_WITH_PARENT") != "1":
        return
    parent = os.getppid()

    def watch() -> None:
        while True:
            time.sleep(1.0)
            if os.getppid() != parent:
                try:   # vLLM's engine-core and worker processes are this process's own children
                    import psutil

                    for child in psutil.Process().children(recursive=True):
                        child.kill()
                except Exception:  # noqa: BLE001
                    pass
                os._exit(113)

    threading.Thread(target=watch, name="exit-with-parent", daemon=True).start()


if __name__ == "__main__":
    args = parse_args()
    exit_with_parent()
    {"front": front_main, "encoder": encoder_main, "llm": llm_main}[args.role](args)
