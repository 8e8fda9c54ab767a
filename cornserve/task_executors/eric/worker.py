"""Encoder worker: one per GPU of the executor's tensor-parallel group.

Loads the model shard, turns decoded inputs into model tensors on the device, runs the forward pass and
hands every item's embeddings to the sidecar (reference: python/cornserve/task_executors/eric/executor/
worker.py:59-405).  Rank 0 lives in the executor's main process next to the engine; ranks > 0 are
separate processes that replay the batches rank 0 broadcasts.
"""

from __future__ import annotations

import os
import time
from pathlib import Path

import torch

from ...logging import get_logger
from ...parallel.state import ParallelGroup, init_distributed, set_tp_group
from ...sidecar.api import Sidecar
from ...sidecar.schema import SidecarConfig
from ...tracing import extract, get_tracer
from ...utils.hub import load_config, load_model_weights
from .config import EricConfig
from .preprocess import (HALF, IMAGENET_MEAN, IMAGENET_STD, anyres_tiles, dynamic_tiles, log_mel_spectrogram,
                         patchify_frames, resize_normalize)
from .registry import MODEL_REGISTRY
from .schema import Batch

logger = get_logger(__name__)
tracer = get_tracer(__name__)


def pick_device(local_index: int) -> torch.device:
    if not torch.cuda.is_available() or os.environ.get("CORNSERVE_DEVICE") == "cpu":
        return torch.device("cpu")
    ids = [int(x) for x in os.environ.get("CORNSERVE_LOCAL_GPUS", "").split(",") if x.strip() != ""]
    return torch.device("cuda", ids[local_index] if ids else local_index)


class Worker:
    def __init__(self, config: EricConfig, tp_rank: int = 0, group: ParallelGroup | None = None):
        self.config = config
        self.tp_rank = tp_rank
        self.device = group.device if group is not None else pick_device(tp_rank)
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        self.group = group or ParallelGroup(0, 1, None, None, self.device)
        set_tp_group(self.group)
        hf_cfg = load_config(config.model.id)
        model_type = hf_cfg.get("model_type", "")
        if model_type not in MODEL_REGISTRY:
            raise ValueError(f"Model type {model_type!r} is not supported by the encoder executor "
                             f"(supported: {sorted(MODEL_REGISTRY)})")
        self.entry = MODEL_REGISTRY[model_type]
        if config.model.modality not in self.entry.modalities:
            raise ValueError(f"{model_type} does not encode {config.model.modality}")
        model_cls, cfg_cls = self.entry.load_classes()
        self.model_cfg = cfg_cls.from_hf(hf_cfg)
        dtype = torch.float32 if self.device.type == "cpu" else torch.bfloat16  # the CUDA kernels are bf16
        torch.manual_seed(int(os.environ.get("CORNSERVE_SEED", "0")))  # reproducible random-weight runs
        kw = {"model_id": config.model.id} if self.entry.adapter_attr else {}
        self.model = model_cls(self.model_cfg, group=self.group, device=self.device, **kw)
        if dtype == torch.float32:
            self.model = self.model.float()
        load_model_weights(self.model, config.model.id, self.entry.weight.required_prefixes,
                           ignored_prefixes=self.entry.weight.ignored_prefixes, strip_prefixes=self.entry.weight.strip_prefixes)
        self.model.eval()
        if self.entry.adapter_attr and config.model.adapter_model_ids:
            # other LLM sizes that share this tower: each contributes its own projector
            add = getattr(self.model, self.entry.adapter_attr)
            for aid in config.model.adapter_model_ids:
                from ...utils.hub import has_weights, iter_safetensors

                w = iter_safetensors(aid, self.entry.weight.adapter_prefixes, True) if has_weights(aid) else None
                add(aid, load_config(aid), w)
        self.sidecar: Sidecar | None = None
        if config.sidecar.ranks:
            self.sidecar = Sidecar(SidecarConfig(
                sidecar_rank=config.sidecar.ranks[tp_rank], group=list(config.sidecar.ranks),
                send_tensor_dtype=self.model.dtype, send_tensor_shape=(-1, *self.model.chunk_shape[1:])))
        self.dump_dir = os.environ.get("CORNSERVE_TEST_DUMP_TENSOR_DIR")
        self.profiler = None
        # raw inputs go through one page-locked staging buffer, so the copy to the GPU is a real asynchronous DMA
        self._stage: torch.Tensor | None = None
        self._stage_used = 0
        self.stats = {"batches": 0, "items": 0, "h2d_bytes": 0, "busy_ms": 0.0, "broadcast_ms": 0.0}
        logger.info("Worker %d ready on %s (%s)", tp_rank, self.device, model_type)

    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        if t.device == self.device or self.device.type != "cuda":
            return t.to(self.device)
        n = t.numel() * t.element_size()
        cap = int(os.environ.get("CORNSERVE_ERIC_STAGING_BYTES", str(256 << 20)))
        if self._stage is None:
            self._stage = torch.empty(cap, dtype=torch.uint8, pin_memory=True)
        self.stats["h2d_bytes"] += n
        if self._stage_used + n > cap:
            return t.contiguous().to(self.device)   # larger than the staging buffer: the pageable path
        lo = -(-self._stage_used // 256) * 256
        if lo + n > cap:
            return t.contiguous().to(self.device)
        view = self._stage[lo: lo + n].view(t.dtype).view(t.shape)
        view.copy_(t)
        self._stage_used = lo + n
        return view.to(self.device, non_blocking=True)

    def stage(self, batch: Batch) -> Batch:
        """The batch with every host tensor copied to this worker's device (through page-locked memory)."""
        self._stage_used = 0
        data = {k: [self._to_device(v) if isinstance(v, torch.Tensor) else v for v in vs] for k, vs in batch.data.items()}
        return Batch(batch.modality, batch.adapter_name, batch.request_ids, batch.data_ids, batch.receiver_ranks, data,
                     batch.trace_carriers)

    def prepare(self, batch: Batch) -> dict[str, list]:
        """Decoded uint8 pixels / float waveforms -> model inputs on the device, by the model's preprocessing recipe."""
        data = dict(batch.data)
        recipe, dev, dt = self.entry.processor, self.device, self.model.dtype
        to_dev = lambda t: t.to(dev, non_blocking=True)  # noqa: E731
        if "raw_audio" in data:
            data["input_features"] = [log_mel_spectrogram(to_dev(w)).to(dt) for w in data.pop("raw_audio")]
            return data
        raw_key = "raw_images" if "raw_images" in data else ("raw_videos" if "raw_videos" in data else None)
        if raw_key is None:
            return data
        items = data.pop(raw_key)
        video = raw_key == "raw_videos"
        if recipe in ("qwen2_vl", "qwen3_vl", "qwen2_5_omni", "qwen3_omni"):
            vc = self.model_cfg.vision if hasattr(self.model_cfg, "vision") else self.model_cfg
            half = recipe in ("qwen3_vl", "qwen3_omni")
            pix, grids = [], []
            for frames in items:
                pv, g = patchify_frames(to_dev(frames), vc.patch_size, vc.temporal_patch_size, vc.spatial_merge_size, out_dtype=dt,
                                        **({"mean": HALF, "std": HALF} if half else {}))
                pix.append(pv)
                grids.append(list(g))
            k = ("pixel_values_videos", "video_grid_thw") if video else ("pixel_values", "image_grid_thw")
            data[k[0]], data[k[1]] = pix, grids
        elif recipe == "gemma3":
            s = self.model_cfg.vision.image_size
            data["pixel_values"] = [resize_normalize(to_dev(im), (s, s), out_dtype=dt) for im in items]
            data["num_crops"] = [torch.zeros(1, dtype=torch.long) for _ in items]
        elif recipe == "llava_onevision":
            cfg = self.model_cfg
            s = cfg.vision.image_size
            if video:
                data["pixel_values_videos"] = [resize_normalize(to_dev(v), (s, s), mode="bicubic", out_dtype=dt) for v in items]
            else:
                tiles = [anyres_tiles(to_dev(im), cfg.image_grid_pinpoints, s, out_dtype=dt) for im in items]
                data["pixel_values"] = [t for t, _ in tiles]
                data["image_sizes"] = [torch.tensor(sz) for _, sz in tiles]
        elif recipe == "internvl":
            s = self.model_cfg.image_size
            if video:
                data["pixel_values_videos"] = [resize_normalize(to_dev(v), (s, s), IMAGENET_MEAN, IMAGENET_STD, "bicubic", dt) for v in items]
            else:
                data["pixel_values"] = [dynamic_tiles(to_dev(im), s, out_dtype=dt) for im in items]
        else:
            raise ValueError(f"unknown preprocessing recipe {recipe}")
        return data

    @torch.inference_mode()
    def execute_model(self, batch: Batch) -> None:
        ctx = extract(batch.trace_carriers[0]) if batch.trace_carriers else None
        t0 = time.perf_counter()
        with tracer.start_as_current_span("Worker.execute_model", context=ctx):
            outputs = self.model(batch.modality.value, batch.adapter_name, self.prepare(self.stage(batch)))
            if self.profiler is not None:
                self.profiler.step()
            for out, data_id, ranks in zip(outputs, batch.data_ids, batch.receiver_ranks, strict=True):
                out = out.contiguous()
                if self.dump_dir and self.tp_rank == 0:
                    torch.save(out.cpu(), Path(self.dump_dir) / f"{data_id}.pt")
                if self.sidecar is not None and ranks:
                    self.sidecar.send(out, id=data_id, dst_sidecar_ranks=ranks)
            if self.sidecar is not None:
                # outputs are shared with the sidecar by reference: they must outlive the hand-off
                self.sidecar.flush()
            elif self.device.type == "cuda":
                torch.cuda.current_stream(self.device).synchronize()   # the staging buffer is reused by the next batch
        self.stats["batches"] += 1
        self.stats["items"] += len(batch.data_ids)
        self.stats["busy_ms"] += (time.perf_counter() - t0) * 1e3

    def start_profile(self, out_dir: str) -> None:
        acts = [torch.profiler.ProfilerActivity.CPU]
        if self.device.type == "cuda":
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        Path(out_dir).mkdir(parents=True, exist_ok=True)
        self.profiler = torch.profiler.profile(
            activities=acts, record_shapes=True, with_stack=True,
            on_trace_ready=torch.profiler.tensorboard_trace_handler(out_dir, worker_name=f"eric-rank{self.tp_rank}"))
        self.profiler.start()

    def stop_profile(self) -> None:
        if self.profiler is not None:
            self.profiler.stop()
            self.profiler = None

    def shutdown(self) -> None:
        if self.sidecar is not None:
            self.sidecar.shutdown_sync()


_TENSOR = "__tensor__"


def split_batch(batch: Batch) -> tuple[Batch, list[torch.Tensor]]:
    """A copy of ``batch`` whose tensors are replaced by (marker, index, shape, dtype) plus the tensors themselves: the
    small part travels as a pickled object, the tensors by a device broadcast."""
    tensors: list[torch.Tensor] = []

    def strip(v):
        if isinstance(v, torch.Tensor):
            tensors.append(v)
            return (_TENSOR, len(tensors) - 1, tuple(v.shape), str(v.dtype).replace("torch.", ""))
        return v

    data = {k: [strip(v) for v in vs] for k, vs in batch.data.items()}
    return Batch(batch.modality, batch.adapter_name, batch.request_ids, batch.data_ids, batch.receiver_ranks, data,
                 batch.trace_carriers), tensors


def join_batch(header: Batch, tensors: list[torch.Tensor]) -> Batch:
    fill = lambda v: tensors[v[1]] if isinstance(v, tuple) and len(v) == 4 and v[0] == _TENSOR else v  # noqa: E731
    header.data = {k: [fill(v) for v in vs] for k, vs in header.data.items()}
    return header


def broadcast_batch(group: ParallelGroup, batch: Batch | None, device: torch.device) -> Batch:
    """Rank 0 passes the staged batch (tensors on its device); the others pass ``None`` and get a batch whose tensors
    sit on their own device.  One small object broadcast + one tensor broadcast per input."""
    import torch.distributed as dist

    if group.rank == 0:
        header, tensors = split_batch(batch)
        group.broadcast_object(("execute_model", header), src=0)
    else:
        header = batch   # the follower loop already received the header
        tensors = []
        for vs in header.data.values():
            for v in vs:
                if isinstance(v, tuple) and len(v) == 4 and v[0] == _TENSOR:
                    tensors.append(torch.empty(v[2], dtype=getattr(torch, v[3]), device=device))
    for t in tensors:
        dist.broadcast(t if t.is_contiguous() else t.contiguous(), src=dist.get_global_rank(group.group, 0) if group.group else 0,
                       group=group.group)
    return batch if group.rank == 0 else join_batch(header, tensors)


def tp_worker_main(config_json: str, tp_rank: int, tp_size: int, master_port: int) -> None:
    """Entry of a TP worker process (rank > 0): replay what rank 0 broadcasts until told to stop."""
    config = EricConfig.model_validate_json(config_json)
    device = pick_device(tp_rank)
    group = init_distributed(tp_rank, tp_size, master_port=master_port,
                             local_device=device.index if device.type == "cuda" else None,
                             backend=None if device.type == "cuda" else "gloo")
    worker = Worker(config, tp_rank, group)
    while True:
        method, arg = group.broadcast_object(None, src=0)
        if method == "shutdown":
            break
        if method == "execute_model":
            worker.execute_model(broadcast_batch(group, arg, worker.device))
            continue
        getattr(worker, method)(*arg)
    worker.shutdown()
