"""In-process first-come-first-served engine of the monolithic executor: one request runs at a time on a worker
thread, streamed outputs are handed to the event loop as they are produced (reference:
python/cornserve/task_executors/huggingface/engine.py:17-89)."""

from __future__ import annotations

import asyncio
import threading
from collections.abc import AsyncIterator

import torch

from ... import ops
from ...logging import get_logger
from .api import HuggingFaceRequest, HuggingFaceResponse, ModelType, Status
from .config import HuggingFaceConfig
from .models import QwenImageMonolith, QwenOmniMonolith

logger = get_logger(__name__)


class Engine:
    def __init__(self, config: HuggingFaceConfig, device: torch.device):
        self.config, self.device = config, device
        if config.model.model_type == ModelType.QWEN_IMAGE:
            self.model = QwenImageMonolith(config.model.id, device, config.model.text_encoder_id)
        else:
            self.model = QwenOmniMonolith(config.model.id, device)
        self.lock = asyncio.Lock()  # FCFS: asyncio locks wake waiters in arrival order
        self.alive = True

    async def generate(self, req: HuggingFaceRequest) -> HuggingFaceResponse:
        async with self.lock:
            try:
                def image():
                    ops.bind_thread(self.device)  # pool threads start on CUDA device 0
                    return self.model.generate(req.prompt, req.height, req.width, req.num_inference_steps)

                img = await asyncio.to_thread(image)
                return HuggingFaceResponse(status=Status.SUCCESS, image=img)
            except Exception as e:  # noqa: BLE001
                logger.exception("image generation failed")
                return HuggingFaceResponse(status=Status.ERROR, error_message=str(e))

    async def stream(self, req: HuggingFaceRequest) -> AsyncIterator[HuggingFaceResponse]:
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()

        def work():
            try:
                ops.bind_thread(self.device)
                for chunk in self.model.generate(req.messages or [], req.max_completion_tokens or 256, req.ignore_eos,
                                                 bool(req.return_audio)):
                    loop.call_soon_threadsafe(q.put_nowait, HuggingFaceResponse(status=Status.SUCCESS, text_chunk=chunk))
            except Exception as e:  # noqa: BLE001
                logger.exception("omni generation failed")
                loop.call_soon_threadsafe(q.put_nowait, HuggingFaceResponse(status=Status.ERROR, error_message=str(e)))
            loop.call_soon_threadsafe(q.put_nowait, None)

        async with self.lock:
            threading.Thread(target=work, daemon=True).start()
            while (item := await q.get()) is not None:
                yield item
