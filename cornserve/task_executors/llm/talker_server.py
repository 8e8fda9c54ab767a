"""The LLM executor in talker mode (``--run-talker [--run-vocoder]``): the speech half of an any-to-any model.

Contract (reference: tasklib/cornserve_tasklib/task_executors/descriptor/omni.py:63-221; the reference runs this inside
its vLLM fork): ``POST /v1/chat/completions`` whose ``vllm_xargs`` name the forwarded thinker view
(``cornserve_hidden_states_recv_id``).  The talker turns it into codec frames.  Without ``--run-vocoder`` the frames
``[T, num_code_groups]`` are forwarded to the generator executor (``cornserve_residual_codes_forward_id/_ranks``) and
the reply is a short JSON; with it, the vocoder runs here in chunks and the reply is an OpenAI-style event stream whose
``choices[0].delta.audio.data`` carries base64 PCM16.

One request at a time: a frame needs one talker step and ``num_code_groups - 1`` code-predictor steps in sequence.
"""

from __future__ import annotations

import argparse
import ast
import asyncio
import base64
import json
import os
import threading
import time
import uuid
from typing import Any

import numpy as np
import torch
from fastapi import FastAPI, Request, Response
from fastapi.responses import JSONResponse, StreamingResponse

from ... import ops
from ...logging import get_logger
from ...models.omni_talker import Talker, TalkerConfig, unpack_thinker_view
from ...utils.hub import load_config, load_model_weights
from .tokenizer import ByteTokenizer, load_tokenizer

logger = get_logger(__name__)


def special_tokens(hf_cfg: dict[str, Any], tokenizer) -> dict[str, Any]:
    """Ids that delimit the turns of the thinker's token sequence, for the tokenizer in use."""
    th = hf_cfg.get("thinker_config") or {}
    mm = tuple(int(th.get(k, hf_cfg.get(k, d))) for k, d in (("audio_token_id", 151646), ("image_token_id", 151655),
                                                            ("video_token_id", 151656)))
    if isinstance(tokenizer, ByteTokenizer):
        # roles are spelled out in bytes: the token after <|im_start|> is the role's first letter
        sp, off = tokenizer.sp, tokenizer.off
        return {"im_start": sp.im_start, "system": off + ord("s"), "user": off + ord("u"), "assistant": off + ord("a"),
                "multimodal": (sp.audio_pad, sp.image_pad, sp.video_pad), "assistant_header": 1 + len("assistant") + 1}
    return {"im_start": int(hf_cfg.get("im_start_token_id", 151644)), "system": int(hf_cfg.get("system_token_id", 8948)),
            "user": int(hf_cfg.get("user_token_id", 872)), "assistant": int(hf_cfg.get("assistant_token_id", 77091)),
            "multimodal": mm, "assistant_header": 3}


class TalkerServer:
    def __init__(self, args: argparse.Namespace):
        from .server import pick_device

        self.args = args
        self.hf_cfg = load_config(args.model)
        if "talker_config" not in self.hf_cfg:
            raise ValueError(f"{args.model} has no talker")
        self.device = pick_device()
        ops.bind_thread(self.device)
        torch.manual_seed(int(os.environ.get("CORNSERVE_SEED", "0")) + 1)
        self.cfg = TalkerConfig.from_hf(self.hf_cfg["talker_config"])
        self.talker = Talker(self.cfg, device=self.device)
        if self.device.type == "cpu":
            self.talker.float()
        load_model_weights(self.talker, args.model, ["talker."], strict=False)
        self.talker.eval()
        self.vocoder = None
        if args.run_vocoder:
            from ...models.code2wav import Code2Wav, Code2WavConfig

            self.vocoder = Code2Wav(Code2WavConfig.from_hf(self.hf_cfg.get("code2wav_config") or {}), device=self.device)
            if self.device.type == "cpu":
                self.vocoder.float()
            load_model_weights(self.vocoder, args.model, ["code2wav."], strict=False)
            self.vocoder.eval()
        th = self.hf_cfg.get("thinker_config") or {}
        vocab = int((th.get("text_config") or th).get("vocab_size", 152064))
        self.special = special_tokens(self.hf_cfg, load_tokenizer(args.model, {**th, **self.hf_cfg}, vocab))
        self.sidecar = None
        if args.cornserve_sidecar_ranks:
            from ...sidecar.api import Sidecar
            from ...sidecar.schema import SidecarConfig

            H = self.cfg.thinker_hidden_size
            self.sidecar = Sidecar(SidecarConfig(sidecar_rank=args.cornserve_sidecar_ranks[0], group=list(args.cornserve_sidecar_ranks), whole_group=True,
                                                 send_tensor_dtype=torch.int64, send_tensor_shape=(-1, self.cfg.num_code_groups),
                                                 recv_tensor_dtype=self.talker.dtype, recv_tensor_shape=(-1, H)))
        self.lock = asyncio.Lock()
        self.alive = True

    # -- generation on a worker thread ---------------------------------------------------------------------
    def _frames(self, rows: torch.Tensor, body: dict[str, Any], loop: asyncio.AbstractEventLoop, q: asyncio.Queue) -> None:
        try:
            ops.bind_thread(self.device)
            ids, embeds, hidden, tts = unpack_thinker_view(rows.to(self.device))
            speakers = self.cfg.speaker_id
            speaker = speakers.get(str(body.get("speaker", "")).lower(), next(iter(speakers.values()), self.cfg.codec_pad_id))
            with torch.inference_mode():
                prefill, trailing, pad = self.talker.build_inputs(ids, embeds, hidden, tts, self.special, speaker)
                max_frames = int(body.get("max_audio_frames") or 4 * int(trailing.shape[0]) + 64)
                gen = None
                if body.get("seed") is not None:
                    gen = torch.Generator(device=self.device).manual_seed(int(body["seed"]))
                for codes in self.talker.generate(prefill, trailing, pad, max_frames=max_frames,
                                                  sample=not (bool(body.get("greedy", False)) or os.environ.get("CORNSERVE_TALKER_GREEDY") == "1"),
                                                  generator=gen, min_frames=int(body.get("min_audio_frames") or
                                                                                os.environ.get("CORNSERVE_TALKER_MIN_FRAMES", "0"))):
                    loop.call_soon_threadsafe(q.put_nowait, codes)
            loop.call_soon_threadsafe(q.put_nowait, None)
        except Exception as e:  # noqa: BLE001
            logger.exception("talker generation failed")
            loop.call_soon_threadsafe(q.put_nowait, e)

    def _vocode(self, codes: torch.Tensor, n_new: int) -> bytes:
        """PCM16 of the last ``n_new`` frames of ``codes`` ``[T, groups]`` (the frames before them are left context; the
        vocoder is causal, so a chunk decoded with enough context equals the same stretch of a one-shot decode)."""
        ops.bind_thread(self.device)
        T = int(codes.shape[0])
        wav = self.vocoder(codes.t()[None].contiguous())          # [1, samples]
        lo = (T - n_new) * self.vocoder.cfg.total_upsample
        return ops.pcm16(wav[0, lo: self.vocoder.output_length(T)].contiguous()).cpu().numpy().tobytes()

    # -- request handling ---------------------------------------------------------------------------------------
    async def chat(self, body: dict[str, Any]):
        xargs = body.get("vllm_xargs") or {}
        rid, created, model = f"chatcmpl-{uuid.uuid4().hex}", int(time.time()), body.get("model", self.args.model)
        recv_id = xargs.get("cornserve_hidden_states_recv_id")
        if recv_id is None or self.sidecar is None:
            return JSONResponse({"error": {"message": "the talker needs cornserve_hidden_states_recv_id and a sidecar"}}, status_code=400)
        try:
            chunks, k = [], 0
            while (t := await self.sidecar.recv(recv_id, k)) is not None:
                chunks.append(t)
                k += 1
            rows = (chunks[0] if len(chunks) == 1 else torch.cat(chunks)).clone()
            for i in range(k):
                await self.sidecar.mark_done(recv_id, i)
        except Exception as e:  # noqa: BLE001
            logger.exception("receiving the thinker view failed")
            return JSONResponse({"error": {"message": str(e)}}, status_code=500)
        loop = asyncio.get_running_loop()
        q: asyncio.Queue = asyncio.Queue()

        async def frames():
            async with self.lock:   # first come, first served
                threading.Thread(target=self._frames, args=(rows, body, loop, q), daemon=True).start()
                while (item := await q.get()) is not None:
                    if isinstance(item, Exception):
                        raise item
                    yield item

        if not (body.get("cornserve_return_audio") and self.vocoder is not None):
            try:
                codes = [c async for c in frames()]
            except Exception as e:  # noqa: BLE001
                return JSONResponse({"error": {"message": str(e)}}, status_code=500)
            out = torch.stack(codes) if codes else torch.zeros((0, self.cfg.num_code_groups), dtype=torch.int64)
            fid = xargs.get("cornserve_residual_codes_forward_id")
            ranks = ast.literal_eval(xargs.get("cornserve_residual_codes_forward_ranks", "[]")) or []
            if fid and ranks:
                self.sidecar.send(out.to(self.device).contiguous(), id=fid, dst_sidecar_ranks=ranks)
                await asyncio.to_thread(self.sidecar.flush)
            return JSONResponse({"id": rid, "object": "chat.completion", "created": created, "model": model, "choices": [],
                                 "cornserve": {"codec_frames": int(out.shape[0])}})

        chunk_size = int(body.get("audio_chunk_frames") or 25)
        left = int(body.get("audio_left_context_frames") or 25)

        def event(data: bytes | None, finish: str | None = None) -> str:
            delta = {"audio": {"data": base64.b64encode(data).decode()}} if data is not None else {}
            return "data: " + json.dumps({"id": rid, "object": "chat.completion.chunk", "created": created, "model": model,
                                          "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}) + "\n\n"

        async def sse():
            history: list[torch.Tensor] = []
            sent = 0
            try:
                async for codes in frames():
                    history.append(codes)
                    if len(history) - sent >= chunk_size:
                        lo = max(0, sent - left)
                        pcm = await asyncio.to_thread(self._vocode, torch.stack(history[lo:]), len(history) - sent)
                        sent = len(history)
                        yield event(pcm)
                if len(history) > sent:
                    lo = max(0, sent - left)
                    yield event(await asyncio.to_thread(self._vocode, torch.stack(history[lo:]), len(history) - sent))
                yield event(None, "stop")
            except Exception as e:  # noqa: BLE001
                yield f"data: {json.dumps({'error': str(e)})}\n\n"
            yield "data: [DONE]\n\n"

        return StreamingResponse(sse(), media_type="text/event-stream")

    def create_app(self) -> FastAPI:
        app = FastAPI(title="cornserve-b200 LLM executor (talker)")
        from ...tracing import instrument_fastapi

        instrument_fastapi(app, "cornserve.llm-talker")

        @app.get("/health")
        async def health():
            return Response(status_code=200 if self.alive else 503)

        @app.get("/v1/models")
        async def models():
            return {"object": "list", "data": [{"id": self.args.model, "object": "model"}]}

        @app.post("/v1/chat/completions")
        async def chat(raw: Request):
            return await self.chat(await raw.json())

        return app

    def shutdown(self) -> None:
        self.alive = False
        if self.sidecar is not None:
            self.sidecar.shutdown_sync()
