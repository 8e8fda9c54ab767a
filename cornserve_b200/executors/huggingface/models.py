"""The two monolithic baselines: whole pipelines inside one process, with no encoder / LLM / generator fission
(reference: python/cornserve/task_executors/huggingface/models/qwen_image.py:19-75 and qwen_omni.py:24-161, which
call ``diffusers`` / ``transformers`` ``generate``).  Here they are assembled from this repository's own models, so
the comparison between fission and no fission runs on the same kernels."""

from __future__ import annotations

import time
import uuid
from collections.abc import Iterator
from typing import Any

import numpy as np
import torch

from ...models.qwen_llm import LLMConfig, QwenLLM
from ...utils.hub import load_config, load_model_weights, resolve_model_dir
from ..geri.loader import load_model as load_generator
from ..llm.engine import EngineConfig, LLMEngine, SamplingParams, Sequence
from ..llm.tokenizer import load_tokenizer

# instruction the image generator was trained with; its tokens are cut from the conditioning
IMAGE_SYSTEM_PROMPT = ("Describe the image by detailing the color, shape, size, texture, quantity, text, spatial relationships "
                       "of the objects and background:")
IMAGE_PROMPT_SKIP_TOKENS = 34


def _build_llm(model_id: str, device: torch.device, pages: int = 256) -> tuple[LLMEngine, Any, dict]:
    hf_cfg = load_config(model_id)
    cfg = LLMConfig.from_hf(hf_cfg)
    llm = QwenLLM(cfg, device=device)
    if device.type == "cpu":  # the CUDA kernels are bf16
        llm = llm.float()
    load_model_weights(llm, model_id, ["model.language_model.", "language_model.", "thinker.model.", "model.", "lm_head.", ""],
                       strict=False, ignored_prefixes=["visual.", "model.visual.", "vision_tower.", "audio_tower."])
    llm.eval()
    engine = LLMEngine(llm, EngineConfig(num_pages=pages, decode_burst=4, max_model_len=8192, use_cuda_graph=device.type == "cuda"))
    return engine, load_tokenizer(model_id, hf_cfg, cfg.vocab_size), hf_cfg


class QwenImageMonolith:
    """Text encoder (the language model run once in hidden-state mode) + diffusion transformer + VAE."""

    def __init__(self, model_id: str, device: torch.device, text_encoder_id: str):
        d = resolve_model_dir(model_id)
        te = str(d / "text_encoder") if d is not None and (d / "text_encoder" / "config.json").is_file() else text_encoder_id
        self.engine, self.tok, _ = _build_llm(te, device)
        _, self.generator = load_generator(model_id, device)
        dim = self.engine.model.cfg.hidden_size
        if dim != self.generator.embedding_dim:
            raise ValueError(f"text encoder width {dim} does not match the generator's conditioning width {self.generator.embedding_dim}")

    def generate(self, prompt: str, height: int, width: int, num_inference_steps: int) -> str:
        ids, _ = self.tok.render_chat([{"role": "system", "content": IMAGE_SYSTEM_PROMPT}, {"role": "user", "content": prompt}])
        seq = Sequence(uuid.uuid4().hex, np.asarray(ids, dtype=np.int32), SamplingParams(1, True), return_hidden=True)
        self.engine.add_request(seq)
        hidden = None
        while self.engine.has_work():
            for out in self.engine.step():
                if out.hidden is not None:
                    hidden = out.hidden
        skip = min(IMAGE_PROMPT_SKIP_TOKENS, max(hidden.shape[0] - 1, 0))
        return self.generator.generate([hidden[skip:]], height, width, num_inference_steps)[0]


class QwenOmniMonolith:
    """Thinker served in-process; yields OpenAI-style text chunks.  Spoken answers need the talker, which this
    baseline does not include."""

    def __init__(self, model_id: str, device: torch.device):
        self.model_id = model_id
        self.engine, self.tok, _ = _build_llm(model_id, device)

    def generate(self, messages: list[dict], max_tokens: int, ignore_eos: bool, return_audio: bool) -> Iterator[dict]:
        if return_audio:
            raise NotImplementedError("the monolithic omni baseline produces text only (return_audio must be false)")
        ids, _ = self.tok.render_chat(messages)
        rid = uuid.uuid4().hex
        self.engine.add_request(Sequence(rid, np.asarray(ids, dtype=np.int32), SamplingParams(max_tokens, ignore_eos)))
        created = int(time.time())
        while self.engine.has_work():
            for out in self.engine.step():
                text = self.tok.decode(out.new_token_ids)
                yield {"id": rid, "object": "chat.completion.chunk", "created": created, "model": self.model_id,
                       "choices": [{"index": 0, "delta": {"content": text}, "finish_reason": out.finish_reason if out.finished else None}]}
