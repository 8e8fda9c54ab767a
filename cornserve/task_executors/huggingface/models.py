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
    cfg = LLMConfig.from_hf(hf_cfg.get("thinker_config") or hf_cfg)
    llm = QwenLLM(cfg, device=device)
    if device.type == "cpu":  # the CUDA kernels are bf16
        llm = llm.float()
    load_model_weights(llm, model_id, ["model.language_model.", "language_model.", "thinker.model.", "model.", ""],
                       strict=False, ignored_prefixes=["visual.", "model.visual.", "vision_tower.", "audio_tower."])
    llm.eval()
    engine = LLMEngine(llm, EngineConfig(num_pages=pages, decode_burst=4, max_model_len=8192, use_cuda_graph=device.type == "cuda"))
    return engine, load_tokenizer(model_id, {**(hf_cfg.get("thinker_config") or {}), **hf_cfg}, cfg.vocab_size), hf_cfg


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
    """Thinker, talker and vocoder in one process; yields OpenAI-style chunks: the text first, then (when asked) the
    spoken answer as base64 PCM16 in ``delta.audio.data``."""

    def __init__(self, model_id: str, device: torch.device):
        self.model_id, self.device = model_id, device
        self.engine, self.tok, self.hf_cfg = _build_llm(model_id, device)
        self.talker = self.vocoder = None
        if "talker_config" in self.hf_cfg:
            from ...models.code2wav import Code2Wav, Code2WavConfig
            from ...models.omni_talker import Talker, TalkerConfig
            from ..llm.talker_server import special_tokens

            torch.manual_seed(1)
            self.talker = Talker(TalkerConfig.from_hf(self.hf_cfg["talker_config"]), device=device)
            self.vocoder = Code2Wav(Code2WavConfig.from_hf(self.hf_cfg.get("code2wav_config") or {}), device=device)
            if device.type == "cpu":
                self.talker.float()
                self.vocoder.float()
            load_model_weights(self.talker, model_id, ["talker."], strict=False)
            load_model_weights(self.vocoder, model_id, ["code2wav."], strict=False)
            self.special = special_tokens(self.hf_cfg, self.tok)

    def _run(self, seq: Sequence):
        self.engine.add_request(seq)
        while self.engine.has_work():
            yield from self.engine.step()

    def generate(self, messages: list[dict], max_tokens: int, ignore_eos: bool, return_audio: bool, greedy_audio: bool = False,
                 min_audio_frames: int = 0) -> Iterator[dict]:
        if return_audio and self.talker is None:
            raise NotImplementedError(f"{self.model_id} has no talker: it produces text only (return_audio must be false)")
        ids, _ = self.tok.render_chat(messages)
        rid, created = uuid.uuid4().hex, int(time.time())
        prompt = np.asarray(ids, dtype=np.int32)

        def chunk(delta: dict, finish=None) -> dict:
            return {"id": rid, "object": "chat.completion.chunk", "created": created, "model": self.model_id,
                    "choices": [{"index": 0, "delta": delta, "finish_reason": finish}]}

        tokens: list[int] = []
        for out in self._run(Sequence(rid, prompt, SamplingParams(max_tokens, ignore_eos))):
            tokens.extend(out.new_token_ids)
            yield chunk({"content": self.tok.decode(out.new_token_ids)}, out.finish_reason if out.finished and not return_audio else None)
        if not return_audio:
            return
        import base64

        from ... import ops
        from ...models.omni_talker import pack_thinker_view, unpack_thinker_view

        tc = self.hf_cfg["talker_config"]
        full = np.concatenate([prompt, np.asarray(tokens, dtype=np.int32)])
        view = None
        for out in self._run(Sequence(rid + "-view", full, SamplingParams(1, True), capture_layers=(0, int(tc.get("accept_hidden_layer", 18))))):
            view = out.hidden if out.hidden is not None else view
        H = self.engine.mcfg.hidden_size
        tts_ids = [int(self.hf_cfg.get(k, d)) for k, d in (("tts_bos_token_id", 151672), ("tts_eos_token_id", 151673), ("tts_pad_token_id", 151671))]
        with torch.inference_mode():
            tts = self.engine.model.embed_tokens(torch.tensor(tts_ids, dtype=torch.int32, device=self.device))
            ids2, emb, hid, tts = unpack_thinker_view(pack_thinker_view(full, view[:, :H], view[:, H:], tts))
            speaker = next(iter(self.talker.cfg.speaker_id.values()), self.talker.cfg.codec_pad_id)
            prefill, trailing, pad = self.talker.build_inputs(ids2, emb, hid, tts, self.special, speaker)
            frames = list(self.talker.generate(prefill, trailing, pad, max_frames=4 * int(trailing.shape[0]) + 64, sample=not greedy_audio,
                                               min_frames=min_audio_frames))
            if frames:
                wav = self.vocoder(torch.stack(frames).t()[None].contiguous())
                pcm = ops.pcm16(wav[0, : self.vocoder.output_length(len(frames))].contiguous()).cpu().numpy().tobytes()
                yield chunk({"audio": {"data": base64.b64encode(pcm).decode()}})
        yield chunk({}, "stop")
