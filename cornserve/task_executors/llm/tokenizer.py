"""Tokenisation for the LLM executor.

If the model directory has Hugging Face tokenizer files they are used (``transformers.AutoTokenizer``),
including the model's chat template.  Otherwise, e.g. for architecture-only runs with random weights, a
byte-level fallback maps UTF-8 bytes to ids ``[byte_offset, byte_offset + 256)`` and renders chats in the
ChatML layout that the Qwen family uses, which is enough to drive the engine end to end.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from ...logging import get_logger
from ...utils.hub import resolve_model_dir

logger = get_logger(__name__)


@dataclass
class SpecialTokens:
    im_start: int
    im_end: int
    vision_start: int
    vision_end: int
    image_pad: int
    video_pad: int
    audio_pad: int
    eos: int


class ByteTokenizer:
    """Fallback tokenizer: one id per UTF-8 byte, ChatML control tokens at the top of the vocabulary."""

    def __init__(self, vocab_size: int, specials: SpecialTokens, byte_offset: int = 3):
        if vocab_size < byte_offset + 256:
            raise ValueError("vocabulary too small for the byte-level fallback tokenizer")
        self.vocab_size, self.sp, self.off = vocab_size, specials, byte_offset

    def encode(self, text: str) -> list[int]:
        return [self.off + b for b in text.encode("utf-8")]

    def decode(self, ids: list[int]) -> str:
        data = bytes(i - self.off for i in ids if self.off <= i < self.off + 256)
        return data.decode("utf-8", errors="replace")

    def render_chat(self, messages: list[dict[str, Any]], add_generation_prompt: bool = True) -> tuple[list[int], list[tuple[int, str]]]:
        """Token ids plus ``(position, modality)`` of every multimodal placeholder (one pad token each; the
        caller expands it to the real number of embedding rows)."""
        ids: list[int] = []
        marks: list[tuple[int, str]] = []
        nl = self.encode("\n")
        for m in messages:
            ids += [self.sp.im_start] + self.encode(m["role"]) + nl
            content = m["content"]
            parts = [{"type": "text", "text": content}] if isinstance(content, str) else content
            for p in parts:
                kind = p.get("type", "text")
                if kind == "text":
                    ids += self.encode(p["text"])
                else:
                    modality = kind.split("_")[0]
                    pad = {"image": self.sp.image_pad, "video": self.sp.video_pad, "audio": self.sp.audio_pad}[modality]
                    ids.append(self.sp.vision_start)
                    marks.append((len(ids), modality))
                    ids.append(pad)
                    ids.append(self.sp.vision_end)
            ids += [self.sp.im_end] + nl
        if add_generation_prompt:
            ids += [self.sp.im_start] + self.encode("assistant") + nl
        return ids, marks


class HFTokenizer:
    """Wrapper over a Hugging Face tokenizer with the same interface as :class:`ByteTokenizer`."""

    def __init__(self, path: str, specials: SpecialTokens):
        from transformers import AutoTokenizer

        self.tok = AutoTokenizer.from_pretrained(path, trust_remote_code=False)
        self.sp = specials
        self.vocab_size = len(self.tok)

    def encode(self, text: str) -> list[int]:
        return self.tok.encode(text, add_special_tokens=False)

    def decode(self, ids: list[int]) -> str:
        return self.tok.decode(ids, skip_special_tokens=True)

    def render_chat(self, messages, add_generation_prompt: bool = True):
        pads = {"image": "<|image_pad|>", "video": "<|video_pad|>", "audio": "<|audio_pad|>"}
        flat = []
        for m in messages:
            content = m["content"]
            if isinstance(content, str):
                flat.append({"role": m["role"], "content": content})
                continue
            text = ""
            for p in content:
                kind = p.get("type", "text")
                text += p["text"] if kind == "text" else f"<|vision_start|>{pads[kind.split('_')[0]]}<|vision_end|>"
            flat.append({"role": m["role"], "content": text})
        try:
            ids = self.tok.apply_chat_template(flat, add_generation_prompt=add_generation_prompt, tokenize=True)
            ids = ids["input_ids"] if isinstance(ids, dict) else list(ids)
        except Exception:
            text = "".join(f"<|im_start|>{m['role']}\n{m['content']}<|im_end|>\n" for m in flat)
            ids = self.tok.encode(text + ("<|im_start|>assistant\n" if add_generation_prompt else ""), add_special_tokens=False)
        pad_to_mod = {self.sp.image_pad: "image", self.sp.video_pad: "video", self.sp.audio_pad: "audio"}
        marks = [(i, pad_to_mod[t]) for i, t in enumerate(ids) if t in pad_to_mod]
        return list(ids), marks


def specials_from_config(cfg: dict[str, Any], vocab_size: int) -> SpecialTokens:
    top = vocab_size - 1
    return SpecialTokens(
        im_start=cfg.get("im_start_token_id", cfg.get("bos_token_id") or top - 6),
        im_end=cfg.get("im_end_token_id", top - 5),
        vision_start=cfg.get("vision_start_token_id", top - 4),
        vision_end=cfg.get("vision_end_token_id", top - 3),
        image_pad=cfg.get("image_token_id", top - 2),
        video_pad=cfg.get("video_token_id", top - 1),
        audio_pad=cfg.get("audio_token_id", top - 7),
        eos=(cfg.get("eos_token_id")[0] if isinstance(cfg.get("eos_token_id"), list) else cfg.get("eos_token_id")) or top,
    )


def load_tokenizer(model_id: str, hf_config: dict[str, Any], vocab_size: int):
    specials = specials_from_config(hf_config, vocab_size)
    d = resolve_model_dir(model_id)
    if d is not None and ((d / "tokenizer.json").is_file() or (d / "tokenizer_config.json").is_file()):
        try:
            return HFTokenizer(str(d), specials)
        except Exception as e:
            logger.warning("Could not load the tokenizer in %s (%s); using the byte-level fallback", d, e)
    return ByteTokenizer(vocab_size, specials)
