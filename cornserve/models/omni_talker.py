"""Qwen3-Omni talker: turns the thinker's token embeddings / hidden states into codec codes for the vocoder.

The reference runs this model inside its vLLM fork (``--run-talker``; contract in
tasklib/cornserve_tasklib/task_executors/descriptor/omni.py:63-221 and task/composite/omni.py:44-122); the model
itself is restated here from the checkpoint's structure:

* two small MLPs project thinker-side vectors to the talker width: ``text_projection`` for token embeddings,
  ``hidden_projection`` for hidden states of multimodal positions;
* the talker decoder is a Qwen3-MoE decoder with a gated shared expert (:class:`..qwen_llm.QwenLLM`) over a codec
  vocabulary: one step yields the first codebook's code of one audio frame;
* the code predictor, a 5-layer dense decoder with one embedding table and one output head per residual codebook,
  fills in the other ``num_code_groups - 1`` codes of the frame, conditioned on the talker's hidden state;
* the next talker input is the sum of the frame's code embeddings plus the projection of the next text token (or the
  TTS pad vector once the text is used up).

Both decoders run on the paged-KV kernels of the LLM executor.  Generation is sequential by nature (15 predictor steps
per 80 ms frame), so the runner drives one request at a time.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable, Iterator

import numpy as np
import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group
from .layers import Embedding, Linear
from .qwen_llm import PAGE_SIZE, BatchMeta, LLMConfig, QwenLLM


@dataclass
class TalkerConfig:
    thinker_hidden_size: int = 2048
    text: LLMConfig = field(default_factory=LLMConfig)
    predictor: LLMConfig = field(default_factory=LLMConfig)
    projection_intermediate: int = 2048
    num_code_groups: int = 16
    accept_hidden_layer: int = 18
    codec_eos_token_id: int = 4198
    codec_nothink_id: int = 4203
    codec_think_bos_id: int = 4204
    codec_think_eos_id: int = 4205
    codec_pad_id: int = 4196
    codec_bos_id: int = 4197
    speaker_id: dict[str, int] = field(default_factory=dict)

    @classmethod
    def from_hf(cls, cfg: dict) -> "TalkerConfig":
        """``cfg`` is the ``talker_config`` section of the checkpoint's config."""
        t, cp = dict(cfg.get("text_config") or {}), dict(cfg.get("code_predictor_config") or {})
        if "num_experts" not in t and "num_local_experts" in t:
            t["num_experts"] = t["num_local_experts"]
        text = LLMConfig.from_hf({**t, "model_type": "qwen3_moe"})
        text.mrope_section = None   # speech positions are sequential on all three axes: plain rotary embedding
        pred = LLMConfig.from_hf({**cp, "model_type": "qwen3"})
        pred.mrope_section = None
        kw = {k: cfg[k] for k in ("thinker_hidden_size", "num_code_groups", "accept_hidden_layer", "codec_eos_token_id",
                                  "codec_nothink_id", "codec_think_bos_id", "codec_think_eos_id", "codec_pad_id", "codec_bos_id")
              if cfg.get(k) is not None}
        return cls(text=text, predictor=pred, projection_intermediate=int(t.get("intermediate_size", 2048)),
                   speaker_id=dict(cfg.get("speaker_id") or {}), **kw)


def pack_thinker_view(token_ids: np.ndarray, embeds: torch.Tensor, hidden: torch.Tensor, tts_embeds: torch.Tensor) -> torch.Tensor:
    """What the thinker executor forwards to the talker executor, as one tensor (the forwarding path carries tensors of
    one dtype, in slots of the thinker's hidden width ``H``): per token ``[embedding | hidden state of the accepted layer |
    token id digits, zero padded to H]``, followed by three rows whose embedding part holds the thinker's embeddings of
    the TTS bos / eos / pad tokens.  Ids travel as base-256 digits, which are exact in bf16."""
    T, H = embeds.shape
    rows = torch.zeros((T + 3, 3 * H), device=embeds.device, dtype=embeds.dtype)
    rows[:T, :H] = embeds
    rows[:T, H: 2 * H] = hidden
    ids = torch.from_numpy(np.asarray(token_ids, dtype=np.int64)).to(embeds.device)
    for d in range(3):
        rows[:T, 2 * H + d] = ((ids >> (8 * d)) & 255).to(embeds.dtype)
    rows[T:, :H] = tts_embeds
    return rows


def unpack_thinker_view(rows: torch.Tensor) -> tuple[np.ndarray, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Inverse of :func:`pack_thinker_view`: ``(token_ids, embeds, hidden, tts_embeds)``."""
    H = rows.shape[1] // 3
    T = rows.shape[0] - 3
    digits = rows[:T, 2 * H: 2 * H + 3].float().round().long().cpu()
    ids = (digits[:, 0] + (digits[:, 1] << 8) + (digits[:, 2] << 16)).numpy()
    return ids, rows[:T, :H], rows[:T, H: 2 * H], rows[T:, :H]


class ResizeMLP(nn.Module):
    def __init__(self, d_in: int, d_mid: int, d_out: int, device):
        super().__init__()
        self.fc1 = Linear(d_in, d_mid, device=device)
        self.fc2 = Linear(d_mid, d_out, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.fc2(self.fc1(x, act="silu"))


class CodePredictor(nn.Module):
    """Dense decoder that emits the residual codebooks of one frame, one code per step."""

    def __init__(self, cfg: LLMConfig, groups: int, device):
        super().__init__()
        self.cfg, self.groups = cfg, groups
        self.model = QwenLLM(cfg, device=device)
        self.codec_embedding = nn.ModuleList([Embedding(cfg.vocab_size, cfg.hidden_size, device=device) for _ in range(groups - 1)])
        self.heads = nn.ModuleList([Linear(cfg.hidden_size, cfg.vocab_size, bias=False, device=device) for _ in range(groups - 1)])


def _embeds_meta(T: int, start: int, pages: list[int], device, decode: bool) -> BatchMeta:
    """One sequence, ``T`` new tokens at positions ``start ..``; every input row is supplied as an embedding."""
    i32 = dict(dtype=torch.int32, device=device)
    pos = torch.arange(start, start + T, **i32)
    pg = torch.tensor(pages, **i32)
    slots = pg[(pos // PAGE_SIZE).long()] * PAGE_SIZE + pos % PAGE_SIZE
    return BatchMeta(input_ids=torch.zeros(T, **i32), positions=pos[None].expand(3, T).contiguous(), slot_mapping=slots.to(torch.int32),
                     cu_q=torch.tensor([0, T], **i32), kv_len=torch.tensor([start + T], **i32), block_table=pg[None].contiguous(),
                     logits_idx=torch.tensor([T - 1], **i32), max_q_len=T, is_decode=decode and T == 1)


class Talker(nn.Module):
    def __init__(self, cfg: TalkerConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        D = cfg.text.hidden_size
        self.text_projection = ResizeMLP(cfg.thinker_hidden_size, cfg.projection_intermediate, D, device)
        self.hidden_projection = ResizeMLP(cfg.thinker_hidden_size, cfg.projection_intermediate, D, device)
        self.decoder = QwenLLM(cfg.text, group=self.group, device=device)   # embed_tokens = codec embedding, lm_head = codec head
        self.code_predictor = CodePredictor(cfg.predictor, cfg.num_code_groups, device)

    @property
    def device(self) -> torch.device:
        return self.decoder.device

    @property
    def dtype(self) -> torch.dtype:
        return self.decoder.embed_tokens.weight.dtype

    # -- input assembly ------------------------------------------------------------------------------------
    def build_inputs(self, token_ids: np.ndarray, embeds: torch.Tensor, hidden: torch.Tensor, tts: torch.Tensor, special: dict,
                     speaker: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """From the thinker's view of the whole conversation (prompt + answer): ``token_ids`` ``[T]``, token embeddings and
        hidden states of the accepted layer ``[T, thinker_hidden]``, the embeddings of the TTS bos / eos / pad tokens
        ``[3, thinker_hidden]``.  ``special`` holds the ids of ``im_start``, ``system``, ``user``, ``assistant`` (the token
        that follows ``im_start``), the multimodal placeholder tokens and optionally ``assistant_header`` (tokens of
        ``<|im_start|>assistant\n``: 3 with the checkpoint's tokenizer).  Returns ``(prefill [P, D], trailing_text
        [n, D], tts_pad [D])``."""
        cfg = self.cfg
        ids = np.asarray(token_ids)
        T = ids.shape[0]
        starts = [int(i) for i in np.nonzero(ids == special["im_start"])[0]] + [T]
        mm = np.isin(ids, list(special["multimodal"]))
        tts_bos, tts_eos, tts_pad = self.text_projection(tts.to(self.dtype)).unbind(0)
        hd = int(special.get("assistant_header", 3))
        parts: list[torch.Tensor] = []
        trailing = tts_eos[None]
        for i in range(len(starts) - 1):
            lo, hi = starts[i], starts[i + 1]
            role = int(ids[lo + 1]) if lo + 1 < T else -1
            if role == special["system"]:
                continue
            if role == special["user"]:
                part = torch.empty((hi - lo, cfg.text.hidden_size), device=self.device, dtype=self.dtype)
                m = torch.from_numpy(mm[lo:hi]).to(self.device)
                if bool(m.any()):
                    part[m] = self.hidden_projection(hidden[lo:hi][m].to(self.dtype))
                if bool((~m).any()):
                    part[~m] = self.text_projection(embeds[lo:hi][~m].to(self.dtype))
                parts.append(part)
            elif role == special["assistant"] and i == len(starts) - 2:
                a = self.text_projection(embeds[lo:hi].to(self.dtype))
                if a.shape[0] < hd + 1:
                    raise ValueError("the assistant turn must hold its header and at least one answer token")
                text = torch.cat([a[:hd], tts_pad[None].expand(4, -1), tts_bos[None], a[hd: hd + 1]])
                codec_ids = torch.tensor([cfg.codec_nothink_id, cfg.codec_think_bos_id, cfg.codec_think_eos_id, speaker,
                                          cfg.codec_pad_id, cfg.codec_bos_id], device=self.device)
                codec = torch.cat([torch.zeros((hd, a.shape[1]), device=self.device, dtype=self.dtype),
                                   self.decoder.embed_tokens(codec_ids.to(torch.int32))])
                parts.append(text + codec)
                trailing = torch.cat([a[hd + 1:], tts_eos[None]])
        if not parts:
            raise ValueError("no user or assistant turn found in the thinker's tokens")
        return torch.cat(parts), trailing, tts_pad

    # -- generation -----------------------------------------------------------------------------------------
    @torch.inference_mode()
    def generate(self, prefill: torch.Tensor, trailing: torch.Tensor, tts_pad: torch.Tensor, max_frames: int = 2048,
                 sample: bool = True, temperature: float = 0.9, top_k: int = 50, top_p: float = 1.0,
                 generator: torch.Generator | None = None, min_frames: int = 0) -> Iterator[torch.Tensor]:
        """Yields one frame of codes ``[num_code_groups]`` (int64) per step until the codec end token (which cannot be
        drawn during the first ``min_frames`` frames)."""
        cfg, dev = self.cfg, self.device
        G = cfg.num_code_groups
        total = prefill.shape[0] + max_frames + 1
        n_pages = -(-total // PAGE_SIZE)
        kv = self.decoder.alloc_kv_cache(n_pages + 1)
        pages = list(range(1, n_pages + 1))
        cp = self.code_predictor
        cp_kv = cp.model.alloc_kv_cache(2)
        # only the codec codes proper and the end token may be drawn
        allowed = torch.zeros(cfg.text.vocab_size, dtype=torch.bool, device=dev)
        allowed[: min(cfg.predictor.vocab_size, cfg.text.vocab_size)] = True
        if cfg.codec_eos_token_id < cfg.text.vocab_size:
            allowed[cfg.codec_eos_token_id] = True
        no_eos = allowed.clone()
        if cfg.codec_eos_token_id < cfg.text.vocab_size:
            no_eos[cfg.codec_eos_token_id] = False

        def pick(logits: torch.Tensor, mask: torch.Tensor | None, k: int, p: float) -> int:
            logits = logits.float().flatten()
            if mask is not None:
                logits = logits.masked_fill(~mask, float("-inf"))
            if not sample:
                return int(torch.argmax(logits))
            logits = logits / temperature
            if k > 0:
                kth = torch.topk(logits, min(k, logits.numel())).values[-1]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            probs = torch.softmax(logits, dim=-1)
            if p < 1.0:
                sp, si = torch.sort(probs, descending=True)
                keep = (torch.cumsum(sp, 0) - sp) < p
                probs = torch.zeros_like(probs).scatter_(0, si, sp * keep)
                probs = probs / probs.sum()
            return int(torch.multinomial(probs, 1, generator=generator))

        def step(model: QwenLLM, caches, x: torch.Tensor, start: int, pg: list[int]) -> torch.Tensor:
            m = _embeds_meta(x.shape[0], start, pg, dev, decode=True)
            m.mm_embeds = x.to(self.dtype).contiguous()
            m.mm_index = torch.arange(x.shape[0], dtype=torch.int32, device=dev)
            return model.forward_hidden(m, caches)

        h = step(self.decoder, kv, prefill, 0, pages)[-1:]
        pos = prefill.shape[0]
        for frame in range(max_frames):
            code0 = pick(self.decoder.compute_logits(h), allowed if frame >= min_frames else no_eos, top_k, top_p)
            if code0 == cfg.codec_eos_token_id:
                return
            e0 = self.decoder.embed_tokens(torch.tensor([code0], dtype=torch.int32, device=dev))
            codes, summed = [code0], e0.float()
            # residual codebooks: the predictor sees [talker hidden, embedding of code 0], then one code at a time
            hp = step(cp.model, cp_kv, torch.cat([h.to(self.dtype), e0]), 0, [1])[-1:]
            for gi in range(G - 1):
                c = pick(cp.heads[gi](hp, out_dtype=torch.float32), None, 50, 0.8)
                codes.append(c)
                e = cp.codec_embedding[gi](torch.tensor([c], dtype=torch.int32, device=dev))
                summed = summed + e.float()
                if gi + 1 < G - 1:
                    hp = step(cp.model, cp_kv, e, 2 + gi, [1])
            yield torch.tensor(codes, dtype=torch.int64)
            nxt = summed + (trailing[frame] if frame < trailing.shape[0] else tts_pad).float()
            h = step(self.decoder, kv, nxt.to(self.dtype), pos, pages)
            pos += 1

    # -- checkpoint loading (names under ``talker.``) --------------------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        loaded: set[str] = set()
        dec: list[tuple[str, torch.Tensor]] = []
        pred: list[tuple[str, torch.Tensor]] = []
        names: dict[str, str] = {}
        for name, t in weights:
            n = name[len("talker."):] if name.startswith("talker.") else name
            p = n.split(".")
            if p[0] in ("text_projection", "hidden_projection"):
                mlp: ResizeMLP = getattr(self, p[0])
                getattr(mlp.fc1 if p[1] == "linear_fc1" else mlp.fc2, p[2]).data.copy_(t)
            elif n == "codec_head.weight":
                dec.append(("lm_head.weight", t)); names["lm_head.weight"] = name
                continue
            elif n == "model.codec_embedding.weight":
                dec.append(("embed_tokens.weight", t)); names["embed_tokens.weight"] = name
                continue
            elif p[0] == "model":
                dec.append((n[len("model."):], t)); names[n[len("model."):]] = name
                continue
            elif n.startswith("code_predictor.model.codec_embedding."):
                self.code_predictor.codec_embedding[int(p[3])].weight.data.copy_(t)
            elif n.startswith("code_predictor.lm_head."):
                self.code_predictor.heads[int(p[2])].weight.data.copy_(t)
            elif n.startswith("code_predictor.model."):
                key = n[len("code_predictor.model."):]
                pred.append((key, t)); names["cp:" + key] = name
                continue
            else:
                continue
            loaded.add(name)
        loaded |= {names[k] for k in self.decoder.load_weights(dec)}
        loaded |= {names["cp:" + k] for k in self.code_predictor.model.load_weights(pred)}
        return loaded
