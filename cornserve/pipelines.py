"""In-process pipelines: the same executors' cores wired together without the HTTP control plane.

``MLLMPipeline`` is the monolithic ("no fission") form of the multimodal-LLM app: raw uint8 images in
pinned host memory -> GPU preprocessing -> vision tower -> embeddings placed into the LLM prompt ->
continuous-batching generation -> token ids on the host.  The served path runs the same two cores in
separate executor processes joined by the sidecar.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from .task_executors.eric.preprocess import patchify_frames
from .task_executors.llm.engine import EngineConfig, LLMEngine, MMItem, SamplingParams, Sequence
from .models.qwen2_5_vl import Qwen25VisionTransformer
from .models.qwen_llm import QwenLLM


@dataclass
class MLLMRequest:
    request_id: str
    prompt_ids: np.ndarray                      # text token ids (int32)
    images: list[torch.Tensor] = field(default_factory=list)   # uint8 [H, W, 3], ideally pinned host memory
    max_tokens: int = 256
    ignore_eos: bool = False


class MLLMPipeline:
    def __init__(self, vision: Qwen25VisionTransformer, llm: QwenLLM, engine_cfg: EngineConfig | None = None,
                 max_patches_per_encode: int = 40000, vision_end_token_id: int = 151653):
        self.vision, self.llm = vision, llm
        self.engine = LLMEngine(llm, engine_cfg)
        self.device = llm.device
        self.max_patches = max_patches_per_encode
        self.vision_end = vision_end_token_id
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    @torch.inference_mode()
    def encode_images(self, images: list[torch.Tensor]) -> list[tuple[torch.Tensor, tuple[int, int, int]]]:
        """uint8 HWC images (host or device) -> ``[(embeddings [n, H_llm], grid_thw)]``."""
        out: list[tuple[torch.Tensor, tuple[int, int, int]]] = []
        pix, grids, count = [], [], 0

        def flush():
            nonlocal pix, grids, count
            if not pix:
                return
            embs = self.vision("image", None, {"pixel_values": pix, "image_grid_thw": [list(g) for g in grids]})
            out.extend(zip(embs, grids))
            pix, grids, count = [], [], 0

        for img in images:
            if img.device != self.device:
                self.h2d_bytes += img.numel() * img.element_size()
                img = img.to(self.device, non_blocking=True)
            pv, g = patchify_frames(img, self.vision.cfg.patch_size, self.vision.cfg.temporal_patch_size,
                                    self.vision.cfg.spatial_merge_size, out_dtype=self.vision.dtype)
            if count + pv.shape[0] > self.max_patches:
                flush()
            pix.append(pv)
            grids.append(g)
            count += pv.shape[0]
        flush()
        return out

    def build_sequence(self, req: MLLMRequest, encoded: list[tuple[torch.Tensor, tuple[int, int, int]]]) -> Sequence:
        cfg = self.llm.cfg
        ids: list[np.ndarray] = []
        items: list[MMItem] = []
        off = 0
        for emb, grid in encoded:
            n = emb.shape[0]
            ids.append(np.array([cfg.vision_start_token_id], dtype=np.int32))
            ids.append(np.full(n, cfg.image_token_id, dtype=np.int32))
            ids.append(np.array([self.vision_end], dtype=np.int32))
            items.append(MMItem(emb, off + 1, grid))
            off += n + 2
        ids.append(np.asarray(req.prompt_ids, dtype=np.int32))
        return Sequence(req.request_id, np.concatenate(ids), SamplingParams(req.max_tokens, req.ignore_eos),
                        mm_items=items)

    def generate(self, requests: list[MLLMRequest]) -> dict[str, list[int]]:
        """Serve a batch of requests to completion; returns ``request_id -> generated token ids`` (host)."""
        all_imgs = [img for r in requests for img in r.images]
        for r in requests:
            self.h2d_bytes += int(np.asarray(r.prompt_ids).nbytes)
        encoded = self.encode_images(all_imgs)
        seqs, k = [], 0
        for r in requests:
            seqs.append(self.build_sequence(r, encoded[k: k + len(r.images)]))
            k += len(r.images)
        out = self.engine.generate(seqs)
        self.d2h_bytes += sum(len(v) for v in out.values()) * 4
        return out
