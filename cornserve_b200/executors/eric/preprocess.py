"""Image / video preprocessing for the Qwen2-VL family of vision towers.

Restates what the Hugging Face ``Qwen2VLImageProcessor`` does (the reference calls it through
``ModalityProcessor``: python/cornserve/task_executors/eric/models/base.py:93-148): resize to a
multiple of ``patch * merge`` within a pixel budget, rescale, normalise, duplicate still images along
time, and cut into ``[L, C * 2 * 14 * 14]`` patch rows ordered by 2x2 merge blocks.  Works on CPU or
CUDA tensors, so an executor can upload the raw uint8 frame (3 bytes/pixel) and do the rest on the GPU.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)


def smart_resize(height: int, width: int, factor: int = 28, min_pixels: int = 56 * 56,
                 max_pixels: int = 14 * 14 * 4 * 16384) -> tuple[int, int]:
    """Closest size with both sides divisible by ``factor`` and area within ``[min_pixels, max_pixels]``."""
    if max(height, width) / min(height, width) > 200:
        raise ValueError("aspect ratio above 200 is not supported")
    h = max(factor, round(height / factor) * factor)
    w = max(factor, round(width / factor) * factor)
    if h * w > max_pixels:
        beta = math.sqrt((height * width) / max_pixels)
        h = max(factor, math.floor(height / beta / factor) * factor)
        w = max(factor, math.floor(width / beta / factor) * factor)
    elif h * w < min_pixels:
        beta = math.sqrt(min_pixels / (height * width))
        h = math.ceil(height * beta / factor) * factor
        w = math.ceil(width * beta / factor) * factor
    return h, w


def patchify_frames(frames: torch.Tensor, patch: int = 14, temporal: int = 2, merge: int = 2,
                    out_dtype: torch.dtype = torch.bfloat16, min_pixels: int = 56 * 56,
                    max_pixels: int = 14 * 14 * 4 * 16384) -> tuple[torch.Tensor, tuple[int, int, int]]:
    """``frames``: uint8 ``[T, H, W, 3]`` (or ``[H, W, 3]`` for one image).

    Returns ``(pixel_values [L, 3 * temporal * patch * patch], (grid_t, grid_h, grid_w))``.
    """
    if frames.dim() == 3:
        frames = frames[None]
    T, H, W, C = frames.shape
    h, w = smart_resize(H, W, patch * merge, min_pixels, max_pixels)
    x = frames.permute(0, 3, 1, 2).float()
    if (h, w) != (H, W):
        x = F.interpolate(x, size=(h, w), mode="bicubic", align_corners=False, antialias=True)
        x = x.clamp_(0.0, 255.0)
    mean = torch.tensor(CLIP_MEAN, device=x.device).view(1, 3, 1, 1) * 255.0
    std = torch.tensor(CLIP_STD, device=x.device).view(1, 3, 1, 1) * 255.0
    x = (x - mean) / std
    if T % temporal != 0:
        x = torch.cat([x, x[-1:].expand(temporal - T % temporal, -1, -1, -1)], dim=0)
    gt, gh, gw = x.shape[0] // temporal, h // patch, w // patch
    x = x.reshape(gt, temporal, C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, C * temporal * patch * patch)
    return x.to(out_dtype), (gt, gh, gw)
