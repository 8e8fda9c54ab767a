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


_norm_cache: dict[tuple, tuple[torch.Tensor, torch.Tensor]] = {}


def _norm_constants(mean, std, device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """``(mean, std)`` of a recipe scaled to 0..255 as ``[1, 3, 1, 1]`` tensors on ``device``, made once per device:
    building a device tensor from Python numbers is a blocking copy that drains the stream it runs on."""
    key = (tuple(mean), tuple(std), str(device))
    got = _norm_cache.get(key)
    if got is None:
        got = _norm_cache[key] = (torch.tensor(mean, device=device).view(1, 3, 1, 1) * 255.0,
                                  torch.tensor(std, device=device).view(1, 3, 1, 1) * 255.0)
    return got


def patchify_frames(frames: torch.Tensor, patch: int = 14, temporal: int = 2, merge: int = 2,
                    out_dtype: torch.dtype = torch.bfloat16, min_pixels: int = 56 * 56,
                    max_pixels: int = 14 * 14 * 4 * 16384, mean=CLIP_MEAN, std=CLIP_STD) -> tuple[torch.Tensor, tuple[int, int, int]]:
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
    mean, std = _norm_constants(mean, std, x.device)
    x = (x - mean) / std
    if T % temporal != 0:
        x = torch.cat([x, x[-1:].expand(temporal - T % temporal, -1, -1, -1)], dim=0)
    gt, gh, gw = x.shape[0] // temporal, h // patch, w // patch
    x = x.reshape(gt, temporal, C, gh // merge, merge, patch, gw // merge, merge, patch)
    x = x.permute(0, 3, 6, 4, 7, 2, 1, 5, 8).reshape(gt * gh * gw, C * temporal * patch * patch)
    return x.to(out_dtype), (gt, gh, gw)


# ------------------------------------------------------------------------------------------------
# fixed-size and tiled image recipes (SigLIP / InternViT towers)
# ------------------------------------------------------------------------------------------------
IMAGENET_MEAN = (0.485, 0.456, 0.406)
IMAGENET_STD = (0.229, 0.224, 0.225)
HALF = (0.5, 0.5, 0.5)


def resize_normalize(frames: torch.Tensor, size: tuple[int, int], mean=HALF, std=HALF, mode: str = "bilinear",
                     out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """uint8 ``[T, H, W, 3]`` (or ``[H, W, 3]``) -> normalised ``[T, 3, size_h, size_w]``."""
    if frames.dim() == 3:
        frames = frames[None]
    x = frames.permute(0, 3, 1, 2).float()
    if tuple(x.shape[-2:]) != tuple(size):
        x = F.interpolate(x, size=size, mode=mode, align_corners=False, antialias=True).clamp_(0.0, 255.0)
    m, s = _norm_constants(mean, std, x.device)
    return ((x - m) / s).to(out_dtype)


def best_resolution(original: tuple[int, int], pinpoints: list[list[int]]) -> tuple[int, int]:
    """Any-resolution tiling: the ``(height, width)`` of ``pinpoints`` that keeps most pixels with least waste."""
    oh, ow = original
    best, best_eff, best_waste = None, 0, float("inf")
    for h, w in pinpoints:
        scale = min(w / ow, h / oh)
        eff = min(int(ow * scale) * int(oh * scale), ow * oh)
        waste = w * h - eff
        if eff > best_eff or (eff == best_eff and waste < best_waste):
            best, best_eff, best_waste = (h, w), eff, waste
    return best


def anyres_tiles(image: torch.Tensor, pinpoints: list[list[int]], tile: int, mean=HALF, std=HALF,
                 out_dtype: torch.dtype = torch.bfloat16) -> tuple[torch.Tensor, tuple[int, int]]:
    """LLaVA-OneVision tiling of one uint8 ``[H, W, 3]`` image: tile 0 is the whole image resized to ``tile`` x
    ``tile``; the rest is the image letter-boxed into the best multiple-of-tile canvas and cut into tiles.
    Returns ``([1 + n, 3, tile, tile], (H, W))``."""
    H, W, _ = image.shape
    bh, bw = best_resolution((H, W), pinpoints)
    scale = min(bw / W, bh / H)
    nw, nh = (bw, min(math.ceil(H * (bw / W)), bh)) if bw / W < bh / H else (min(math.ceil(W * (bh / H)), bw), bh)
    del scale
    x = image.permute(2, 0, 1)[None].float()
    body = F.interpolate(x, size=(nh, nw), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255)
    canvas = torch.zeros((1, 3, bh, bw), device=image.device)
    top, left = (bh - nh) // 2, (bw - nw) // 2
    canvas[:, :, top: top + nh, left: left + nw] = body
    tiles = canvas.view(1, 3, bh // tile, tile, bw // tile, tile).permute(0, 2, 4, 1, 3, 5).reshape(-1, 3, tile, tile)
    base = F.interpolate(x, size=(tile, tile), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255)
    allt = torch.cat([base, tiles], dim=0)
    m, s = _norm_constants(mean, std, image.device)
    return ((allt - m) / s).to(out_dtype), (H, W)


def dynamic_tiles(image: torch.Tensor, size: int = 448, min_num: int = 1, max_num: int = 12, thumbnail: bool = True,
                  out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """InternVL tiling of one uint8 ``[H, W, 3]`` image: resize to the grid of ``size``-pixel tiles whose aspect ratio
    is closest to the image's (at most ``max_num`` tiles), cut it, and append a thumbnail of the whole image."""
    H, W, _ = image.shape
    ratios = sorted({(i, j) for n in range(min_num, max_num + 1) for i in range(1, n + 1) for j in range(1, n + 1)
                     if min_num <= i * j <= max_num}, key=lambda r: r[0] * r[1])
    aspect, best, best_diff = W / H, (1, 1), float("inf")
    for r in ratios:
        diff = abs(aspect - r[0] / r[1])
        if diff < best_diff or (diff == best_diff and H * W > 0.5 * size * size * r[0] * r[1]):
            best, best_diff = r, diff
    gw, gh = best
    x = image.permute(2, 0, 1)[None].float()
    full = F.interpolate(x, size=(gh * size, gw * size), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255)
    tiles = full.view(1, 3, gh, size, gw, size).permute(0, 2, 4, 1, 3, 5).reshape(-1, 3, size, size)
    if thumbnail and tiles.shape[0] > 1:
        thumb = F.interpolate(x, size=(size, size), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 255)
        tiles = torch.cat([tiles, thumb], dim=0)
    m, s = _norm_constants(IMAGENET_MEAN, IMAGENET_STD, image.device)
    return ((tiles - m) / s).to(out_dtype)


# ------------------------------------------------------------------------------------------------
# audio: Whisper-style log-mel spectrogram
# ------------------------------------------------------------------------------------------------
def mel_filterbank(n_mels: int = 128, n_fft: int = 400, sampling_rate: int = 16000) -> torch.Tensor:
    """Slaney-scale triangular filters ``[n_mels, n_fft // 2 + 1]`` with Slaney normalisation."""
    import numpy as np

    def hz_to_mel(f):
        f = np.asarray(f, dtype=np.float64)
        mel = 3.0 * f / 200.0
        log_t = f >= 1000.0
        mel[log_t] = 15.0 + np.log(f[log_t] / 1000.0) * (27.0 / np.log(6.4))
        return mel

    def mel_to_hz(m):
        m = np.asarray(m, dtype=np.float64)
        f = 200.0 * m / 3.0
        log_t = m >= 15.0
        f[log_t] = 1000.0 * np.exp(np.log(6.4) / 27.0 * (m[log_t] - 15.0))
        return f

    fft_freqs = np.linspace(0, sampling_rate / 2, n_fft // 2 + 1)
    pts = mel_to_hz(np.linspace(hz_to_mel([0.0])[0], hz_to_mel([sampling_rate / 2.0])[0], n_mels + 2))
    diff = np.diff(pts)
    ramps = pts[:, None] - fft_freqs[None, :]
    lower, upper = -ramps[:-2] / diff[:-1, None], ramps[2:] / diff[1:, None]
    fb = np.maximum(0, np.minimum(lower, upper)) * (2.0 / (pts[2:] - pts[:-2]))[:, None]
    return torch.from_numpy(fb.astype(np.float32))


def log_mel_spectrogram(wave: torch.Tensor, n_mels: int = 128, n_fft: int = 400, hop: int = 160,
                        sampling_rate: int = 16000) -> torch.Tensor:
    """Mono waveform ``[samples]`` -> ``[n_mels, frames]`` as the Whisper feature extractor computes it (Hann
    window, power spectrum, mel filters, log10 clamped to 8 dB below the maximum, rescaled to about [-1, 1])."""
    wave = wave.float()
    window = torch.hann_window(n_fft, device=wave.device)
    spec = torch.stft(wave, n_fft, hop, window=window, return_complex=True)
    power = spec[..., :-1].abs() ** 2
    mel = mel_filterbank(n_mels, n_fft, sampling_rate).to(wave.device) @ power
    log = torch.clamp(mel, min=1e-10).log10()
    log = torch.maximum(log, log.max() - 8.0)
    return (log + 4.0) / 4.0
