"""Loading and preprocessing of multimodal inputs on the CPU side of the encoder executor.

Reference: python/cornserve/task_executors/eric/router/processor.py:46-369.  URLs may be ``http(s)://``,
``data:<mime>;base64,<payload>`` or ``file://``.  Images are decoded with Pillow, videos with OpenCV
(uniformly sampled down to ``max_num_frames``; ``data:video/jpeg;base64,a,b,c`` carries a list of JPEG
frames), audio from WAV / raw float32 with resampling.  Decoding runs in a thread pool; the result is
the uint8 pixel data (or waveform) that the worker turns into model inputs on the GPU.
"""

from __future__ import annotations

import asyncio
import base64
import io
import wave
from concurrent.futures import ThreadPoolExecutor
from urllib.parse import urlparse
from urllib.request import urlopen

import numpy as np
import torch

from .config import ModalityConfig
from .schema import Modality, ProcessedItem


def fetch_bytes(url: str, timeout: float = 30.0) -> tuple[bytes, str]:
    """``(payload, mime)`` of a URL."""
    if url.startswith("data:"):
        header, _, payload = url.partition(",")
        mime = header[5:].split(";")[0]
        if ";base64" in header:
            return base64.b64decode(payload), mime
        return payload.encode(), mime
    u = urlparse(url)
    if u.scheme == "file" or u.scheme == "":
        with open(u.path if u.scheme else url, "rb") as f:
            return f.read(), ""
    if u.scheme in ("http", "https"):
        with urlopen(url, timeout=timeout) as r:  # noqa: S310
            return r.read(), r.headers.get_content_type()
    raise ValueError(f"Unsupported URL scheme: {u.scheme}")


def load_image(url: str) -> np.ndarray:
    """RGB uint8 ``[H, W, 3]``."""
    from PIL import Image

    if url.startswith("synthetic:"):  # synthetic:<H>x<W>[:seed] -- uniform random pixels, for load tests
        spec = url.split(":")
        h, w = (int(v) for v in spec[1].split("x"))
        rng = np.random.default_rng(int(spec[2]) if len(spec) > 2 else 0)
        return rng.integers(0, 256, (h, w, 3), dtype=np.uint8)
    data, _ = fetch_bytes(url)
    return np.asarray(Image.open(io.BytesIO(data)).convert("RGB"))


def load_video(url: str, max_num_frames: int) -> np.ndarray:
    """RGB uint8 ``[T, H, W, 3]`` with at most ``max_num_frames`` uniformly spaced frames."""
    import cv2

    if url.startswith("data:video/jpeg"):
        _, _, payload = url.partition(",")
        frames = [load_image("data:image/jpeg;base64," + p) for p in payload.split(",") if p]
    else:
        data, _ = fetch_bytes(url)
        import os
        import tempfile

        with tempfile.NamedTemporaryFile(suffix=".mp4", delete=False) as f:
            f.write(data)
            path = f.name
        try:
            cap = cv2.VideoCapture(path)
            frames = []
            while True:
                ok, frame = cap.read()
                if not ok:
                    break
                frames.append(cv2.cvtColor(frame, cv2.COLOR_BGR2RGB))
            cap.release()
        finally:
            os.unlink(path)
    if not frames:
        raise ValueError("video has no frames")
    if len(frames) > max_num_frames:
        idx = np.linspace(0, len(frames) - 1, max_num_frames).round().astype(int)
        frames = [frames[i] for i in idx]
    return np.stack(frames)


def load_audio(url: str, sampling_rate: int) -> np.ndarray:
    """Mono float32 waveform at ``sampling_rate``."""
    if url.startswith("synthetic:"):  # synthetic:<seconds>[:seed] -- Gaussian noise
        spec = url.split(":")
        rng = np.random.default_rng(int(spec[2]) if len(spec) > 2 else 0)
        return rng.standard_normal(int(float(spec[1]) * sampling_rate)).astype(np.float32)
    data, mime = fetch_bytes(url)
    if data[:4] == b"RIFF":
        with wave.open(io.BytesIO(data)) as w:
            sr, ch, width = w.getframerate(), w.getnchannels(), w.getsampwidth()
            raw = w.readframes(w.getnframes())
        dt = {1: np.uint8, 2: np.int16, 4: np.int32}[width]
        x = np.frombuffer(raw, dtype=dt).astype(np.float32)
        x = (x - 128.0) / 128.0 if width == 1 else x / float(2 ** (8 * width - 1))
        x = x.reshape(-1, ch).mean(axis=1)
    else:
        x, sr = np.frombuffer(data, dtype=np.float32).copy(), sampling_rate
    if sr != sampling_rate:
        from scipy.signal import resample_poly
        from math import gcd

        g = gcd(sr, sampling_rate)
        x = resample_poly(x, sampling_rate // g, sr // g).astype(np.float32)
    return x


def to_model_inputs(recipe: str, modality: Modality, raw: np.ndarray) -> dict[str, torch.Tensor]:
    """Raw decoded data -> the keys a model's ``forward`` reads.  The expensive part (resize, normalise,
    patchify) is deferred to the worker, which does it on the GPU; here only the tensor is wrapped."""
    t = torch.from_numpy(np.ascontiguousarray(raw))
    if recipe == "qwen2_vl":
        if modality == Modality.IMAGE:
            return {"raw_images": t}
        if modality == Modality.VIDEO:
            return {"raw_videos": t}
    if modality == Modality.AUDIO:
        return {"raw_audio": t}
    return {f"raw_{modality.value}": t}


class Processor:
    def __init__(self, recipe: str, config: ModalityConfig) -> None:
        self.recipe = recipe
        self.config = config
        self.pool = ThreadPoolExecutor(max_workers=config.num_workers, thread_name_prefix="eric-proc")

    def _load(self, modality: Modality, url: str) -> np.ndarray:
        if modality == Modality.IMAGE:
            return load_image(url)
        if modality == Modality.VIDEO:
            return load_video(url, self.config.video_config.max_num_frames)
        if modality == Modality.AUDIO:
            return load_audio(url, self.config.audio_config.sampling_rate)
        raise ValueError(f"unsupported modality {modality}")

    def _one(self, item_id: str, modality: Modality, model_id: str, url: str, ranks) -> ProcessedItem:
        return ProcessedItem(item_id, modality, model_id, to_model_inputs(self.recipe, modality, self._load(modality, url)), ranks)

    async def process(self, items: list[tuple[str, Modality, str, str, list[list[int]] | None]]) -> list[ProcessedItem]:
        loop = asyncio.get_running_loop()
        return list(await asyncio.gather(*(loop.run_in_executor(self.pool, self._one, *it) for it in items)))

    def shutdown(self) -> None:
        self.pool.shutdown(wait=False, cancel_futures=True)
