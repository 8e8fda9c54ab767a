"""PCM audio sink for streamed responses (reference: python/cornserve/cli/audio_streamer.py:11-175 plays through
PortAudio).  When the ``sounddevice`` module and an output device exist the chunks are played after a short
pre-buffer; otherwise (headless machines) they are collected and can be written out as a WAV file."""

from __future__ import annotations

import io
import queue
import threading
import wave


class PCMStreamPlayer:
    def __init__(self, sample_rate: int = 24000, channels: int = 1, sample_width: int = 2, prebuffer_s: float = 0.2,
                 play: bool = True) -> None:
        self.sample_rate, self.channels, self.sample_width = sample_rate, channels, sample_width
        self.prebuffer_bytes = int(prebuffer_s * sample_rate * channels * sample_width)
        self.collected = bytearray()
        self._q: queue.Queue[bytes | None] = queue.Queue()
        self._stream = None
        self._thread: threading.Thread | None = None
        if play:
            try:
                import sounddevice as sd  # noqa: F401

                dtype = {1: "int8", 2: "int16", 3: "int24", 4: "int32"}[sample_width]
                self._stream = sd.RawOutputStream(samplerate=sample_rate, channels=channels, dtype=dtype)
                self._thread = threading.Thread(target=self._pump, daemon=True)
                self._thread.start()
            except Exception:
                self._stream = None  # no audio stack on this machine: collect only

    @property
    def playing(self) -> bool:
        return self._stream is not None

    def _pump(self) -> None:
        pending = bytearray()
        started = False
        while True:
            item = self._q.get()
            if item is None:
                break
            pending += item
            if not started and len(pending) < self.prebuffer_bytes:
                continue
            if not started:
                self._stream.start()
                started = True
            self._stream.write(bytes(pending))
            pending.clear()
        if pending and self._stream is not None:
            if not started:
                self._stream.start()
            self._stream.write(bytes(pending))

    def feed(self, chunk: bytes) -> None:
        self.collected += chunk
        if self._stream is not None:
            self._q.put(chunk)

    def close(self) -> None:
        if self._thread is not None:
            self._q.put(None)
            self._thread.join(timeout=30)
        if self._stream is not None:
            try:
                self._stream.stop()
                self._stream.close()
            except Exception:
                pass

    def wav_bytes(self) -> bytes:
        buf = io.BytesIO()
        with wave.open(buf, "wb") as w:
            w.setnchannels(self.channels)
            w.setsampwidth(self.sample_width)
            w.setframerate(self.sample_rate)
            w.writeframes(bytes(self.collected))
        return buf.getvalue()

    def save_wav(self, path: str) -> None:
        with open(path, "wb") as f:
            f.write(self.wav_bytes())
