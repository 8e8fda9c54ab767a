"""Audio towers of Qwen2.5-Omni (Whisper-style Conv1d stem) and Qwen3-Omni (three stride-2 Conv2d layers), reference:
python/cornserve/task_executors/eric/models/qwen2_5_omni.py:100-300 and qwen3_omni_moe.py:500-720.

A mel spectrogram ``[mel, frames]`` is cut into fixed-size chunks, every chunk goes through the convolutional stem
(tap-gather kernel + tcgen05 GEMM with the GELU in its epilogue), sinusoidal positions are added in the last GEMM's
residual operand, the valid frames of all chunks are packed and run through LayerNorm transformer blocks whose
attention is confined to windows of chunks (var-len tcgen05 attention), and a small head maps to the LLM width.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable

import numpy as np
import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group
from .layers import LayerNorm, Linear, _param
from .vit import HF_ACT, BlockSpec, EncoderBlock, fused_tp_blocks, fused_tp_context, sinusoid_positions


@dataclass
class AudioEncoderConfig:
    num_mel_bins: int = 128
    d_model: int = 1280
    encoder_layers: int = 32
    encoder_attention_heads: int = 20
    encoder_ffn_dim: int = 5120
    activation_function: str = "gelu"
    max_source_positions: int = 1500
    n_window: int = 100
    output_dim: int = 3584
    # Qwen3-Omni only
    downsample_hidden_size: int = 480
    n_window_infer: int = 400
    conv2d_stem: bool = False

    @classmethod
    def from_hf(cls, cfg: dict, conv2d_stem: bool) -> "AudioEncoderConfig":
        a = cfg.get("audio_config") or (cfg.get("thinker_config") or {}).get("audio_config") or cfg
        kw = {k: a[k] for k in cls.__dataclass_fields__ if k in a}
        kw["conv2d_stem"] = conv2d_stem
        return cls(**kw)


def chunk_lengths(feature_len: int, chunk: int) -> list[int]:
    n = -(-feature_len // chunk)
    tail = feature_len % chunk or chunk
    return [chunk] * (n - 1) + [tail]


def qwen3_after_cnn_len(n: np.ndarray | int):
    """Frames left after the three stride-2 convolutions of the Qwen3-Omni stem (13 per full 100-frame chunk)."""
    n = np.asarray(n)
    leave = n % 100
    feat = (leave - 1) // 2 + 1
    return ((feat - 1) // 2 + 1 - 1) // 2 + 1 + (n // 100) * 13


class AudioEncoder(nn.Module):
    modalities = ("audio",)

    def __init__(self, cfg: AudioEncoderConfig, group: ParallelGroup | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        D, mel = cfg.d_model, cfg.num_mel_bins
        if cfg.conv2d_stem:
            C = cfg.downsample_hidden_size
            self.conv_w = nn.ParameterList([_param(C, 9 * 8, device=device, dtype=torch.bfloat16),
                                            _param(C, 9 * C, device=device, dtype=torch.bfloat16),
                                            _param(C, 9 * C, device=device, dtype=torch.bfloat16)])
            self.conv_b = nn.ParameterList([_param(C, device=device, dtype=torch.bfloat16, std=None) for _ in range(3)])
            self.freq_out = ((((mel + 1) // 2 + 1) // 2 + 1) // 2)
            self.conv_out = Linear(C * self.freq_out, D, bias=False, device=device)
            self.proj1 = Linear(D, D, device=device)
            self.proj2 = Linear(D, cfg.output_dim, device=device)
        else:
            self.conv_w = nn.ParameterList([_param(D, 3 * mel, device=device, dtype=torch.bfloat16),
                                            _param(D, 3 * D, device=device, dtype=torch.bfloat16)])
            self.conv_b = nn.ParameterList([_param(D, device=device, dtype=torch.bfloat16, std=None) for _ in range(2)])
            self.proj = Linear(D, cfg.output_dim, device=device)
        spec = BlockSpec(D, cfg.encoder_attention_heads, cfg.encoder_ffn_dim, norm="layer", eps=1e-5,
                         act=HF_ACT[cfg.activation_function])
        self.layers = nn.ModuleList([EncoderBlock(spec, self.group, device) for _ in range(cfg.encoder_layers)])
        self.ln_post = LayerNorm(D, 1e-5, device=device)
        self.register_buffer("positions", sinusoid_positions(cfg.max_source_positions, D).to(device), persistent=False)

    @property
    def dtype(self) -> torch.dtype:
        return self.ln_post.weight.dtype

    @property
    def device(self) -> torch.device:
        return self.ln_post.weight.device

    @property
    def chunk_shape(self) -> tuple[int, ...]:
        return (1, self.cfg.output_dim)

    def forward(self, modality: str, adapter_name: str | None, batch: dict[str, list]) -> list[torch.Tensor]:
        if modality != "audio":
            raise ValueError(f"unsupported modality {modality}")
        feats = batch.get("input_features") or batch["input_audio_features"]
        lens = batch.get("feature_lens") or batch.get("audio_feature_lengths") or [None] * len(feats)
        mels = []
        for f, n in zip(feats, lens):
            f = f.reshape(self.cfg.num_mel_bins, -1) if f.dim() != 2 else f
            mels.append(f[:, : int(n)] if n is not None else f)
        return self.encode(mels)

    # -- stems -------------------------------------------------------------------------------------------
    def _stem_conv1d(self, chunks: torch.Tensor, lens: np.ndarray) -> tuple[torch.Tensor, np.ndarray]:
        """``chunks`` [n, Tmax, mel] (zero padded) -> ([n, T2, D] with positions added, valid length per chunk)."""
        n, Tmax, mel = chunks.shape
        D = self.cfg.d_model
        x = chunks.reshape(n * Tmax, mel)
        x = ops.linear(ops.im2col1d(x, n, Tmax, Tmax, 3, -1), self.conv_w[0], self.conv_b[0], act="gelu")
        valid = (torch.arange(Tmax, device=x.device)[None, :] < torch.as_tensor(lens, device=x.device)[:, None])
        x = x * valid.reshape(-1, 1).to(x.dtype)
        T2 = (Tmax - 1) // 2 + 1
        cols = ops.im2col1d(x.contiguous(), n, Tmax, T2, 3, -1, stride=2)
        y = ops.linear(cols, self.conv_w[1], self.conv_b[1], act="gelu")
        y = y.view(n, T2, D) + self.positions[:T2].to(y.dtype)[None]
        return y, (lens - 1) // 2 + 1

    def _stem_conv2d(self, chunks: torch.Tensor, lens: np.ndarray) -> tuple[torch.Tensor, np.ndarray]:
        n, Tmax, mel = chunks.shape
        C = self.cfg.downsample_hidden_size
        # image with H = time, W = mel, one real channel padded to the 8-channel vector width of the gather kernel
        x = torch.zeros((n * Tmax * mel, 8), device=chunks.device, dtype=chunks.dtype)
        x[:, 0] = chunks.reshape(-1)
        H, W = Tmax, mel
        for w, b in zip(self.conv_w, self.conv_b):
            x = ops.conv3x3(x, w, b, n, H, W, stride=2, act="gelu")
            H, W = (H - 1) // 2 + 1, (W - 1) // 2 + 1
        y = self.conv_out(x.view(n * H, W * C)).view(n, H, -1)
        y = y + self.positions[:H].to(y.dtype)[None]
        return y, qwen3_after_cnn_len(lens)

    @torch.inference_mode()
    def encode(self, mels: list[torch.Tensor]) -> list[torch.Tensor]:
        cfg, dev = self.cfg, self.device
        chunk = cfg.n_window * 2
        per_audio = [chunk_lengths(int(m.shape[1]), chunk) for m in mels]
        lens = np.asarray([n for c in per_audio for n in c], dtype=np.int64)
        Tmax = int(lens.max())
        chunks = torch.zeros((len(lens), Tmax, cfg.num_mel_bins), device=dev, dtype=self.dtype)
        k = 0
        for m, cl in zip(mels, per_audio):
            mt = m.to(dev, self.dtype).t()
            off = 0
            for n in cl:
                chunks[k, :n] = mt[off: off + n]
                off += n
                k += 1
        y, after = (self._stem_conv2d if cfg.conv2d_stem else self._stem_conv1d)(chunks, lens)
        T2 = y.shape[1]
        keep = (torch.arange(T2, device=dev)[None, :] < torch.as_tensor(after, device=dev)[:, None]).reshape(-1)
        x = y.reshape(-1, cfg.d_model)[keep].contiguous()
        # attention windows: one chunk (Qwen2.5-Omni) or n_window_infer / (2 n_window) chunks' worth of frames
        audio_after = [int(np.sum(after[sum(len(c) for c in per_audio[:i]): sum(len(c) for c in per_audio[:i + 1])]))
                       for i in range(len(mels))]
        if cfg.conv2d_stem:
            win = T2 * (cfg.n_window_infer // chunk)
            seg = [w for n in audio_after for w in [win] * (n // win) + ([n % win] if n % win else [])]
        else:
            seg = [int(a) for a in after]
        cu = torch.from_numpy(np.concatenate([[0], np.cumsum(seg)]).astype(np.int32)).to(dev)
        max_len = max(seg)
        tp = fused_tp_context(self, self.group, cfg.d_model, x.shape[0], self.layers[0].spec)
        if tp is not None:
            x = fused_tp_blocks(tp, list(self.layers), x, None, [(cu, max_len)] * len(self.layers))
        else:
            for layer in self.layers:
                x = layer(x, None, cu, max_len)
        outs = []
        for h in x.split(audio_after, dim=0):
            if cfg.conv2d_stem:
                h = self.proj2(self.proj1(self.ln_post(h), act=HF_ACT[cfg.activation_function]))
            else:
                n2 = h.shape[0] // 2
                h = h[: 2 * n2].view(n2, 2, -1).float().mean(dim=1).to(h.dtype)  # average pooling over frame pairs
                h = self.proj(self.ln_post(h))
            outs.append(h)
        return outs

    # -- checkpoint loading (HF names below ``audio_tower.``) -------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        cfg = self.cfg
        loaded: set[str] = set()
        for name, t in weights:
            p = name.split(".")
            leaf = p[-1]
            if p[0] in ("conv1", "conv2") and not cfg.conv2d_stem:
                i = int(p[0][-1]) - 1
                if leaf == "weight":  # [out, in, k] -> [out, k*in]
                    self.conv_w[i].data.copy_(t.permute(0, 2, 1).reshape(t.shape[0], -1))
                else:
                    self.conv_b[i].data.copy_(t)
            elif p[0] in ("conv2d1", "conv2d2", "conv2d3") and cfg.conv2d_stem:
                i = int(p[0][-1]) - 1
                if leaf == "weight":  # [out, in, k_mel, k_time] -> taps (time, mel, in)
                    w = t.permute(0, 3, 2, 1)
                    if i == 0:
                        w = torch.nn.functional.pad(w, (0, 7))
                    self.conv_w[i].data.copy_(w.reshape(t.shape[0], -1))
                else:
                    self.conv_b[i].data.copy_(t)
            elif name == "conv_out.weight":
                C, Fq = cfg.downsample_hidden_size, self.freq_out
                self.conv_out.load(weight=t.view(-1, C, Fq).permute(0, 2, 1).reshape(t.shape[0], -1))
            elif p[0] in ("proj", "proj1", "proj2", "ln_post"):
                m = getattr(self, p[0])
                if p[0] == "ln_post":
                    getattr(m, leaf).data.copy_(t)
                else:
                    m.load(**{leaf: t})
            elif p[0] == "layers":
                blk: EncoderBlock = self.layers[int(p[1])]
                sub = ".".join(p[2:-1])
                if sub == "self_attn_layer_norm":
                    blk.load_norm(1, leaf, t)
                elif sub == "final_layer_norm":
                    blk.load_norm(2, leaf, t)
                elif sub in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                    blk.qkv.load(sub[-6], **{leaf: t})
                elif sub == "self_attn.out_proj":
                    blk.proj.load(**{leaf: t})
                elif sub in ("fc1", "fc2"):
                    blk.load_mlp(sub, leaf, t)
                else:
                    continue
            else:
                continue  # e.g. audio_bos_eos_token: used by the language model side, not by the encoder
            loaded.add(name)
        return loaded
