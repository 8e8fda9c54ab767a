"""Qwen3-Omni code-to-waveform vocoder (streaming audio generator).

Same network as the reference's vocoder, which it assembles from ``transformers`` building blocks
(python/cornserve/task_executors/geri/models/qwen3_omni_moe.py:32-220): mean of the quantizer code embeddings ->
sliding-window causal transformer -> transposed-conv + ConvNeXt upsamplers -> SnakeBeta / dilated causal-conv
decoder -> waveform in [-1, 1], generated chunk by chunk with a short left context.

Everything runs channels-last (``[B*T, C]`` bf16) on this library's kernels: the transformer uses the fused
GEMM / norm / rotary / windowed tcgen05 attention ops; every (transposed) convolution is a tap-gather kernel
(SnakeBeta applied while gathering) followed by the tcgen05 GEMM with bias and residual in its epilogue;
layer scales ride in the GEMM's gate operand.  Checkpoint names are the Hugging Face ones (``code2wav.``
prefix stripped).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Iterable, Iterator

import numpy as np
import torch
from torch import nn

from .. import ops
from .layers import Embedding, LayerNorm, Linear, RMSNorm, _param


@dataclass
class Code2WavConfig:
    codebook_size: int = 2048
    hidden_size: int = 1024
    num_attention_heads: int = 16
    num_key_value_heads: int = 16
    sliding_window: int = 72
    intermediate_size: int = 3072
    layer_scale_initial_scale: float = 0.01
    rms_norm_eps: float = 1e-5
    num_hidden_layers: int = 8
    num_quantizers: int = 16
    upsample_rates: tuple[int, ...] = (8, 5, 4, 3)
    upsampling_ratios: tuple[int, ...] = (2, 2)
    decoder_dim: int = 1536
    rope_theta: float = 10000.0

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def total_upsample(self) -> int:
        return int(np.prod(list(self.upsample_rates) + list(self.upsampling_ratios)))

    @classmethod
    def from_hf(cls, cfg: dict) -> "Code2WavConfig":
        c = cfg.get("code2wav_config", cfg)
        kw = {k: (tuple(c[k]) if isinstance(c[k], list) else c[k]) for k in cls.__dataclass_fields__ if k in c}
        rp = c.get("rope_parameters") or {}
        if "rope_theta" in rp:
            kw["rope_theta"] = rp["rope_theta"]
        return cls(**kw)


class Snake(nn.Module):
    """Parameters of ``x + sin^2(x e^alpha) / (e^beta + 1e-9)``; applied inside the tap-gather of the next conv."""

    def __init__(self, dim: int, device):
        super().__init__()
        self.alpha = _param(dim, device=device, dtype=torch.float32, std=None)
        self.beta = _param(dim, device=device, dtype=torch.float32, std=None)


class CausalConv1d(nn.Module):
    def __init__(self, cin: int, cout: int, k: int, dilation: int = 1, *, device, pad_out: int | None = None):
        super().__init__()
        self.cin, self.cout, self.k, self.dilation = cin, cout, k, dilation
        n = pad_out or cout
        self.weight = _param(n, k * cin, device=device, dtype=torch.bfloat16, std=(k * cin) ** -0.5)
        self.bias = _param(n, device=device, dtype=torch.bfloat16, std=None)
        if n != cout:
            self.weight.data[cout:].zero_()

    def forward(self, x, B, T, snake: Snake | None = None, residual=None):
        a, b = (snake.alpha, snake.beta) if snake is not None else (None, None)
        return ops.conv1d_causal(x, self.weight, self.bias, B, T, self.k, self.dilation, alpha=a, beta=b, residual=residual)

    def load(self, weight=None, bias=None):
        if weight is not None:  # [cout, cin, k] -> [cout, k*cin]
            self.weight.data[: self.cout].copy_(weight.permute(0, 2, 1).reshape(self.cout, -1))
        if bias is not None:
            self.bias.data[: self.cout].copy_(bias)


class CausalTransConv1d(nn.Module):
    """Transposed convolution with kernel ``k`` in {stride, 2*stride}, trimmed as the checkpoint's network does."""

    def __init__(self, cin: int, cout: int, k: int, stride: int, *, device):
        super().__init__()
        assert k in (stride, 2 * stride)
        self.cin, self.cout, self.k, self.stride = cin, cout, k, stride
        taps = k // stride
        self.weight = _param(stride * cout, taps * cin, device=device, dtype=torch.bfloat16, std=(taps * cin) ** -0.5)
        self.bias = _param(stride * cout, device=device, dtype=torch.bfloat16, std=None)

    def forward(self, x, B, T, snake: Snake | None = None):
        a, b = (snake.alpha, snake.beta) if snake is not None else (None, None)
        return ops.conv_transpose1d_causal(x, self.weight, self.bias, B, T, self.stride, self.k, alpha=a, beta=b)

    def load(self, weight=None, bias=None):
        s, co, ci = self.stride, self.cout, self.cin
        if weight is not None:  # [cin, cout, k]
            w = weight.permute(2, 1, 0)  # [k, cout, cin]
            self.weight.data[:, :ci].copy_(w[:s].reshape(s * co, ci))
            if self.k == 2 * s:
                self.weight.data[:, ci:].copy_(w[s:].reshape(s * co, ci))
        if bias is not None:
            self.bias.data.copy_(bias.repeat(s))


class ConvNeXtBlock(nn.Module):
    def __init__(self, dim: int, device):
        super().__init__()
        self.dw_weight = _param(dim, 7, device=device, dtype=torch.bfloat16, std=0.3)
        self.dw_bias = _param(dim, device=device, dtype=torch.bfloat16, std=None)
        self.norm = LayerNorm(dim, 1e-6, device=device)
        self.pw1 = Linear(dim, 4 * dim, device=device)
        self.pw2 = Linear(4 * dim, dim, device=device)
        self.gamma = _param(1, dim, device=device, dtype=torch.bfloat16, std=None)

    def forward(self, x, B, T):
        h = ops.dwconv1d(x, self.dw_weight, self.dw_bias, B, T)
        h = self.pw1(self.norm(h), act="gelu")
        return ops.linear(h, self.pw2.weight, self.pw2.bias, gate=self.gamma, gate_rows_per_batch=x.shape[0], residual=x)


class TransformerLayer(nn.Module):
    def __init__(self, cfg: Code2WavConfig, device):
        super().__init__()
        H, d = cfg.hidden_size, cfg.head_dim
        self.cfg = cfg
        self.input_norm = RMSNorm(H, cfg.rms_norm_eps, device=device)
        self.post_norm = RMSNorm(H, cfg.rms_norm_eps, device=device)
        self.qkv = Linear(H, (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * d, bias=False, device=device)
        self.o_proj = Linear(cfg.num_attention_heads * d, H, bias=False, device=device)
        self.gate_up = Linear(H, 2 * cfg.intermediate_size, bias=False, device=device)
        self.down = Linear(cfg.intermediate_size, H, bias=False, device=device)
        self.attn_scale = _param(1, H, device=device, dtype=torch.bfloat16, std=None)
        self.mlp_scale = _param(1, H, device=device, dtype=torch.bfloat16, std=None)
        self.attn_scale.data.fill_(cfg.layer_scale_initial_scale)
        self.mlp_scale.data.fill_(cfg.layer_scale_initial_scale)

    def forward(self, x, cs, cu, T):
        cfg = self.cfg
        hq, hkv, d = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        rows = x.shape[0]
        qkv = self.qkv(self.input_norm(x))
        ops.rope_(qkv[:, : (hq + hkv) * d].view(rows, hq + hkv, d), cs)
        q = qkv[:, : hq * d].view(rows, hq, d)
        k = qkv[:, hq * d: (hq + hkv) * d].view(rows, hkv, d)
        v = qkv[:, (hq + hkv) * d:].view(rows, hkv, d)
        a = ops.attention_varlen(q, k, v, cu, cu, T, causal=True, window=cfg.sliding_window)
        x = ops.linear(a.view(rows, hq * d), self.o_proj.weight, None, gate=self.attn_scale, gate_rows_per_batch=rows,
                       residual=x)
        h = ops.swiglu_linear(self.post_norm(x), self.gate_up.weight)
        return ops.linear(h, self.down.weight, None, gate=self.mlp_scale, gate_rows_per_batch=rows, residual=x)


class ResidualUnit(nn.Module):
    def __init__(self, dim: int, dilation: int, device):
        super().__init__()
        self.act1, self.conv1 = Snake(dim, device), CausalConv1d(dim, dim, 7, dilation, device=device)
        self.act2, self.conv2 = Snake(dim, device), CausalConv1d(dim, dim, 1, device=device)

    def forward(self, x, B, T):
        h = self.conv1(x, B, T, snake=self.act1)
        # kernel-size-1 convolution with SnakeBeta on its input and the unit's residual in the epilogue
        cols = ops.im2col1d(h, B, T, T, 1, 0, 1, self.act2.alpha, self.act2.beta)
        return ops.linear(cols, self.conv2.weight, self.conv2.bias, residual=x)


class DecoderBlock(nn.Module):
    def __init__(self, cin: int, cout: int, rate: int, device):
        super().__init__()
        self.act = Snake(cin, device)
        self.up = CausalTransConv1d(cin, cout, 2 * rate, rate, device=device)
        self.units = nn.ModuleList([ResidualUnit(cout, dil, device) for dil in (1, 3, 9)])

    def forward(self, x, B, T):
        x, T = self.up(x, B, T, snake=self.act)
        for u in self.units:
            x = u(x, B, T)
        return x, T


class Code2Wav(nn.Module):
    """``forward(codes [B, num_quantizers, T]) -> waveform [B, samples]`` and the chunked streaming ``generate``."""

    def __init__(self, cfg: Code2WavConfig | None = None, device="cpu"):
        super().__init__()
        self.cfg = cfg = cfg or Code2WavConfig()
        H = cfg.hidden_size
        self.code_embedding = Embedding(cfg.codebook_size * cfg.num_quantizers, H, device=device)
        self.layers = nn.ModuleList([TransformerLayer(cfg, device) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(H, cfg.rms_norm_eps, device=device)
        self.up_conv = nn.ModuleList([CausalTransConv1d(H, H, f, f, device=device) for f in cfg.upsampling_ratios])
        self.up_next = nn.ModuleList([ConvNeXtBlock(H, device) for _ in cfg.upsampling_ratios])
        self.dec_in = CausalConv1d(H, cfg.decoder_dim, 7, device=device)
        self.dec_blocks = nn.ModuleList([
            DecoderBlock(cfg.decoder_dim >> i, cfg.decoder_dim >> (i + 1), r, device)
            for i, r in enumerate(cfg.upsample_rates)])
        out_dim = cfg.decoder_dim >> len(cfg.upsample_rates)
        self.out_act = Snake(out_dim, device)
        self.out_conv = CausalConv1d(out_dim, 1, 7, device=device, pad_out=8)
        d = cfg.head_dim
        self.inv_freq = 1.0 / (cfg.rope_theta ** (np.arange(0, d, 2, dtype=np.float64) / d))

    @property
    def device(self) -> torch.device:
        return self.code_embedding.weight.device

    @property
    def dtype(self) -> torch.dtype:
        return self.code_embedding.weight.dtype

    @property
    def embedding_dim(self) -> int:
        return self.cfg.num_quantizers

    @torch.inference_mode()
    def forward(self, codes: torch.Tensor) -> torch.Tensor:
        cfg = self.cfg
        B, Q, T = codes.shape
        if Q != cfg.num_quantizers:
            raise ValueError(f"expected {cfg.num_quantizers} code layers, got {Q}")
        dev = self.device
        off = torch.arange(Q, device=dev).view(1, Q, 1) * cfg.codebook_size
        idx = (codes.to(dev) + off).permute(0, 2, 1).reshape(-1).to(torch.int32)  # [B*T*Q]
        emb = self.code_embedding(idx).view(B * T, Q, cfg.hidden_size)
        x = emb.float().mean(dim=1).to(self.dtype)
        ang = np.arange(T, dtype=np.float64)[:, None] * self.inv_freq[None, :]
        cs = torch.from_numpy(np.tile(np.stack([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32), (B, 1, 1))).to(dev)
        cu = torch.arange(B + 1, device=dev, dtype=torch.int32) * T
        for layer in self.layers:
            x = layer(x, cs, cu, T)
        x = self.norm(x)
        for conv, nxt in zip(self.up_conv, self.up_next):
            x, T = conv(x, B, T)
            x = nxt(x, B, T)
        x = self.dec_in(x, B, T)
        for blk in self.dec_blocks:
            x, T = blk(x, B, T)
        y = self.out_conv(x, B, T, snake=self.out_act)  # [B*T, 8], waveform in column 0
        return y[:, 0].float().clamp(-1, 1).view(B, T)

    def generate(self, prompt_embeds: list[torch.Tensor], chunk_size: int | None = None,
                 left_context_size: int | None = None) -> Iterator[list[torch.Tensor | None]]:
        """Streaming decode: ``prompt_embeds[i]`` holds the codes ``[num_quantizers, T_i]`` of request ``i``.  Each
        iteration yields one waveform chunk per request (``None`` once a request has run out of codes)."""
        chunk = chunk_size or 300
        ctx = left_context_size if left_context_size is not None else 25
        up = self.cfg.total_upsample
        lens = [int(c.shape[-1]) for c in prompt_embeds]
        start = 0
        while start < max(lens):
            live = [i for i, n in enumerate(lens) if start < n]
            c0 = ctx if start - ctx > 0 else start
            ends = [min(start + chunk, lens[i]) for i in live]
            width = max(ends) - (start - c0)
            batch = torch.zeros((len(live), self.cfg.num_quantizers, width), dtype=torch.long)
            for j, i in enumerate(live):
                seg = prompt_embeds[i][..., start - c0: ends[j]]
                batch[j, :, : seg.shape[-1]] = seg.to("cpu")
            wav = self(batch)  # causal network: right padding never changes earlier samples
            out: list[torch.Tensor | None] = [None] * len(lens)
            for j, i in enumerate(live):
                n_codes = ends[j] - (start - c0)
                out[i] = wav[j, c0 * up: self.output_length(n_codes)]
            yield out
            start += chunk

    def output_length(self, n_codes: int) -> int:
        """Waveform samples produced for ``n_codes`` input codes."""
        T = n_codes
        for f in self.cfg.upsampling_ratios:
            T *= f
        for r in self.cfg.upsample_rates:
            T = (T - 1) * r
        return T

    # -- checkpoint loading (HF names below ``code2wav.``) ------------------------------------------------
    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        cfg = self.cfg
        loaded: set[str] = set()
        d, hq, hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
        for name, t in weights:
            p = name.split(".")
            leaf = p[-1]
            try:
                if name == "code_embedding.weight":
                    self.code_embedding.weight.data.copy_(t)
                elif p[0] == "pre_transformer":
                    if p[1] == "norm":
                        self.norm.weight.data.copy_(t)
                    elif p[1] == "layers":
                        L: TransformerLayer = self.layers[int(p[2])]
                        sub = ".".join(p[3:-1])
                        if sub == "input_layernorm":
                            L.input_norm.weight.data.copy_(t)
                        elif sub == "post_attention_layernorm":
                            L.post_norm.weight.data.copy_(t)
                        elif sub in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                            lo = {"q": 0, "k": hq * d, "v": (hq + hkv) * d}[sub[-6]]
                            L.qkv.weight.data[lo: lo + t.shape[0]].copy_(t)
                        elif sub == "self_attn.o_proj":
                            L.o_proj.load(weight=t)
                        elif sub == "mlp.gate_proj":
                            L.gate_up.weight.data[: cfg.intermediate_size].copy_(t)
                        elif sub == "mlp.up_proj":
                            L.gate_up.weight.data[cfg.intermediate_size:].copy_(t)
                        elif sub == "mlp.down_proj":
                            L.down.load(weight=t)
                        elif sub == "self_attn_layer_scale":
                            L.attn_scale.data.copy_(t.view(1, -1))
                        elif sub == "mlp_layer_scale":
                            L.mlp_scale.data.copy_(t.view(1, -1))
                        else:
                            continue
                    else:
                        continue
                elif p[0] == "upsample":
                    i, j = int(p[1]), int(p[2])
                    if j == 0:
                        self.up_conv[i].load(**{leaf: t})
                    else:
                        nx: ConvNeXtBlock = self.up_next[i]
                        sub = ".".join(p[3:-1])
                        if sub == "dwconv.conv":
                            (nx.dw_weight if leaf == "weight" else nx.dw_bias).data.copy_(t.reshape(nx.dw_weight.shape) if leaf == "weight" else t)
                        elif sub == "norm":
                            (nx.norm.weight if leaf == "weight" else nx.norm.bias).data.copy_(t)
                        elif sub == "pwconv1":
                            nx.pw1.load(**{leaf: t})
                        elif sub == "pwconv2":
                            nx.pw2.load(**{leaf: t})
                        elif leaf == "gamma":
                            nx.gamma.data.copy_(t.view(1, -1))
                        else:
                            continue
                elif p[0] == "decoder":
                    i = int(p[1])
                    n_blocks = len(self.dec_blocks)
                    if i == 0:
                        self.dec_in.load(**{leaf: t})
                    elif i <= n_blocks:
                        blk: DecoderBlock = self.dec_blocks[i - 1]
                        j = int(p[3])  # decoder.i.block.j....
                        if j == 0:
                            getattr(blk.act, leaf).data.copy_(t)
                        elif j == 1:
                            blk.up.load(**{leaf: t})
                        else:
                            u: ResidualUnit = blk.units[j - 2]
                            which = p[4]
                            if which in ("act1", "act2"):
                                getattr(getattr(u, which), leaf).data.copy_(t)
                            else:
                                getattr(u, which).load(**{leaf: t})
                    elif i == n_blocks + 1:
                        getattr(self.out_act, leaf).data.copy_(t)
                    else:
                        self.out_conv.load(**{leaf: t})
                else:
                    continue
            except Exception as e:  # pragma: no cover
                raise RuntimeError(f"failed to load {name}: {e}") from e
            loaded.add(name)
        return loaded
