"""Decoder-only LLM used by the own LLM executor: Qwen2 / Qwen2.5-VL / Qwen3 (dense and MoE) text models.

The reference delegates this part to a vLLM fork that is not in its tree (only the contract is:
tasklib/cornserve_tasklib/task_executors/descriptor/llm.py:68-210).  This is a from-scratch decoder
over a paged KV cache (128-token pages) driven by flattened, mixed prefill/decode batches:

  embed (+ scatter of encoder embeddings) -> L x [RMSNorm(+residual) -> qkv GEMM -> fused RoPE +
  KV-cache append -> paged tcgen05 attention -> o_proj GEMM -> RMSNorm(+residual) -> SwiGLU GEMM ->
  down GEMM] -> final norm -> lm_head GEMM on the last token of each sequence -> greedy arg-max.

M-RoPE (3-row position ids with sections) covers Qwen2.5-VL; plain RoPE is the special case of
three identical rows.  Tensor parallelism shards heads / MLP columns; row-parallel outputs are
reduced over the group.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Iterable

import torch
from torch import nn

from .. import ops
from ..parallel.state import ParallelGroup, single_group
from .layers import (ColumnParallelLinear, Embedding, Linear, MergedColumnParallelLinear, QKVParallelLinear,
                     RMSNorm, RowParallelLinear)

PAGE_SIZE = 128


@dataclass
class LLMConfig:
    hidden_size: int = 3584
    num_hidden_layers: int = 28
    num_attention_heads: int = 28
    num_key_value_heads: int = 4
    head_dim: int | None = None
    intermediate_size: int = 18944
    vocab_size: int = 152064
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    mrope_section: list[int] | None = field(default_factory=lambda: [16, 24, 24])
    attention_bias: bool = True
    qk_norm: bool = False
    tie_word_embeddings: bool = False
    # mixture of experts (0 experts = dense)
    num_experts: int = 0
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 768
    norm_topk_prob: bool = True
    shared_expert_intermediate_size: int = 0   # > 0: a dense expert with a sigmoid gate runs beside the routed ones
    # multimodal placeholder token ids (used by the executor to place encoder embeddings)
    image_token_id: int = 151655
    video_token_id: int = 151656
    vision_start_token_id: int = 151652
    eos_token_id: int = 151645
    spatial_merge_size: int = 2
    tokens_per_second: float | None = None   # Qwen2.5-VL: temporal positions of videos are in units of 1 / this; None = per frame

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads

    @classmethod
    def from_hf(cls, cfg: dict) -> "LLMConfig":
        t = dict(cfg.get("text_config") or cfg)
        for k in ("image_token_id", "video_token_id", "vision_start_token_id"):
            if k in cfg:
                t.setdefault(k, cfg[k])
        rs = t.get("rope_scaling") or cfg.get("rope_scaling") or t.get("rope_parameters") or {}
        kw = {k: t[k] for k in cls.__dataclass_fields__.keys() if k in t}
        if "mrope_section" in rs:
            kw["mrope_section"] = list(rs["mrope_section"])
        elif "mrope_section" not in kw:
            kw["mrope_section"] = None
        if "rope_theta" in rs:
            kw["rope_theta"] = rs["rope_theta"]
        mt = t.get("model_type", cfg.get("model_type", ""))
        if "qwen2_5_vl" in cfg.get("model_type", "") or "qwen2_5_vl" in mt or "qwen2_5_omni" in cfg.get("model_type", ""):
            kw.setdefault("tokens_per_second", float((cfg.get("vision_config") or {}).get("tokens_per_second", 2.0)))
        if "qwen3" in mt:
            kw.setdefault("qk_norm", True)
            kw.setdefault("attention_bias", t.get("attention_bias", False))
        if isinstance(kw.get("eos_token_id"), list):
            kw["eos_token_id"] = kw["eos_token_id"][0]
        if kw.get("eos_token_id") is None:
            kw.pop("eos_token_id", None)
        return cls(**kw)


@dataclass
class BatchMeta:
    """One engine step over a flattened batch of ``T`` tokens from ``B`` sequences."""

    input_ids: torch.Tensor        # [T] int32
    positions: torch.Tensor        # [3, T] int32
    slot_mapping: torch.Tensor     # [T] int32 (page * 128 + offset; -1 = do not cache)
    cu_q: torch.Tensor             # [B + 1] int32
    kv_len: torch.Tensor           # [B] int32, keys per sequence including this step's tokens
    block_table: torch.Tensor      # [B, max_blocks] int32
    logits_idx: torch.Tensor       # [B] int32, flattened index of each sequence's last token
    max_q_len: int = 1
    is_decode: bool = False
    # encoder rows to place into the input embeddings: per source tensor [n_i, H] the destination rows
    # [n_i] int32 (-1 = skip).  A source may live in another GPU's memory (a sidecar slab mapped through
    # CUDA IPC): the placement kernel then reads it over NVLink and writes the local embedding rows.
    mm_embeds: list[torch.Tensor] | torch.Tensor | None = None
    mm_index: list[torch.Tensor] | torch.Tensor | None = None


class Attention(nn.Module):
    def __init__(self, cfg: LLMConfig, group: ParallelGroup, device):
        super().__init__()
        self.cfg, self.group = cfg, group
        d = cfg.head_dim
        self.qkv = QKVParallelLinear(cfg.hidden_size, d, cfg.num_attention_heads, cfg.num_key_value_heads,
                                     bias=cfg.attention_bias, group=group, device=device)
        self.o_proj = RowParallelLinear(cfg.num_attention_heads * d, cfg.hidden_size, bias=False, group=group,
                                        device=device)
        self.hq, self.hkv = self.qkv.heads_local, self.qkv.kv_heads_local
        if cfg.qk_norm:
            self.q_norm = RMSNorm(d, cfg.rms_norm_eps, device=device)
            self.k_norm = RMSNorm(d, cfg.rms_norm_eps, device=device)

    def attend(self, h: torch.Tensor, cs: torch.Tensor, cache: torch.Tensor, m: BatchMeta) -> torch.Tensor:
        """Attention context ``[T, heads_local * d]`` (before the output projection)."""
        return self.attend_qkv(self.qkv(h), cs, cache, m)

    def attend_qkv(self, qkv: torch.Tensor, cs: torch.Tensor, cache: torch.Tensor, m: BatchMeta) -> torch.Tensor:
        """The same from an already projected ``q | k | v`` (``[T, (heads_local + 2 kv_heads_local) * d]``, changed in place)."""
        d = self.cfg.head_dim
        T = qkv.shape[0]
        if self.cfg.qk_norm:
            qk = qkv[:, : (self.hq + self.hkv) * d]
            normed_q = self.q_norm(qkv[:, : self.hq * d].reshape(-1, d)).view(T, self.hq * d)
            normed_k = self.k_norm(qkv[:, self.hq * d: (self.hq + self.hkv) * d].reshape(-1, d)).view(T, self.hkv * d)
            qk[:, : self.hq * d] = normed_q
            qk[:, self.hq * d:] = normed_k
        q = ops.rope_kv_write_(qkv, self.hq, self.hkv, d, cs, cache, m.slot_mapping)
        o = ops.attention_paged(q, cache, m.block_table, m.kv_len, m.cu_q, m.max_q_len, causal=True,
                                pack_gqa=m.is_decode and self.hq > self.hkv)
        return o.view(T, self.hq * d)

    def forward(self, h, cs, cache, m):
        return self.o_proj(self.attend(h, cs, cache, m))


class MLP(nn.Module):
    def __init__(self, cfg: LLMConfig, group: ParallelGroup, device, intermediate: int | None = None):
        super().__init__()
        inter = intermediate or cfg.intermediate_size
        self.gate_up = MergedColumnParallelLinear(cfg.hidden_size, inter, bias=False, group=group, device=device)
        self.down = RowParallelLinear(inter, cfg.hidden_size, bias=False, group=group,
                                      in_padded=self.gate_up.inter_padded, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.down(self.gate_up(x))


class SparseMoE(nn.Module):
    """Top-k routed experts.  Expert weights are stacked ``[E_local, ...]``; with expert parallelism each
    rank owns ``E / ep`` experts and tokens travel by all-to-all (see ``parallel.moe``)."""

    def __init__(self, cfg: LLMConfig, group: ParallelGroup, device):
        super().__init__()
        self.cfg, self.group = cfg, group
        E, H, inter = cfg.num_experts, cfg.hidden_size, cfg.moe_intermediate_size
        assert E % group.size == 0
        self.e_local = E // group.size
        self.router = Linear(H, E, bias=False, device=device)
        self.w_gate_up = nn.Parameter(torch.empty(self.e_local, 2 * inter, H, device=device, dtype=torch.bfloat16)
                                      .normal_(0, 0.02), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty(self.e_local, H, inter, device=device, dtype=torch.bfloat16)
                                   .normal_(0, 0.02), requires_grad=False)
        self.shared = None
        if cfg.shared_expert_intermediate_size > 0:
            self.shared = MLP(cfg, group, device, intermediate=cfg.shared_expert_intermediate_size)
            self.shared_gate = Linear(H, 1, bias=False, device=device)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y = self._routed(x)
        if self.shared is None:
            return y
        g = torch.sigmoid(torch.nn.functional.linear(x.float(), self.shared_gate.weight.float()))  # [T, 1]: too narrow for a tile
        return torch.addcmul(y.float(), g, self.shared(x).float()).to(x.dtype)

    def _routed(self, x: torch.Tensor) -> torch.Tensor:
        from ..parallel import moe

        logits = self.router(x, out_dtype=torch.float32)
        if x.is_cuda and (self.group.size == 1 or self.group.fabric is not None):
            cfg = self.cfg
            fm = moe.fused_layer(self.group, cfg.num_experts, cfg.num_experts_per_tok, cfg.hidden_size, cfg.moe_intermediate_size,
                                 -(-x.shape[0] // self.group.size), cfg.norm_topk_prob)
            # tensor-parallel ranks hold the same tokens: each routes a slice, the combine kernel fills every rank's output
            return fm.forward(x, logits, self.w_gate_up, self.w_down, replicated=self.group.size > 1)
        return moe.moe_forward(x, logits, self.w_gate_up, self.w_down, self.cfg.num_experts_per_tok,
                               self.cfg.norm_topk_prob, self.group)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: LLMConfig, group: ParallelGroup, device, ep_group: ParallelGroup | None = None):
        super().__init__()
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device)
        self.self_attn = Attention(cfg, group, device)
        self.mlp = SparseMoE(cfg, ep_group or group, device) if cfg.num_experts > 0 else MLP(cfg, group, device)

    def forward(self, h, residual, cs, cache, m: BatchMeta, next_norm: RMSNorm, fused=None):
        """``h`` = this layer's normalised input, ``residual`` = the un-normalised stream.  Returns the
        normalised input of the next layer (through ``next_norm``) and the updated residual stream.

        Each half (attention, MLP) ends in "row-parallel projection -> reduce over the group -> add residual
        -> RMSNorm".  With tensor parallelism and few tokens that whole tail is one fused kernel
        (``parallel.fused.FusedRowParallel``: the partial sums travel over NVLink from the GEMM epilogue);
        otherwise the projection's epilogue adds the residual and a norm kernel follows."""
        attn = self.self_attn.attend(h, cs, cache, m)
        h, residual = row_parallel_tail(attn, self.self_attn.o_proj, residual, self.post_attention_layernorm, fused)
        if isinstance(self.mlp, SparseMoE):
            y = self.mlp(h)
            h, residual = next_norm(y, residual=residual)
            return h, residual
        act = self.mlp.gate_up(h)
        return row_parallel_tail(act, self.mlp.down, residual, next_norm, fused)


def row_parallel_tail(x: torch.Tensor, proj: RowParallelLinear, residual: torch.Tensor, norm: RMSNorm, fused=None):
    """``residual' = all_reduce(x @ W^T) + residual`` and ``norm(residual')``; returns ``(normed, residual')``."""
    g = proj.group
    if g.size > 1 and fused is not None and x.is_cuda and x.shape[0] <= fused.m_cap:
        new_res, normed = fused(x, proj.weight, proj.bias, residual, norm.weight, norm.eps)
        return normed, new_res
    if g.size == 1:
        new_res = proj(x, residual=residual)  # residual add in the GEMM epilogue
        return norm(new_res), new_res
    y = proj(x)  # partial sums reduced by the library collective
    normed, new_res = norm(y, residual=residual)
    return normed, new_res


def dequantize_fp8_checkpoint(weights: Iterable[tuple[str, torch.Tensor]]) -> Iterable[tuple[str, torch.Tensor]]:
    """Pass checkpoint tensors through; an e4m3 ``X.weight`` is paired with its ``X.weight_scale_inv`` (one fp32 scale
    per 128 x 128 block, in whichever order the two arrive) and leaves as bf16 ``X.weight``."""
    pending: dict[str, torch.Tensor] = {}
    for name, t in weights:
        is_scale = name.endswith(".weight_scale_inv")
        if not is_scale and t.dtype != torch.float8_e4m3fn:
            yield name, t
            continue
        base = name[: -len("_scale_inv")] if is_scale else name
        other = pending.pop(base, None)
        if other is None:
            pending[base] = t
            continue
        q, sc = (other, t) if is_scale else (t, other)
        N, K = q.shape
        full = sc.float().repeat_interleave(128, dim=0)[:N].repeat_interleave(128, dim=1)[:, :K]
        yield base, (q.float() * full).to(torch.bfloat16)
    if pending:
        raise ValueError(f"fp8 checkpoint tensors without their partner: {sorted(pending)[:4]}")


class QwenLLM(nn.Module):
    def __init__(self, cfg: LLMConfig, group: ParallelGroup | None = None, device="cpu",
                 ep_group: ParallelGroup | None = None):
        super().__init__()
        self.cfg = cfg
        self.group = group or single_group(device)
        self.embed_tokens = Embedding(cfg.vocab_size, cfg.hidden_size, device=device)
        self.layers = nn.ModuleList([DecoderLayer(cfg, self.group, device, ep_group) for _ in range(cfg.num_hidden_layers)])
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, device=device)
        # tensor-parallel prefill through the peer-memory chain (GEMM -> reduce-scatter -> norm -> all-gather -> GEMM);
        # the engine raises the hint to its token budget so that the buffers are allocated once
        self.prefill_chain = True
        self.prefill_rows_hint = 2048
        if cfg.tie_word_embeddings:
            self.lm_head = None
        else:
            self.lm_head = ColumnParallelLinear(cfg.hidden_size, cfg.vocab_size, bias=False, group=self.group,
                                                pad_multiple=64, device=device)

    @property
    def device(self) -> torch.device:
        return self.embed_tokens.weight.device

    @property
    def kv_heads_local(self) -> int:
        return self.layers[0].self_attn.hkv

    def alloc_kv_cache(self, num_pages: int) -> list[torch.Tensor]:
        """One zero-initialised cache ``[pages, 2, Hkv_local, 128, d]`` per layer, all views of one allocation
        ``[layers, pages, 2, Hkv_local, 128, d]`` (kept as ``self.kv_backing``) so that another executor can map the
        whole cache with one handle and copy pages of every layer in one launch."""
        shape = (self.cfg.num_hidden_layers, num_pages, 2, self.kv_heads_local, PAGE_SIZE, self.cfg.head_dim)
        self.kv_backing = torch.zeros(shape, device=self.device, dtype=self.embed_tokens.weight.dtype)
        return list(self.kv_backing.unbind(0))

    def kv_bytes_per_page(self) -> int:
        return 2 * self.kv_heads_local * PAGE_SIZE * self.cfg.head_dim * 2 * self.cfg.num_hidden_layers

    def embed(self, m: BatchMeta) -> torch.Tensor:
        x = self.embed_tokens(m.input_ids)
        if m.mm_embeds is None:
            return x
        embeds = m.mm_embeds if isinstance(m.mm_embeds, (list, tuple)) else [m.mm_embeds]
        index = m.mm_index if isinstance(m.mm_index, (list, tuple)) else [m.mm_index]
        for rows, idx in zip(embeds, index, strict=True):
            if rows.shape[0] == 0:
                continue
            if rows.dtype != x.dtype or (x.is_cuda and not rows.is_cuda):
                rows = rows.to(device=x.device, dtype=x.dtype)
            ops.scatter_rows_(x, idx, rows)
        return x

    def forward_hidden(self, m: BatchMeta, kv_caches: list[torch.Tensor], capture: dict[int, torch.Tensor] | None = None) -> torch.Tensor:
        """Final-norm hidden states of every token ``[T, H]``.  ``capture``: keys are indices into the sequence
        "embeddings, output of layer 0, output of layer 1, ..." (un-normalised residual stream); the tensors are
        filled in."""
        cfg = self.cfg
        x = self.embed(m)
        if capture is not None and 0 in capture:
            capture[0] = x.clone()
        half = cfg.head_dim // 2
        sections = cfg.mrope_section or [half, 0, 0]
        cs = ops.mrope_table(m.positions, half, cfg.rope_theta, sections)
        if capture is None and not m.is_decode and x.shape[0] > 256:
            chain = self._fused_chain(x.shape[0])
            if chain is not None:
                return self._forward_hidden_chain(chain, x, cs, kv_caches, m)
        residual = x
        h = self.layers[0].input_layernorm(x)
        fused = self._fused_tail() if (self.group.size > 1 and x.is_cuda) else None
        n = len(self.layers)
        for i, (layer, cache) in enumerate(zip(self.layers, kv_caches)):
            next_norm = self.layers[i + 1].input_layernorm if i + 1 < n else self.norm
            h, residual = layer(h, residual, cs, cache, m, next_norm, fused)
            if capture is not None and i + 1 in capture:
                capture[i + 1] = residual.clone()
        return h

    def _fused_chain(self, rows: int):
        """Peer-memory context of the tensor-parallel prefill chain, or ``None`` when it does not apply (one rank, no
        fabric, experts, quantised projections).  Every rank sees the same sequence of row counts, so the buffers are
        (re)allocated by all ranks at the same step."""
        if (self.group.size == 1 or self.group.fabric is None or self.cfg.num_experts > 0 or self.device.type != "cuda"
                or getattr(self, "quantization", None) is not None or not self.prefill_chain
                or self.cfg.hidden_size > 4096):   # the reduce + norm kernel keeps a row in registers: up to 4096 wide
            return None
        ctx = getattr(self, "_chain", None)
        if ctx is None or ctx.S_cap < rows:
            from ..parallel.fused import FusedEncoderTP

            ctx = self._chain = FusedEncoderTP(self.group, self.cfg.hidden_size, max(rows, self.prefill_rows_hint))
        return ctx

    def _forward_hidden_chain(self, tp, x: torch.Tensor, cs: torch.Tensor, kv_caches: list[torch.Tensor], m: BatchMeta) -> torch.Tensor:
        """Prefill with the residual stream sharded by rows over the tensor-parallel ranks and no library collective
        inside the layers: each row-parallel projection (o_proj, down_proj) pushes its partial tiles from the GEMM
        epilogue to the rank that owns the rows (the reduce-scatter is the store), one kernel per owned row reduces them,
        adds the residual, applies the next RMSNorm and stores the normalised row into every rank's operand buffer (the
        all-gather is that store), and the following column-parallel GEMM (q|k|v, gate/up) starts on each 128-row chunk
        as soon as it has landed.  Attention runs between them on all tokens of this rank's heads, as without the chain.
        One library all-gather of the residual shards at the end gives every rank the full rows for the final norm."""
        import torch.distributed as dist

        T = x.shape[0]
        tp.begin(T)
        lo, hi = tp.row_range
        xs = x[lo:hi].contiguous()
        layers = self.layers
        n = len(layers)
        tp.reduce_norm_push(bias=None, residual=xs, dst=0, reduce=False, norm_w=layers[0].input_layernorm.weight,
                            eps=layers[0].input_layernorm.eps)
        for i, (layer, cache) in enumerate(zip(layers, kv_caches)):
            at, mlp = layer.self_attn, layer.mlp
            qkv = tp.gemm_gathered(0, at.qkv.weight, at.qkv.bias)
            o = at.attend_qkv(qkv, cs, cache, m)
            tp.gemm_push(o, at.o_proj.weight)
            pn = layer.post_attention_layernorm
            xs = tp.reduce_norm_push(bias=at.o_proj.bias, residual=xs, dst=1, norm_w=pn.weight, eps=pn.eps)
            act = tp.gemm_gathered(1, mlp.gate_up.weight, mlp.gate_up.bias, act="silu", swiglu=True)
            tp.gemm_push(act, mlp.down.weight)
            if i + 1 < n:
                nn_ = layers[i + 1].input_layernorm
                xs = tp.reduce_norm_push(bias=mlp.down.bias, residual=xs, dst=0, norm_w=nn_.weight, eps=nn_.eps)
            else:
                xs = tp.reduce_norm_push(bias=mlp.down.bias, residual=xs, norm_w=None, eps=0.0, dst=None)
        full = torch.zeros((tp.group.size * tp.R, x.shape[1]), device=x.device, dtype=x.dtype)
        mine = full[lo: lo + tp.R]
        mine[: xs.shape[0]] = xs
        dist.all_gather_into_tensor(full, mine.clone(), group=tp.group.group)
        return self.norm(full[:T])

    def _fused_tail(self):
        """Lazily built fused GEMM + all-reduce + residual + RMSNorm kernel context (needs the fabric)."""
        if getattr(self, "quantization", None) is not None:
            return None
        if getattr(self, "_fused", None) is None and self.group.fabric is not None:
            from ..parallel.fused import FusedRowParallel

            self._fused = FusedRowParallel(self.group, self.cfg.hidden_size, m_cap=256)
        return getattr(self, "_fused", None)

    def compute_logits(self, h_last: torch.Tensor) -> torch.Tensor:
        if self.lm_head is None:
            return ops.linear(h_last, self.embed_tokens.weight, out_dtype=torch.float32)
        logits = ops.linear(h_last, self.lm_head.weight, out_dtype=torch.float32)
        if self.group.size > 1:
            logits = self.group.all_gather(logits, dim=-1)
        return logits[:, : self.cfg.vocab_size]

    def forward(self, m: BatchMeta, kv_caches: list[torch.Tensor], return_hidden: bool = False,
                capture: dict[int, torch.Tensor] | None = None, sampler: tuple | None = None,
                penalties: tuple | None = None, logprobs: tuple | None = None):
        """Returns ``(next_token_ids [B] int32, hidden [T, H] or None)``.  Greedy unless ``sampler`` gives the per-row
        ``(temperature, top_p, top_k, seed, draws)`` tensors of :func:`ops.sample_rows` (every tensor-parallel rank
        holds the same gathered logits and the same streams, so all ranks draw the same token).

        ``logprobs`` = ``(chosen [S, B] f32, top_values [S, B, K] f32, top_ids [S, B, K] i32, step [1] i32)``: the log
        probability of the chosen token and the ``K`` most likely ones (of the distribution after penalties, before
        temperature) are written at index ``step`` -- a device value, so the same launches serve every step of a
        captured decode burst."""
        h = self.forward_hidden(m, kv_caches, capture)
        h_last = ops.gather_rows(h, m.logits_idx)
        logits = self.compute_logits(h_last)
        if penalties is not None:
            # (counts [B, V] int32, frequency [B], presence [B], active [B] or None): repetition control on the logits,
            # then the chosen token is added to its row's counts
            counts, freq, pres, active = penalties
            ops.apply_penalties_(logits, counts, freq, pres)
        lsm = torch.log_softmax(logits, dim=-1) if logprobs is not None else None   # before the sampler touches the logits
        tok = ops.argmax(logits) if sampler is None else ops.sample_rows(logits, *sampler)
        if penalties is not None:
            ops.count_tokens_(counts, tok, active)
        if logprobs is not None:
            chosen, top_v, top_i, step = logprobs
            at = step.long()
            chosen.index_copy_(0, at, lsm.gather(1, tok.long().unsqueeze(1)).view(1, -1))
            tv, ti = lsm.topk(top_v.shape[-1], dim=-1)
            top_v.index_copy_(0, at, tv.unsqueeze(0))
            top_i.index_copy_(0, at, ti.to(torch.int32).unsqueeze(0))
        return tok, (h if return_hidden else None)

    # -- checkpoint loading -------------------------------------------------------------------------
    def quantize_fp8_(self) -> "QwenLLM":
        """Store the attention and dense-MLP projections as e4m3 with 128 x 128 block scales (half the weight memory);
        their GEMMs then run the block-scaled tcgen05 kernel with activations quantised per row and 128 columns.
        Embeddings, lm_head, norms, the router and the stacked expert weights stay bf16; the fused tensor-parallel
        tail (which streams bf16 weights) is switched off in favour of the library reduction."""
        from .layers import quantize_fp8_

        for layer in self.layers:
            quantize_fp8_(layer.self_attn.qkv)
            quantize_fp8_(layer.self_attn.o_proj)
            mlps = [layer.mlp] if isinstance(layer.mlp, MLP) else ([layer.mlp.shared] if layer.mlp.shared is not None else [])
            for mlp in mlps:
                quantize_fp8_(mlp.gate_up)
                quantize_fp8_(mlp.down)
        self.quantization = "fp8"
        return self

    def load_weights(self, weights: Iterable[tuple[str, torch.Tensor]]) -> set[str]:
        """Accepts HF names with or without the ``model.`` / ``model.language_model.`` prefixes.  Block-scaled fp8
        checkpoints (``*.weight`` in e4m3 with ``*.weight_scale_inv``) are widened to bf16 on the way in; call
        :meth:`quantize_fp8_` afterwards to serve them in fp8."""
        loaded: set[str] = set()
        for name, t in dequantize_fp8_checkpoint(weights):
            n = name
            for pre in ("model.language_model.", "language_model.model.", "language_model.", "model.", "thinker.model."):
                if n.startswith(pre):
                    n = n[len(pre):]
                    break
            p = n.split(".")
            leaf = p[-1]
            if n == "embed_tokens.weight":
                self.embed_tokens.weight.data.copy_(t)
            elif n == "norm.weight":
                self.norm.weight.data.copy_(t)
            elif n in ("lm_head.weight", "head.weight") or name == "lm_head.weight":
                if self.lm_head is not None:
                    self.lm_head.load(weight=t)
            elif p[0] == "layers":
                layer: DecoderLayer = self.layers[int(p[1])]
                sub = ".".join(p[2:-1])
                kw = {leaf: t}
                if sub == "input_layernorm":
                    layer.input_layernorm.weight.data.copy_(t)
                elif sub == "post_attention_layernorm":
                    layer.post_attention_layernorm.weight.data.copy_(t)
                elif sub in ("self_attn.q_proj", "self_attn.k_proj", "self_attn.v_proj"):
                    layer.self_attn.qkv.load(sub[-6], **kw)
                elif sub == "self_attn.o_proj":
                    layer.self_attn.o_proj.load(**kw)
                elif sub == "self_attn.q_norm":
                    layer.self_attn.q_norm.weight.data.copy_(t)
                elif sub == "self_attn.k_norm":
                    layer.self_attn.k_norm.weight.data.copy_(t)
                elif sub == "mlp.gate_proj":
                    layer.mlp.gate_up.load("gate", **kw)
                elif sub == "mlp.up_proj":
                    layer.mlp.gate_up.load("up", **kw)
                elif sub == "mlp.down_proj":
                    layer.mlp.down.load(**kw)
                elif sub == "mlp.gate":
                    layer.mlp.router.load(weight=t)
                elif sub == "mlp.shared_expert_gate":
                    layer.mlp.shared_gate.weight.data.copy_(t)
                elif sub in ("mlp.shared_expert.gate_proj", "mlp.shared_expert.up_proj"):
                    layer.mlp.shared.gate_up.load("gate" if "gate_proj" in sub else "up", **kw)
                elif sub == "mlp.shared_expert.down_proj":
                    layer.mlp.shared.down.load(**kw)
                elif n.endswith("mlp.experts.gate_up_proj") or n.endswith("mlp.experts.down_proj"):
                    # stacked form: [E, 2I, H] (gate rows then up rows) and [E, H, I]
                    moe_l: SparseMoE = layer.mlp
                    lo = moe_l.group.rank * moe_l.e_local
                    dst = moe_l.w_gate_up if leaf == "gate_up_proj" else moe_l.w_down
                    dst.data.copy_(t[lo: lo + moe_l.e_local])
                elif sub.startswith("mlp.experts."):
                    e = int(p[4])
                    moe: SparseMoE = layer.mlp
                    lo = moe.group.rank * moe.e_local
                    if not (lo <= e < lo + moe.e_local):
                        continue
                    inter = self.cfg.moe_intermediate_size
                    which = p[5]
                    if which == "gate_proj":
                        moe.w_gate_up.data[e - lo, :inter].copy_(t)
                    elif which == "up_proj":
                        moe.w_gate_up.data[e - lo, inter:].copy_(t)
                    elif which == "down_proj":
                        moe.w_down.data[e - lo].copy_(t)
                else:
                    continue
            else:
                continue
            loaded.add(name)
        return loaded
