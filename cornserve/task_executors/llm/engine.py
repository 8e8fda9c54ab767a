"""LLM engine: request queue, paged-KV scheduling, batch construction, CUDA-graph decode.

This is the in-process core of the LLM executor (the reference uses an external vLLM fork for this
role; its contract is in tasklib/cornserve_tasklib/task_executors/descriptor/llm.py:68-210).

Prefill/decode disaggregation: a sequence with ``hold_kv`` keeps its pages after it finished (the prefill executor's
one-token requests); ``kv_transfer_params`` describes them, ``release_held`` frees them.  A sequence that arrives
with ``prefilled`` set skips the prompt computation: its pages are pulled from the producer's cache by one copy
kernel (``ops.kv_copy_pages``: over NVLink / CUDA IPC) or filled from bytes fetched over the network.

Scheduling: first-come-first-served.  A step is either a *prefill* step (waiting prompts, possibly
chunked, packed up to ``max_batched_tokens`` tokens) or a *decode burst* (``decode_burst`` tokens for
every running sequence).  During a burst the sampled token, the positions, the key counts and the
cache slots are advanced on the device, the whole step is replayed from a CUDA graph, and the host
reads the produced tokens once per burst.
"""

from __future__ import annotations

import enum
import random
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Iterable

import numpy as np
import torch

from ... import ops
from ...models.qwen_llm import PAGE_SIZE, BatchMeta, LLMConfig, QwenLLM
from .block_manager import BlockManager
from .mrope import mrope_positions


MAX_TOP_LOGPROBS = 20   # as the OpenAI API allows


@dataclass
class SamplingParams:
    max_tokens: int = 256
    ignore_eos: bool = False
    stop_token_ids: tuple[int, ...] = ()
    temperature: float = 0.0      # 0 = greedy (arg-max); > 0 samples from softmax(logits / temperature)
    top_p: float = 1.0            # nucleus: smallest set of most likely tokens whose mass reaches top_p
    top_k: int = 0                # <= 0: off
    seed: int | None = None       # names the request's random stream; None = drawn once when the request is added
    frequency_penalty: float = 0.0   # OpenAI semantics: a token generated c times loses frequency_penalty * c ...
    presence_penalty: float = 0.0    # ... and presence_penalty once it was generated at all
    logprobs: int = -1               # -1: off; k >= 0: report the chosen token's log probability and the k most likely tokens

    @classmethod
    def from_request(cls, body: dict, default_temperature: float = 1.0, **kw) -> "SamplingParams":
        """OpenAI-style request fields.  A request without ``temperature`` samples at ``default_temperature`` (1.0 as
        in the OpenAI API unless the model's ``generation_config.json`` says otherwise); ``temperature: 0`` is greedy."""
        t = body.get("temperature")
        k = body.get("top_k")
        seed = body.get("seed")
        lp = body.get("logprobs")
        if lp is True:      # chat completions: a switch plus ``top_logprobs``
            kw.setdefault("logprobs", max(0, min(MAX_TOP_LOGPROBS, int(body.get("top_logprobs") or 0))))
        elif lp is not None and lp is not False:   # completions: a count
            kw.setdefault("logprobs", max(0, min(MAX_TOP_LOGPROBS, int(lp))))
        return cls(temperature=float(t) if t is not None else float(default_temperature),
                   top_p=float(body["top_p"]) if body.get("top_p") is not None else 1.0,
                   top_k=int(k) if k is not None and int(k) > 0 else 0,
                   seed=int(seed) if seed is not None else None,
                   frequency_penalty=float(body.get("frequency_penalty") or 0.0),
                   presence_penalty=float(body.get("presence_penalty") or 0.0), **kw)

    @property
    def samples(self) -> bool:
        return self.temperature > 0.0

    @property
    def penalized(self) -> bool:
        return self.frequency_penalty != 0.0 or self.presence_penalty != 0.0


@dataclass
class MMItem:
    """Encoder output for one image/video/audio: ``embeds`` rows replace the placeholder run that starts
    at prompt index ``offset``."""

    embeds: torch.Tensor
    offset: int
    grid_thw: tuple[int, int, int] | None = None
    second_per_grid: float | None = None   # videos: seconds between two temporal grid steps (Qwen2.5-VL scales time by it)


@dataclass
class PrefilledKV:
    """Where the KV pages of an already-prefilled prompt are: ``src_cache`` is the producer's cache
    ``[layers, pages, 2, heads, 128, d]`` (mapped into this process) with the page numbers ``src_pages``; or ``raw``
    holds the pages themselves ``[layers, len(src_pages), 2, heads, 128, d]``."""

    first_token: int
    next_pos: int
    src_pages: list[int]
    src_cache: torch.Tensor | None = None
    raw: torch.Tensor | None = None


@dataclass
class HeldKV:
    pages: list[int]
    num_tokens: int
    next_pos: int
    first_token: int
    held_at: float = field(default_factory=time.monotonic)


class SeqStatus(enum.Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


@dataclass
class Sequence:
    seq_id: str
    prompt_ids: np.ndarray
    params: SamplingParams = field(default_factory=SamplingParams)
    mm_items: list[MMItem] = field(default_factory=list)
    return_hidden: bool = False
    capture_layers: tuple[int, ...] = ()    # return these points of the residual stream instead (0 = embeddings, i = after layer i-1)
    hold_kv: bool = False                   # keep the pages after finishing (prefill half of a disaggregated pair)
    prefilled: PrefilledKV | None = None    # the prompt's KV comes from another executor (decode half)
    kv_source: str | None = None            # "mapped" (peer copy kernel) or "network" once prefilled was consumed
    positions: np.ndarray | None = None     # [3, T]
    next_pos: int = 0
    status: SeqStatus = SeqStatus.WAITING
    num_computed: int = 0                   # prompt tokens already in the KV cache
    output_ids: list[int] = field(default_factory=list)
    hidden_chunks: list[torch.Tensor] = field(default_factory=list)
    arrival: float = field(default_factory=time.monotonic)
    first_token_time: float | None = None
    finish_reason: str | None = None

    @property
    def prompt_len(self) -> int:
        return int(self.prompt_ids.shape[0])


@dataclass
class EngineConfig:
    num_pages: int = 2048
    max_batched_tokens: int = 18944   # 148 SMs x 128-row tiles: every prefill GEMM gets whole tile waves
    max_num_seqs: int = 256
    decode_burst: int = 8
    use_cuda_graph: bool = True
    graph_batch_sizes: tuple[int, ...] = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    max_model_len: int = 32768


@dataclass
class StepOutput:
    seq_id: str
    new_token_ids: list[int]
    finished: bool
    finish_reason: str | None = None
    hidden: torch.Tensor | None = None
    # per new token, for requests that asked: (log probability of the token, [(token id, log probability), ...] most likely)
    logprobs: list[tuple[float, list[tuple[int, float]]]] | None = None


def _logprob_entry(lp: list[np.ndarray], step: int, row: int, k: int) -> tuple[float, list[tuple[int, float]]]:
    chosen, top_v, top_i = lp
    return float(chosen[step, row]), [(int(top_i[step, row, j]), float(top_v[step, row, j])) for j in range(k)]


class _DecodeState:
    """Static device buffers (and the captured graph) for one decode batch-size bucket."""

    def __init__(self, B: int, max_blocks: int, burst: int, device: torch.device):
        i32 = dict(dtype=torch.int32, device=device)
        self.B = B
        self.input_ids = torch.zeros(B, **i32)
        self.positions = torch.zeros(3, B, **i32)
        self.slot = torch.zeros(B, **i32)
        self.kv_len = torch.ones(B, **i32)
        self.block_table = torch.zeros(B, max_blocks, **i32)
        self.active = torch.zeros(B, **i32)
        self.cu_q = torch.arange(B + 1, **i32)
        self.logits_idx = torch.arange(B, **i32)
        self.out_log = torch.zeros(max(burst, 1), B, **i32)
        self.step_counter = torch.zeros(1, **i32)
        # sampling parameters of every row (used by the buckets whose graph ends in the sampling kernel)
        self.temperature = torch.zeros(B, dtype=torch.float32, device=device)
        self.top_p = torch.ones(B, dtype=torch.float32, device=device)
        self.top_k = torch.zeros(B, **i32)
        self.seed = torch.zeros(B, dtype=torch.int64, device=device)
        self.draws = torch.zeros(B, **i32)
        self.sampling = False
        # repetition control (buckets whose graph applies penalties): how often each row generated each token
        self.frequency = torch.zeros(B, dtype=torch.float32, device=device)
        self.presence = torch.zeros(B, dtype=torch.float32, device=device)
        self.counts: torch.Tensor | None = None
        # log probabilities (buckets whose graph reports them): per step of a burst, chosen token and the most likely ones
        self.lp_chosen: torch.Tensor | None = None
        self.lp_top_v: torch.Tensor | None = None
        self.lp_top_i: torch.Tensor | None = None
        self.graph: torch.cuda.CUDAGraph | None = None
        self.launches_per_replay = 0
        self.paths_per_replay: dict[str, int] = {}

    def sampler(self):
        return (self.temperature, self.top_p, self.top_k, self.seed, self.draws) if self.sampling else None

    def penalties(self):
        return (self.counts, self.frequency, self.presence, self.active) if self.counts is not None else None

    def enable_logprobs(self, burst: int, device: torch.device) -> None:
        self.lp_chosen = torch.zeros(max(burst, 1), self.B, dtype=torch.float32, device=device)
        self.lp_top_v = torch.zeros(max(burst, 1), self.B, MAX_TOP_LOGPROBS, dtype=torch.float32, device=device)
        self.lp_top_i = torch.zeros(max(burst, 1), self.B, MAX_TOP_LOGPROBS, dtype=torch.int32, device=device)

    def logprobs(self):
        return (self.lp_chosen, self.lp_top_v, self.lp_top_i, self.step_counter) if self.lp_chosen is not None else None

    def meta(self) -> BatchMeta:
        return BatchMeta(self.input_ids, self.positions, self.slot, self.cu_q, self.kv_len, self.block_table,
                         self.logits_idx, 1, True)


class LLMEngine:
    """Synchronous engine core.  ``add_request`` + ``step`` drive it; ``generate`` is the batch helper."""

    def __init__(self, model: QwenLLM, cfg: EngineConfig | None = None):
        self.model = model
        self.mcfg: LLMConfig = model.cfg
        self.cfg = cfg or EngineConfig()
        self.device = model.device
        self.on_gpu = self.device.type == "cuda"
        model.prefill_rows_hint = max(getattr(model, "prefill_rows_hint", 0), self.cfg.max_batched_tokens)
        self.blocks = BlockManager(self.cfg.num_pages)
        self.kv_caches = model.alloc_kv_cache(self.cfg.num_pages)
        self.kv_backing: torch.Tensor = model.kv_backing  # [layers, pages, 2, heads, 128, d]; kv_caches are its views
        self.max_blocks = -(-self.cfg.max_model_len // PAGE_SIZE)
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self._decode_states: dict[int, _DecodeState] = {}
        self._copy_stream = torch.cuda.Stream(device=self.device) if self.on_gpu else None
        self.held: dict[str, HeldKV] = {}
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "steps": 0, "kv_pages_pulled": 0, "prefill_steps": 0,
                      "decode_bursts": 0, "prefill_ms": 0.0, "decode_ms": 0.0, "decode_host_ms": 0.0}

    # ---------------------------------------------------------------------------------------------
    # requests
    # ---------------------------------------------------------------------------------------------
    def add_request(self, seq: Sequence) -> None:
        if seq.params.samples and seq.params.seed is None:
            seq.params.seed = random.getrandbits(62)
        # a sequence is admitted only when its whole lifetime fits in free pages: one that needs more pages than the
        # pool has would wait at the head of the queue for ever and block everything behind it
        need = -(-(seq.prompt_len + seq.params.max_tokens + 1) // PAGE_SIZE)
        if need > self.blocks.capacity:
            raise ValueError(f"request needs {need} KV pages (prompt {seq.prompt_len} + {seq.params.max_tokens} new tokens) "
                             f"but the cache holds {self.blocks.capacity}")
        if seq.prefilled is not None:
            if seq.prompt_len + seq.params.max_tokens > self.cfg.max_model_len:
                raise ValueError("request exceeds max_model_len")
            if len(seq.prefilled.src_pages) < -(-seq.prompt_len // PAGE_SIZE):
                raise ValueError("the transferred pages do not cover the prompt")
            seq.next_pos = seq.prefilled.next_pos
            self.waiting.append(seq)
            return
        if seq.positions is None:
            grids = [it.grid_thw for it in seq.mm_items if it.grid_thw is not None]
            if grids:
                # videos of Qwen2.5-VL advance the temporal index by seconds_per_grid * tokens_per_second per grid
                # step (1.0 s and 2 tokens/s unless the processor says otherwise); images are unaffected
                spg = [it.second_per_grid for it in seq.mm_items if it.grid_thw is not None]
                timed = self.mcfg.tokens_per_second is not None
                seq.positions, seq.next_pos = mrope_positions(
                    seq.prompt_ids, grids, self.mcfg.image_token_id, self.mcfg.video_token_id,
                    self.mcfg.spatial_merge_size,
                    second_per_grid=[1.0 if v is None else float(v) for v in spg] if timed else None,
                    tokens_per_second=float(self.mcfg.tokens_per_second or 2.0))
            else:
                T = seq.prompt_len
                seq.positions = np.broadcast_to(np.arange(T, dtype=np.int32)[None], (3, T)).copy()
                seq.next_pos = T
        if seq.prompt_len + seq.params.max_tokens > self.cfg.max_model_len:
            raise ValueError("request exceeds max_model_len")
        self.waiting.append(seq)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def abort(self, seq_id: str) -> None:
        for q in (self.waiting, self.running):
            for s in list(q):
                if s.seq_id == seq_id:
                    q.remove(s)
                    self.blocks.free(seq_id)

    # ---------------------------------------------------------------------------------------------
    # one engine step
    # ---------------------------------------------------------------------------------------------
    def step(self) -> list[StepOutput]:
        self.stats["steps"] += 1
        outs = self._admit_prefilled()
        if outs:
            return outs
        batch = self._schedule_prefill()
        if batch:
            t0 = time.perf_counter()
            outs = self._run_prefill(batch)
            self.stats["prefill_steps"] += 1
            self.stats["prefill_ms"] += (time.perf_counter() - t0) * 1e3
            return outs
        if self.running:
            t0 = time.perf_counter()
            outs = self._run_decode_burst()
            self.stats["decode_bursts"] += 1
            self.stats["decode_ms"] += (time.perf_counter() - t0) * 1e3
            return outs
        return []

    def _admit_prefilled(self) -> list[StepOutput]:
        """Sequences whose prompt was computed elsewhere: allocate pages, pull the prompt's KV, start decoding."""
        outs: list[StepOutput] = []
        while self.waiting and self.waiting[0].prefilled is not None and len(self.running) < self.cfg.max_num_seqs:
            s = self.waiting[0]
            total = s.prompt_len + s.params.max_tokens + 1
            if not self.blocks.can_allocate(total, s.seq_id):
                break
            self.waiting.popleft()
            pf = s.prefilled
            s.kv_source = "network" if pf.raw is not None else "mapped"
            n = -(-s.prompt_len // PAGE_SIZE)
            pages = self.blocks.ensure(s.seq_id, total)[:n]
            dst = self.kv_backing
            try:
                if pf.raw is not None:
                    dst[:, torch.as_tensor(pages, device=self.device)] = pf.raw[:, :n].to(self.device, dst.dtype)
                else:
                    i32 = lambda a: self._to_dev(np.asarray(a, dtype=np.int32))  # noqa: E731
                    ops.kv_copy_pages(dst, pf.src_cache, i32(pf.src_pages[:n]), i32(pages))
            except Exception as e:  # noqa: BLE001  (a bad transfer fails this request, not the engine)
                self.blocks.free(s.seq_id)
                s.prefilled = None
                s.status = SeqStatus.FINISHED
                outs.append(StepOutput(s.seq_id, [], True, f"error: KV transfer failed: {e}"))
                continue
            self.stats["kv_pages_pulled"] += n
            s.prefilled = None  # drops the reference to the producer's mapping / the fetched bytes
            s.num_computed = s.prompt_len
            s.status = SeqStatus.RUNNING
            s.first_token_time = time.monotonic()
            s.output_ids.append(int(pf.first_token))
            self.running.append(s)
            outs.append(self._emit(s, [int(pf.first_token)]))
        if outs:
            if self.on_gpu:
                torch.cuda.current_stream(self.device).synchronize()  # the producer may free its pages after this
            self._reap()
        return outs

    # -- producer side of a transfer ---------------------------------------------------------------------------
    def kv_transfer_params(self, seq_id: str) -> dict:
        h = self.held[seq_id]
        return {"request_id": seq_id, "num_tokens": h.num_tokens, "pages": h.pages[: -(-h.num_tokens // PAGE_SIZE)],
                "next_pos": h.next_pos, "first_token": h.first_token}

    def release_held(self, seq_id: str) -> bool:
        h = self.held.pop(seq_id, None)
        if h is None:
            return False
        self.blocks.release(h.pages)
        return True

    def expire_held(self, max_age_s: float) -> list[str]:
        """Free the pages of transfers nobody fetched (a decode executor that died, a cancelled request)."""
        now = time.monotonic()
        old = [sid for sid, h in self.held.items() if now - h.held_at > max_age_s]
        for sid in old:
            self.release_held(sid)
        return old

    def read_pages(self, pages: list[int]) -> torch.Tensor:
        """The pages themselves, on the host: ``[layers, len(pages), 2, heads, 128, d]`` (network fallback)."""
        idx = torch.as_tensor(pages, device=self.device, dtype=torch.long)
        return self.kv_backing[:, idx].cpu()

    def kv_geometry(self) -> dict:
        kv = self.kv_backing
        return {"shape": list(kv.shape), "dtype": str(kv.dtype).replace("torch.", "")}

    def _schedule_prefill(self) -> list[tuple[Sequence, int]]:
        """Pick prompt chunks for one prefill step: unfinished chunked prefills first, then new arrivals
        while the token budget, the sequence limit and the page pool allow.  A sequence is admitted only
        if its whole lifetime (prompt + max_tokens) fits in free pages, so decode never runs out."""
        budget = self.cfg.max_batched_tokens
        batch: list[tuple[Sequence, int]] = []
        for s in self.running:
            if s.num_computed < s.prompt_len and budget > 0:
                n = min(s.prompt_len - s.num_computed, budget)
                batch.append((s, n))
                budget -= n
        while self.waiting and budget > 0 and len(self.running) + len(batch) < self.cfg.max_num_seqs:
            s = self.waiting[0]
            if s.prefilled is not None:
                break  # first come, first served: it is admitted by _admit_prefilled once pages are free
            total = s.prompt_len + s.params.max_tokens + 1
            if not self.blocks.can_allocate(total, s.seq_id):
                break
            self.waiting.popleft()
            self.blocks.ensure(s.seq_id, total)
            n = min(s.prompt_len, budget)
            batch.append((s, n))
            budget -= n
        return batch

    def _run_prefill(self, batch: list[tuple[Sequence, int]]) -> list[StepOutput]:
        dev = self.device
        ids, pos, slots, cu, kvl, last = [], [], [], [0], [], []
        mm_rows, mm_idx = [], []
        bt = np.zeros((len(batch), self.max_blocks), dtype=np.int32)
        tok = 0
        for b, (s, n) in enumerate(batch):
            lo, hi = s.num_computed, s.num_computed + n
            pages = self.blocks.ensure(s.seq_id, hi + 1)
            bt[b, : len(pages)] = pages
            ids.append(s.prompt_ids[lo:hi])
            pos.append(s.positions[:, lo:hi])
            ar = np.arange(lo, hi)
            slots.append(np.asarray(pages, dtype=np.int64)[ar // PAGE_SIZE] * PAGE_SIZE + ar % PAGE_SIZE)
            for it in s.mm_items:
                a, e = max(it.offset, lo), min(it.offset + it.embeds.shape[0], hi)
                if a < e:
                    mm_rows.append(it.embeds[a - it.offset: e - it.offset])
                    mm_idx.append(np.arange(a, e) - lo + tok)
            tok += n
            cu.append(tok)
            kvl.append(hi)
            last.append(tok - 1)
        max_blk = max(1, max(-(-k // PAGE_SIZE) for k in kvl) + 1)
        f = lambda a, dt=np.int32: self._to_dev(np.ascontiguousarray(np.asarray(a).astype(dt)))  # noqa: E731
        m = BatchMeta(
            input_ids=f(np.concatenate(ids)), positions=f(np.concatenate(pos, axis=1)),
            slot_mapping=f(np.concatenate(slots)), cu_q=f(cu), kv_len=f(kvl), block_table=f(bt[:, :max_blk]),
            logits_idx=f(last), max_q_len=max(n for _, n in batch), is_decode=False,
        )
        if mm_rows:
            m.mm_embeds = mm_rows  # placed row by row by the scatter kernel, from wherever they live
            m.mm_index = [f(i) for i in mm_idx]
        want_hidden = any(s.return_hidden for s, _ in batch)
        cap_layers = sorted({layer for s, _ in batch for layer in s.capture_layers})
        capture = dict.fromkeys(cap_layers) if cap_layers else None
        sampler = None
        if any(s.params.samples for s, _ in batch):
            # the first token of a sampled request is draw 0 of its stream (rows of greedy requests keep temperature 0)
            sampler = (f([s.params.temperature for s, _ in batch], np.float32), f([s.params.top_p for s, _ in batch], np.float32),
                       f([s.params.top_k for s, _ in batch]), f([s.params.seed or 0 for s, _ in batch], np.int64),
                       f([len(s.output_ids) for s, _ in batch]))
        lp_dev = None
        if any(s.params.logprobs >= 0 for s, _ in batch):
            nb = len(batch)
            lp_dev = (torch.zeros(1, nb, dtype=torch.float32, device=dev),
                      torch.zeros(1, nb, MAX_TOP_LOGPROBS, dtype=torch.float32, device=dev),
                      torch.zeros(1, nb, MAX_TOP_LOGPROBS, dtype=torch.int32, device=dev),
                      torch.zeros(1, dtype=torch.int32, device=dev))
        with torch.inference_mode():
            next_tok, hidden = self.model(m, self.kv_caches, return_hidden=want_hidden, capture=capture, sampler=sampler,
                                          logprobs=lp_dev)
        toks = next_tok.tolist()
        lp = [t.cpu().numpy() for t in lp_dev[:3]] if lp_dev is not None else None
        self.stats["prefill_tokens"] += tok
        outs: list[StepOutput] = []
        now = time.monotonic()
        for b, (s, n) in enumerate(batch):
            s.num_computed += n
            if s not in self.running:
                self.running.append(s)
            if s.capture_layers:
                s.hidden_chunks.append(torch.cat([capture[layer][cu[b]: cu[b + 1]] for layer in s.capture_layers], dim=1))
            elif s.return_hidden and hidden is not None:
                s.hidden_chunks.append(hidden[cu[b]: cu[b + 1]])
            if s.num_computed < s.prompt_len:
                continue
            s.status = SeqStatus.RUNNING
            s.first_token_time = now
            s.output_ids.append(int(toks[b]))
            out = self._emit(s, [int(toks[b])])
            if lp is not None and s.params.logprobs >= 0:
                out.logprobs = [_logprob_entry(lp, 0, b, s.params.logprobs)]
            outs.append(out)
        self._reap()
        return outs

    # ---------------------------------------------------------------------------------------------
    # decode
    # ---------------------------------------------------------------------------------------------
    def _bucket(self, n: int) -> int:
        for b in self.cfg.graph_batch_sizes:
            if b >= n:
                return b
        return n

    def _run_decode_burst(self) -> list[StepOutput]:
        seqs = [s for s in self.running if s.status is SeqStatus.RUNNING]
        if not seqs:
            return []
        t_host = time.perf_counter()
        burst = max(1, min(self.cfg.decode_burst, min(s.params.max_tokens - len(s.output_ids) for s in seqs)))
        n = len(seqs)
        B = self._bucket(n) if (self.on_gpu and self.cfg.use_cuda_graph) else n
        penalized = any(s.params.penalized for s in seqs)
        sampling = penalized or any(s.params.samples for s in seqs)
        # a bucket's graph ends in the arg-max, in the sampling kernel, or in penalties + the sampling kernel
        key = (B, "penalty") if penalized else ((B, "sample") if sampling else B)
        want_lp = any(s.params.logprobs >= 0 for s in seqs)
        if want_lp:
            key = (key if isinstance(key, tuple) else (key, "greedy")) + ("logprobs",)
        st = self._decode_states.get(key)
        if st is None:
            st = self._decode_states[key] = _DecodeState(B, self.max_blocks, self.cfg.decode_burst, self.device)
            st.sampling = sampling
            if want_lp:
                st.enable_logprobs(self.cfg.decode_burst, self.device)
            if penalized:
                st.counts = torch.zeros(B, self.mcfg.vocab_size, dtype=torch.int32, device=self.device)
        # host-side batch state
        ids = np.zeros(B, np.int32); pos = np.zeros((3, B), np.int32); slot = np.zeros(B, np.int32)
        kvl = np.ones(B, np.int32); act = np.zeros(B, np.int32)
        bt = np.zeros((B, self.max_blocks), np.int32)
        for b, s in enumerate(seqs):
            cur = s.prompt_len + len(s.output_ids) - 1  # index of the token being fed = keys already cached
            pages = self.blocks.ensure(s.seq_id, cur + burst + 1)
            bt[b, : len(pages)] = pages
            ids[b] = s.output_ids[-1]
            pos[:, b] = s.next_pos + len(s.output_ids) - 1
            slot[b] = pages[cur // PAGE_SIZE] * PAGE_SIZE + cur % PAGE_SIZE
            kvl[b] = cur + 1
            act[b] = 1
        for t, a in ((st.input_ids, ids), (st.positions, pos), (st.slot, slot), (st.kv_len, kvl), (st.active, act),
                     (st.block_table, bt)):
            t.copy_(self._pin(a), non_blocking=True)
        if sampling:
            temp = np.zeros(B, np.float32); tp = np.ones(B, np.float32); tk = np.zeros(B, np.int32)
            sd = np.zeros(B, np.int64); dr = np.zeros(B, np.int32)
            for b, s in enumerate(seqs):
                temp[b], tp[b], tk[b] = s.params.temperature, s.params.top_p, s.params.top_k
                sd[b], dr[b] = s.params.seed or 0, len(s.output_ids)
            for t, a in ((st.temperature, temp), (st.top_p, tp), (st.top_k, tk), (st.seed, sd), (st.draws, dr)):
                t.copy_(self._pin(a), non_blocking=True)
        if penalized:
            # rows are re-assigned every burst: rebuild each row's counts from what its sequence generated so far
            fr = np.zeros(B, np.float32); pr = np.zeros(B, np.float32)
            rows_idx, tok_idx = [], []
            for b, s in enumerate(seqs):
                fr[b], pr[b] = s.params.frequency_penalty, s.params.presence_penalty
                if s.params.penalized:
                    rows_idx.extend([b] * len(s.output_ids))
                    tok_idx.extend(s.output_ids)
            st.frequency.copy_(self._pin(fr), non_blocking=True)
            st.presence.copy_(self._pin(pr), non_blocking=True)
            st.counts.zero_()
            if rows_idx:
                r = self._to_dev(np.asarray(rows_idx, dtype=np.int64))
                t = self._to_dev(np.asarray(tok_idx, dtype=np.int64))
                st.counts.index_put_((r, t), torch.ones(len(rows_idx), dtype=torch.int32, device=self.device), accumulate=True)
        st.step_counter.zero_()
        with torch.inference_mode():
            for _ in range(burst):
                self._decode_once(st)
        self.stats["decode_host_ms"] += (time.perf_counter() - t_host) * 1e3   # batch state + launches, before the wait
        log = st.out_log[:burst].cpu().numpy()  # one sync per burst
        lp = [t[:burst].cpu().numpy() for t in (st.lp_chosen, st.lp_top_v, st.lp_top_i)] if want_lp else None
        self.stats["decode_tokens"] += burst * n
        outs = []
        for b, s in enumerate(seqs):
            new = []
            for t in log[:, b].tolist():
                s.output_ids.append(int(t))
                new.append(int(t))
                if self._should_stop(s):
                    break
            out = self._emit(s, new)
            if lp is not None and s.params.logprobs >= 0:
                out.logprobs = [_logprob_entry(lp, i, b, s.params.logprobs) for i in range(len(new))]
            outs.append(out)
        self._reap()
        return outs

    def capture_decode_graphs(self) -> int:
        """Capture the decode graph of every batch-size bucket up to ``max_num_seqs`` now, with all rows inactive
        (they read the scratch page), so that no request pays for a capture later.  Every rank of a tensor-parallel
        group calls this at the same point of its start-up.  Returns the number of graphs captured."""
        if not (self.on_gpu and self.cfg.use_cuda_graph):
            return 0
        n = 0
        for B in self.cfg.graph_batch_sizes:
            if B > self._bucket(self.cfg.max_num_seqs) or B in self._decode_states:
                continue
            st = self._decode_states[B] = _DecodeState(B, self.max_blocks, self.cfg.decode_burst, self.device)
            with torch.inference_mode():
                self._decode_once(st)
            st.step_counter.zero_()
            n += 1
        torch.cuda.synchronize(self.device)
        return n

    def _decode_once(self, st: _DecodeState) -> None:
        def body():
            tok, _ = self.model(st.meta(), self.kv_caches, sampler=st.sampler(), penalties=st.penalties(),
                                logprobs=st.logprobs())
            ops.decode_advance_(tok, st.input_ids, st.positions, st.kv_len, st.slot, st.block_table, st.active,
                                st.out_log, st.step_counter)

        if not (self.on_gpu and self.cfg.use_cuda_graph) or st.lp_chosen is not None:
            # buckets that report log probabilities run eagerly: their soft-max and top-k are library calls whose
            # behaviour under stream capture is not relied upon, and such requests are rare
            body()
            return
        if st.graph is None:
            # warm-up run outside the graph (sets kernel attributes, fills allocator pools), then capture;
            # the state is restored afterwards so the warm-up leaves no trace
            keep = [st.input_ids, st.positions, st.slot, st.kv_len, st.step_counter, st.draws]
            if st.counts is not None:
                keep.append(st.counts)
            snap = [t.clone() for t in keep]
            body()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            before, paths_before = ops.kernel_launches(), ops.path_counts()
            with torch.cuda.graph(g):
                body()
            st.launches_per_replay = ops.kernel_launches() - before
            st.paths_per_replay = {k: v - paths_before.get(k, 0) for k, v in ops.path_counts().items()
                                   if v != paths_before.get(k, 0)}
            st.graph = g
            for t, v in zip(keep, snap):
                t.copy_(v)
        st.graph.replay()
        ops._count(st.launches_per_replay)
        for k, v in st.paths_per_replay.items():
            ops.count_path(k, v)

    # ---------------------------------------------------------------------------------------------
    # helpers
    # ---------------------------------------------------------------------------------------------
    def _pin(self, a: np.ndarray) -> torch.Tensor:
        t = torch.from_numpy(a)
        return t.pin_memory() if self.on_gpu else t

    def _to_dev(self, a: np.ndarray) -> torch.Tensor:
        return self._pin(a).to(self.device, non_blocking=True)

    def _should_stop(self, s: Sequence) -> bool:
        if len(s.output_ids) >= s.params.max_tokens:
            s.finish_reason = "length"
            return True
        last = s.output_ids[-1]
        if not s.params.ignore_eos and (last == self.mcfg.eos_token_id or last in s.params.stop_token_ids):
            s.finish_reason = "stop"
            return True
        return False

    def _emit(self, s: Sequence, new: list[int]) -> StepOutput:
        done = s.finish_reason is not None or self._should_stop(s)
        hidden = None
        if done:
            s.status = SeqStatus.FINISHED
            if (s.return_hidden or s.capture_layers) and s.hidden_chunks:
                hidden = torch.cat(s.hidden_chunks, dim=0)
        return StepOutput(s.seq_id, new, done, s.finish_reason, hidden)

    def _reap(self) -> None:
        for s in [s for s in self.running if s.status is SeqStatus.FINISHED]:
            self.running.remove(s)
            if s.hold_kv and s.output_ids and (s.finish_reason or "").startswith(("length", "stop")):
                self.held[s.seq_id] = HeldKV(self.blocks.detach(s.seq_id), s.prompt_len, s.next_pos, s.output_ids[0])
            else:
                self.blocks.free(s.seq_id)

    # ---------------------------------------------------------------------------------------------
    # batch helper
    # ---------------------------------------------------------------------------------------------
    def generate(self, seqs: Iterable[Sequence]) -> dict[str, list[int]]:
        """Run the given requests to completion; returns ``seq_id -> generated token ids``."""
        out: dict[str, list[int]] = {}
        for s in seqs:
            out[s.seq_id] = []
            self.add_request(s)
        while self.has_work():
            for o in self.step():
                out[o.seq_id].extend(o.new_token_ids)
        return out
