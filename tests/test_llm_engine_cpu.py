"""LLM engine on CPU: continuous batching, chunked prefill, decode bursts and encoder-embedding
injection must reproduce a plain full-sequence forward (same model, fp32)."""

import numpy as np
import pytest
import torch

from cornserve.task_executors.llm.block_manager import BlockManager, OutOfPages
from cornserve.task_executors.llm.engine import EngineConfig, LLMEngine, MMItem, SamplingParams, Sequence
from cornserve.task_executors.llm.mrope import mrope_positions
from cornserve.models.qwen_llm import BatchMeta, LLMConfig, QwenLLM


def _model():
    torch.manual_seed(0)
    cfg = LLMConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                    intermediate_size=256, vocab_size=512, mrope_section=[4, 6, 6], rope_theta=10000.0,
                    image_token_id=500, eos_token_id=511)
    m = QwenLLM(cfg, device="cpu").float()
    for p in m.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.1)
    return m


def _greedy_reference(model, ids, positions, n_new, mm=None):
    """Recompute the whole sequence every step (no cache reuse), greedy."""
    ids = list(ids)
    pos = positions.copy()
    out = []
    for _ in range(n_new):
        T = len(ids)
        caches = model.alloc_kv_cache(2 + T // 128 + 1)
        nblk = T // 128 + 1
        bt = torch.arange(1, 1 + nblk, dtype=torch.int32)[None]
        meta = BatchMeta(torch.tensor(ids, dtype=torch.int32), torch.from_numpy(pos).int(),
                         (128 + torch.arange(T)).int(), torch.tensor([0, T], dtype=torch.int32),
                         torch.tensor([T], dtype=torch.int32), bt, torch.tensor([T - 1], dtype=torch.int32), T)
        if mm is not None:
            meta.mm_embeds, meta.mm_index = mm
        tok, _ = model(meta, caches)
        t = int(tok[0])
        out.append(t)
        ids.append(t)
        pos = np.concatenate([pos, np.full((3, 1), pos.max() + 1 if len(out) == 1 else pos[0, -1] + 1, np.int32)], 1)
    return out


def test_engine_matches_full_recompute_with_chunked_prefill_and_bursts():
    model = _model()
    prompts = [np.arange(3, 40, dtype=np.int32), np.arange(50, 57, dtype=np.int32), np.arange(100, 250, dtype=np.int32)]
    eng = LLMEngine(model, EngineConfig(num_pages=32, max_batched_tokens=64, decode_burst=3, max_model_len=512))
    seqs = [Sequence(f"s{i}", p, SamplingParams(max_tokens=7, ignore_eos=True)) for i, p in enumerate(prompts)]
    got = eng.generate(seqs)
    for i, p in enumerate(prompts):
        pos = np.broadcast_to(np.arange(len(p), dtype=np.int32)[None], (3, len(p))).copy()
        assert got[f"s{i}"] == _greedy_reference(model, p, pos, 7), f"sequence {i}"
    assert eng.blocks.num_free == 31 and not eng.has_work()


def test_engine_injects_encoder_embeddings_with_mrope():
    model = _model()
    grid = (1, 4, 6)  # -> 6 merged tokens
    ids = np.array([1, 2, 3] + [500] * 6 + [7, 8], dtype=np.int32)
    emb = torch.randn(6, 128)
    pos, nxt = mrope_positions(ids, [grid], 500)
    assert pos[:, :3].tolist() == [[0, 1, 2]] * 3 and pos[1, 3:9].tolist() == [3, 3, 3, 4, 4, 4]
    assert pos[2, 3:9].tolist() == [3, 4, 5, 3, 4, 5] and pos[0, 9] == 6 and nxt == 8
    eng = LLMEngine(model, EngineConfig(num_pages=8, decode_burst=2, max_model_len=256))
    got = eng.generate([Sequence("a", ids, SamplingParams(max_tokens=4, ignore_eos=True),
                                 mm_items=[MMItem(emb, 3, grid)], return_hidden=True)])
    want = _greedy_reference(model, ids, pos, 4, mm=(emb, torch.arange(3, 9, dtype=torch.int32)))
    assert got["a"] == want


def test_eos_stops_generation():
    model = _model()
    eng = LLMEngine(model, EngineConfig(num_pages=8, decode_burst=4, max_model_len=256))
    p = np.arange(10, 30, dtype=np.int32)
    free_run = eng.generate([Sequence("x", p, SamplingParams(max_tokens=12, ignore_eos=True))])["x"]
    stop_tok = free_run[5]
    first = free_run.index(stop_tok)
    out = eng.generate([Sequence("y", p, SamplingParams(max_tokens=12, stop_token_ids=(stop_tok,)))])["y"]
    assert out == free_run[: first + 1]


def test_sampling_streams_are_reproducible_and_leave_greedy_requests_alone():
    """temperature / top-k / top-p with a seed: the same request gives the same tokens whatever shares its batch, a
    different seed gives other tokens, top_k = 1 equals greedy, and sampled tokens stay inside the allowed set."""
    model = _model()
    prompts = [np.arange(3, 40, dtype=np.int32), np.arange(50, 57, dtype=np.int32), np.arange(100, 130, dtype=np.int32)]

    def run(params, chosen=(0, 1, 2)):
        eng = LLMEngine(model, EngineConfig(num_pages=32, max_batched_tokens=64, decode_burst=3, max_model_len=512))
        return eng.generate([Sequence(f"s{i}", prompts[i], params[i]) for i in chosen])

    greedy = run([SamplingParams(9, True)] * 3)
    sp = [SamplingParams(9, True), SamplingParams(9, True, temperature=1.3, top_p=0.9, seed=11),
          SamplingParams(9, True, temperature=0.8, top_k=1, seed=5)]
    a = run(sp)
    assert a["s0"] == greedy["s0"]                       # a greedy request in a sampling batch
    assert a["s2"] == greedy["s2"]                       # top_k = 1 leaves only the arg-max
    assert a["s1"] != greedy["s1"]
    assert run(sp, chosen=(1,))["s1"] == a["s1"]         # alone or in company: same stream
    other = [sp[0], SamplingParams(9, True, temperature=1.3, top_p=0.9, seed=12), sp[2]]
    assert run(other)["s1"] != a["s1"]
    # without a seed the engine draws one per request
    free = SamplingParams(9, True, temperature=1.3)
    eng = LLMEngine(model, EngineConfig(num_pages=32, max_batched_tokens=64, decode_burst=3, max_model_len=512))
    eng.generate([Sequence("x", prompts[1], free)])
    assert free.seed is not None


def test_sampling_params_from_request_fields():
    p = SamplingParams.from_request({"temperature": 0.7, "top_p": 0.8, "top_k": 40, "seed": 3}, max_tokens=5)
    assert (p.temperature, p.top_p, p.top_k, p.seed, p.max_tokens, p.samples) == (0.7, 0.8, 40, 3, 5, True)
    q = SamplingParams.from_request({"top_k": -1, "temperature": 0}, max_tokens=2)
    assert (q.temperature, q.top_p, q.top_k, q.seed, q.samples) == (0.0, 1.0, 0, None, False)


def test_sampler_restatement_respects_cutoffs():
    from cornserve.ops import reference as ref

    torch.manual_seed(3)
    V, rows = 400, 600
    base = torch.randn(V) * 2.5
    logits = base[None].repeat(rows, 1)
    temp, top_p, top_k = 0.9, 0.8, 25
    keep, w = ref.sample_kept_mask(base, temp, top_p, top_k)
    assert 1 <= keep.sum() <= top_k
    probs = torch.softmax(base / temp, -1)
    order = probs.argsort(descending=True)
    topk_mass = probs[order[:top_k]].sum()
    n_keep = int(keep.sum())
    assert probs[order[:n_keep]].sum() >= top_p * topk_mass - 1e-4            # the kept prefix reaches the nucleus mass
    assert n_keep == 1 or probs[order[:n_keep - 1]].sum() < top_p * topk_mass + 1e-4   # and is the smallest that does
    draws = torch.zeros(rows, dtype=torch.int32)
    toks = ref.sample_rows(logits, torch.full((rows,), temp), torch.full((rows,), top_p),
                           torch.full((rows,), top_k, dtype=torch.int32), torch.arange(rows), draws)
    assert bool(torch.from_numpy(keep)[toks.long()].all()) and int(draws.min()) == 1
    want = (probs * torch.from_numpy(keep)) / (probs * torch.from_numpy(keep)).sum()
    freq = torch.bincount(toks.long(), minlength=V).float() / rows
    assert (freq - want).abs().max() < 0.06


def test_fp8_projections_track_the_full_precision_model():
    """Attention and MLP projections in block-scaled e4m3: hidden states stay close to the fp32 model, the bf16 weights
    are gone, generation still runs; an fp8 checkpoint (weights + ``weight_scale_inv``) is widened on the way in."""
    from cornserve import ops
    from cornserve.models.qwen_llm import dequantize_fp8_checkpoint

    model = _model()
    prompt = np.arange(3, 60, dtype=np.int32)

    def hidden(m):
        eng = LLMEngine(m, EngineConfig(num_pages=16, max_batched_tokens=64, decode_burst=3, max_model_len=256))
        eng.add_request(Sequence("a", prompt, SamplingParams(1, True), return_hidden=True))
        outs = []
        while eng.has_work():
            outs += eng.step()
        return outs[-1].hidden.float().flatten()

    want = hidden(model)
    model.quantize_fp8_()
    got = hidden(model)
    assert torch.nn.functional.cosine_similarity(want, got, dim=0).item() > 0.98
    lay = model.layers[0]
    assert lay.self_attn.qkv.weight is None and lay.mlp.down.fp8[0].dtype == torch.float8_e4m3fn
    eng = LLMEngine(model, EngineConfig(num_pages=16, max_batched_tokens=64, decode_burst=3, max_model_len=256))
    assert len(eng.generate([Sequence("g", prompt, SamplingParams(6, True))])["g"]) == 6

    w = torch.randn(200, 256)
    q, sc = ops.quantize_fp8_weight(w)
    out = dict(dequantize_fp8_checkpoint([("l.q_proj.weight_scale_inv", sc), ("l.q_proj.weight", q), ("l.norm.weight", torch.ones(3))]))
    assert sorted(out) == ["l.norm.weight", "l.q_proj.weight"] and out["l.q_proj.weight"].dtype == torch.bfloat16
    assert (out["l.q_proj.weight"].float() - w).abs().max().item() < 0.3
    with pytest.raises(ValueError):
        list(dequantize_fp8_checkpoint([("l.q_proj.weight", q)]))


def test_block_manager():
    bm = BlockManager(5)
    assert bm.ensure("a", 129) == [1, 2] and bm.num_free == 2
    assert bm.ensure("a", 200) == [1, 2]
    assert not bm.can_allocate(400, "b")
    try:
        bm.ensure("b", 400)
        raise AssertionError
    except OutOfPages:
        pass
    bm.free("a")
    assert bm.num_free == 4


def test_request_larger_than_the_page_pool_is_refused_not_queued():
    """A prompt that can never fit must fail at ``add_request``; queued, it would block every later request."""
    import numpy as np
    import pytest

    from cornserve.models.qwen_llm import LLMConfig, QwenLLM
    from cornserve.task_executors.llm.engine import EngineConfig, LLMEngine, SamplingParams, Sequence

    cfg = LLMConfig(hidden_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=32,
                    intermediate_size=64, vocab_size=128, mrope_section=None)
    eng = LLMEngine(QwenLLM(cfg).float().eval(), EngineConfig(num_pages=3, use_cuda_graph=False, max_model_len=4096))
    with pytest.raises(ValueError, match="KV pages"):
        eng.add_request(Sequence("big", np.arange(300, dtype=np.int32) % 100, SamplingParams(max_tokens=8, ignore_eos=True)))
    ok = Sequence("small", np.arange(20, dtype=np.int32), SamplingParams(max_tokens=4, ignore_eos=True))
    assert len(eng.generate([ok])["small"]) == 4


def _tiny_engine(**kw):
    import torch

    from cornserve.models.qwen_llm import LLMConfig, QwenLLM
    from cornserve.task_executors.llm.engine import EngineConfig, LLMEngine

    torch.manual_seed(3)
    cfg = LLMConfig(hidden_size=64, num_hidden_layers=2, num_attention_heads=2, num_key_value_heads=1, head_dim=32,
                    intermediate_size=64, vocab_size=96, mrope_section=None)
    return LLMEngine(QwenLLM(cfg).float().eval(), EngineConfig(num_pages=8, use_cuda_graph=False, max_model_len=1024, **kw))


def test_frequency_and_presence_penalties_change_greedy_decoding_as_specified():
    """With penalties the engine must produce exactly what a step-by-step restatement produces: greedy over
    ``logits - frequency * count - presence * (count > 0)`` with counts over the tokens generated so far."""
    import numpy as np
    import torch

    from cornserve.task_executors.llm.engine import SamplingParams, Sequence

    prompt = np.arange(5, 25, dtype=np.int32)
    eng = _tiny_engine(decode_burst=3)
    plain = eng.generate([Sequence("a", prompt, SamplingParams(max_tokens=12, ignore_eos=True))])["a"]
    pen = eng.generate([Sequence("b", prompt, SamplingParams(max_tokens=12, ignore_eos=True, frequency_penalty=1.5,
                                                               presence_penalty=4.0))])["b"]
    assert plain != pen, "random tiny models repeat themselves: penalties have to change the continuation"
    # restatement: feed the prefix again for every token, apply the penalties on the host
    ref_eng = _tiny_engine()
    out: list[int] = []
    for _ in range(12):
        ids = np.concatenate([prompt, np.asarray(out, dtype=np.int32)])
        seq = Sequence(f"r{len(out)}", ids, SamplingParams(max_tokens=1, ignore_eos=True))
        ref_eng.add_request(seq)
        batch = ref_eng._schedule_prefill()
        logits = _last_logits(ref_eng, batch)
        counts = torch.bincount(torch.as_tensor(out, dtype=torch.long), minlength=logits.numel()).float() if out else torch.zeros_like(logits)
        out.append(int((logits - 1.5 * counts - 4.0 * (counts > 0)).argmax()) if len(out) else int(logits.argmax()))
        ref_eng.blocks.free(seq.seq_id)   # scheduled by hand, so never in the running list: give the pages back
    assert pen == out
    # a batch that mixes penalised and plain requests keeps the plain ones unchanged
    both = eng.generate([Sequence("c", prompt, SamplingParams(max_tokens=12, ignore_eos=True)),
                         Sequence("d", prompt, SamplingParams(max_tokens=12, ignore_eos=True, frequency_penalty=1.5, presence_penalty=4.0))])
    assert both["c"] == plain and both["d"] == pen


def _last_logits(eng, batch):
    """Logits of the last prompt token of a one-sequence prefill batch, computed through the model's own layers."""
    import numpy as np
    import torch

    from cornserve import ops
    from cornserve.models.qwen_llm import PAGE_SIZE, BatchMeta

    (s, n), = batch
    pages = eng.blocks.ensure(s.seq_id, n + 1)
    ar = np.arange(n)
    t = lambda a, dt=np.int32: torch.from_numpy(np.ascontiguousarray(np.asarray(a).astype(dt)))  # noqa: E731
    bt = np.zeros((1, eng.max_blocks), np.int32)
    bt[0, : len(pages)] = pages
    m = BatchMeta(t(s.prompt_ids), t(s.positions), t(np.asarray(pages)[ar // PAGE_SIZE] * PAGE_SIZE + ar % PAGE_SIZE), t([0, n]), t([n]),
                  t(bt[:, : n // PAGE_SIZE + 2]), t([n - 1]), n, False)
    with torch.inference_mode():
        h = eng.model.forward_hidden(m, eng.kv_caches, None)
        return eng.model.compute_logits(ops.gather_rows(h, m.logits_idx))[0].float()


def test_sampling_params_follow_the_openai_defaults():
    from cornserve.task_executors.llm.engine import SamplingParams

    assert SamplingParams.from_request({}).temperature == 1.0            # OpenAI: temperature defaults to 1
    assert SamplingParams.from_request({}, 0.0).temperature == 0.0         # the model's generation config may say greedy
    p = SamplingParams.from_request({"temperature": 0, "frequency_penalty": 0.5, "presence_penalty": None})
    assert p.temperature == 0.0 and not p.samples and p.frequency_penalty == 0.5 and p.presence_penalty == 0.0 and p.penalized


def test_video_positions_scale_time_by_seconds_per_grid():
    """Qwen2.5-VL (Hugging Face ``get_rope_index``): the temporal index of a video's tokens is
    ``floor(frame_index * second_per_grid_t * tokens_per_second)``, height / width indices count merged cells, all three
    offset by the running position; text resumes at ``max + 1``.  Images keep a temporal index of zero."""
    import numpy as np

    IMG, VID = 900, 901
    # text a | video of 2 temporal steps x (2 x 4 patches -> 1 x 2 merged cells) | text b | image 4 x 4 -> 2 x 2 | text c
    ids = np.asarray([5, VID, VID, VID, VID, 6, IMG, IMG, IMG, IMG, 7], dtype=np.int32)
    got, nxt = mrope_positions(ids, [(2, 2, 4), (1, 4, 4)], IMG, VID, 2, second_per_grid=[1.5, 1.0], tokens_per_second=2.0)
    want = np.asarray([[0, 1, 1, 4, 4, 5, 6, 6, 6, 6, 8],      # time: frames at 0 and floor(1 * 1.5 * 2) = 3, offset 1
                       [0, 1, 1, 1, 1, 5, 6, 6, 7, 7, 8],      # height
                       [0, 1, 2, 1, 2, 5, 6, 7, 6, 7, 8]])     # width
    assert np.array_equal(got, want) and nxt == 9
    # without timing information a video is indexed per frame (Qwen2-VL)
    plain, _ = mrope_positions(ids, [(2, 2, 4), (1, 4, 4)], IMG, VID, 2)
    assert plain[0].tolist() == [0, 1, 1, 2, 2, 3, 4, 4, 4, 4, 6]


def test_engine_passes_video_timing_to_the_positions():
    import numpy as np
    import torch

    from cornserve.models.qwen_llm import LLMConfig, QwenLLM
    from cornserve.task_executors.llm.engine import EngineConfig, LLMEngine, MMItem, SamplingParams, Sequence

    cfg = LLMConfig(hidden_size=64, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1, head_dim=32, intermediate_size=64,
                    vocab_size=1024, mrope_section=[4, 6, 6], image_token_id=900, video_token_id=901, tokens_per_second=2.0)
    eng = LLMEngine(QwenLLM(cfg).float().eval(), EngineConfig(num_pages=4, use_cuda_graph=False, max_model_len=256))
    ids = np.asarray([5, 901, 901, 901, 901, 6], dtype=np.int32)
    seq = Sequence("v", ids, SamplingParams(max_tokens=1, ignore_eos=True),
                   mm_items=[MMItem(torch.zeros(4, 64), 1, (2, 2, 4), second_per_grid=1.5)])
    eng.add_request(seq)
    assert seq.positions[0].tolist() == [0, 1, 1, 4, 4, 5] and seq.next_pos == 6
