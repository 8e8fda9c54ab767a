"""GPU: the flagship models (vision tower, LLM engine, pipeline) against their CPU fp32 restatements."""

import copy

import numpy as np
import pytest
import torch

from cornserve import ops
from cornserve.task_executors.llm.engine import EngineConfig, LLMEngine, SamplingParams, Sequence
from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer
from cornserve.models.qwen_llm import LLMConfig, QwenLLM
from cornserve.pipelines import MLLMPipeline, MLLMRequest

pytestmark = pytest.mark.gpu


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().float().cpu(), b.flatten().float().cpu(), dim=0).item()


def _to_cpu_fp32(model_gpu, ctor):
    m = ctor()
    m.load_state_dict({k: v.float().cpu() for k, v in model_gpu.state_dict().items()})
    return m.float()


def test_vision_tower_gpu_vs_cpu():
    torch.manual_seed(0)
    cfg = Qwen25VisionConfig(depth=4, hidden_size=1280, num_heads=16, intermediate_size=3420, out_hidden_size=512,
                             fullatt_block_indexes=[1, 3])
    g = Qwen25VisionTransformer(cfg, device="cuda")
    c = _to_cpu_fp32(g, lambda: Qwen25VisionTransformer(cfg, device="cpu"))
    grids = [[1, 20, 36], [1, 8, 12]]
    pix = [torch.randn(a[1] * a[2], cfg.patch_dim) for a in grids]
    batch = lambda dev, dt: {"pixel_values": [p.to(dev, dt) for p in pix], "image_grid_thw": grids}  # noqa: E731
    with torch.inference_mode():
        yg = g("image", None, batch("cuda", torch.bfloat16))
        yc = c("image", None, batch("cpu", torch.float32))
    torch.cuda.synchronize()
    ops.check_error("vision")
    for a, b in zip(yg, yc):
        assert a.shape == b.shape and _cos(a, b) > 0.99


def _llm_cfg():
    return LLMConfig(hidden_size=512, num_hidden_layers=3, num_attention_heads=8, num_key_value_heads=2, head_dim=128,
                     intermediate_size=1024, vocab_size=2048, eos_token_id=2047)


def test_llm_engine_gpu_graph_matches_eager_and_cpu_hidden():
    torch.manual_seed(1)
    cfg = _llm_cfg()
    g = QwenLLM(cfg, device="cuda")
    for p in g.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.05)
    prompts = [np.arange(5, 300, dtype=np.int32), np.arange(900, 917, dtype=np.int32), np.arange(30, 160, dtype=np.int32)]
    mk = lambda: [Sequence(f"s{i}", p, SamplingParams(max_tokens=20, ignore_eos=True), return_hidden=True)  # noqa: E731
                  for i, p in enumerate(prompts)]
    res = {}
    for graph in (False, True):
        eng = LLMEngine(g, EngineConfig(num_pages=32, max_batched_tokens=256, decode_burst=5, use_cuda_graph=graph,
                                        max_model_len=1024))
        res[graph] = eng.generate(mk())
    torch.cuda.synchronize()
    ops.check_error("llm engine")
    assert res[True] == res[False]
    # prefill hidden states against the CPU fp32 model
    c = _to_cpu_fp32(g, lambda: QwenLLM(cfg, device="cpu"))
    hid = {}
    for name, model in (("g", g), ("c", c)):
        eng = LLMEngine(model, EngineConfig(num_pages=32, max_batched_tokens=4096, use_cuda_graph=False, max_model_len=1024))
        seqs = [Sequence(f"s{i}", p, SamplingParams(max_tokens=1, ignore_eos=True), return_hidden=True)
                for i, p in enumerate(prompts)]
        for s in seqs:
            eng.add_request(s)
        outs = []
        while eng.has_work():
            outs += eng.step()
        hid[name] = {o.seq_id: o.hidden for o in outs}
    for k in hid["g"]:
        assert _cos(hid["g"][k], hid["c"][k]) > 0.99


def test_llm_engine_gpu_sampling_in_graph_matches_eager():
    """Sampled requests: the CUDA-graph bursts (the draw index advances on the device) give the tokens of eager
    launches, a greedy request in the same batch keeps its tokens, and another seed changes the sampled ones."""
    torch.manual_seed(2)
    cfg = _llm_cfg()
    g = QwenLLM(cfg, device="cuda")
    for p in g.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.05)
    prompts = [np.arange(5, 300, dtype=np.int32), np.arange(900, 917, dtype=np.int32), np.arange(30, 160, dtype=np.int32)]

    def run(graph, seed, sample=True):
        ps = [SamplingParams(20, True), SamplingParams(20, True, temperature=1.2 if sample else 0.0, top_p=0.9, seed=seed),
              SamplingParams(20, True, temperature=0.8 if sample else 0.0, top_k=30, seed=seed + 1)]
        eng = LLMEngine(g, EngineConfig(num_pages=32, max_batched_tokens=256, decode_burst=5, use_cuda_graph=graph,
                                        max_model_len=1024))
        return eng.generate([Sequence(f"s{i}", p, ps[i]) for i, p in enumerate(prompts)])

    eager, graph, other, greedy = run(False, 3), run(True, 3), run(True, 4), run(True, 3, sample=False)
    torch.cuda.synchronize()
    ops.check_error("llm engine sampling")
    assert graph == eager
    assert graph["s0"] == greedy["s0"] and graph["s1"] != greedy["s1"] and graph["s2"] != greedy["s2"]
    assert other["s1"] != graph["s1"] and other["s0"] == graph["s0"]


def test_llm_fp8_projections_on_gpu():
    """The block-scaled e4m3 GEMM path inside the decoder (prefill, then CUDA-graph decode bursts) against the same
    weights in bf16."""
    torch.manual_seed(5)
    cfg = _llm_cfg()
    g = QwenLLM(cfg, device="cuda")
    for p in g.parameters():
        if p.dim() > 1:
            p.data.normal_(0, 0.05)
    prompts = [np.arange(5, 300, dtype=np.int32), np.arange(900, 917, dtype=np.int32)]

    def run(model, n_new=1):
        eng = LLMEngine(model, EngineConfig(num_pages=32, max_batched_tokens=256, decode_burst=5, max_model_len=1024))
        seqs = [Sequence(f"s{i}", p, SamplingParams(n_new, True), return_hidden=n_new == 1) for i, p in enumerate(prompts)]
        for s in seqs:
            eng.add_request(s)
        hid, toks = {}, {}
        while eng.has_work():
            for o in eng.step():
                toks.setdefault(o.seq_id, []).extend(o.new_token_ids)
                if o.hidden is not None:
                    hid[o.seq_id] = o.hidden
        return hid, toks

    h0, t0 = run(g)
    g.quantize_fp8_()
    h1, _ = run(g)
    _, t1 = run(g, n_new=12)
    torch.cuda.synchronize()
    ops.check_error("fp8 llm")
    assert g.layers[0].self_attn.o_proj.weight is None
    for k in h0:
        assert h0[k].shape == h1[k].shape and _cos(h0[k], h1[k]) > 0.97, k
    assert all(len(v) == 12 for v in t1.values())


def test_mllm_pipeline_end_to_end():
    torch.manual_seed(2)
    vcfg = Qwen25VisionConfig(depth=2, hidden_size=256, num_heads=4, intermediate_size=512, out_hidden_size=512,
                              fullatt_block_indexes=[1])
    lcfg = _llm_cfg()
    lcfg.vocab_size = 152064
    pipe = MLLMPipeline(Qwen25VisionTransformer(vcfg, device="cuda"), QwenLLM(lcfg, device="cuda"),
                        EngineConfig(num_pages=64, decode_burst=4, max_model_len=2048))
    rng = np.random.default_rng(0)
    reqs = [MLLMRequest(f"r{i}", rng.integers(10, 1000, 16).astype(np.int32),
                        [torch.from_numpy(rng.integers(0, 256, (224, 224, 3), dtype=np.uint8)) for _ in range(1 + i % 2)],
                        max_tokens=9, ignore_eos=True) for i in range(3)]
    a = pipe.generate(reqs)
    b = pipe.generate(reqs)
    torch.cuda.synchronize()
    ops.check_error("pipeline")
    assert a == b and all(len(v) == 9 for v in a.values())
    assert pipe.h2d_bytes > 0 and pipe.d2h_bytes > 0
