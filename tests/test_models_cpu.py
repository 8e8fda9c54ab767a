"""CPU fp32 checks of the model definitions against Hugging Face modules with shared random weights."""

import numpy as np
import pytest
import torch

from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer, window_index
from cornserve.models.qwen_llm import BatchMeta, LLMConfig, QwenLLM


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().float(), b.flatten().float(), dim=0).item()


def _tiny_vision_cfg():
    return Qwen25VisionConfig(depth=2, hidden_size=128, num_heads=4, intermediate_size=500, out_hidden_size=256,
                              fullatt_block_indexes=[1])


def test_vision_tower_matches_hf():
    hf = pytest.importorskip("transformers.models.qwen2_5_vl.modeling_qwen2_5_vl")
    from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLVisionConfig

    cfg = _tiny_vision_cfg()
    torch.manual_seed(0)
    hf_cfg = Qwen2_5_VLVisionConfig(depth=cfg.depth, hidden_size=cfg.hidden_size, num_heads=cfg.num_heads,
                                    intermediate_size=cfg.intermediate_size, out_hidden_size=cfg.out_hidden_size,
                                    fullatt_block_indexes=cfg.fullatt_block_indexes, window_size=cfg.window_size)
    hf_cfg._attn_implementation = "eager"
    ref = hf.Qwen2_5_VisionTransformerPretrainedModel(hf_cfg).float().eval()
    for p in ref.parameters():
        torch.nn.init.normal_(p, 0, 0.05)
    mine = Qwen25VisionTransformer(cfg, device="cpu").float()
    loaded = mine.load_weights(ref.state_dict().items())
    assert len(loaded) == len(ref.state_dict())
    grids = [[1, 16, 24], [1, 10, 8]]
    pix = [torch.randn(g[1] * g[2], cfg.patch_dim) for g in grids]
    with torch.inference_mode():
        want = ref(torch.cat(pix), torch.tensor(grids))
        want = getattr(want, "pooler_output", want)
        if isinstance(want, tuple):
            want = want[0]
        got = mine("image", None, {"pixel_values": pix, "image_grid_thw": [torch.tensor(g) for g in grids]})
    got = torch.cat(got)
    assert got.shape == want.shape
    assert _cos(got, want) > 0.999
    assert torch.allclose(got, want, atol=2e-3, rtol=2e-3)


def test_window_index_is_permutation():
    grid = np.array([[1, 52, 92], [2, 16, 16]])
    idx, cu = window_index(grid, 112, 2, 14)
    n = int((grid[:, 0] * grid[:, 1] * grid[:, 2]).sum()) // 4
    assert sorted(idx.tolist()) == list(range(n))
    assert cu[0] == 0 and cu[-1] == n * 4 and (np.diff(cu) > 0).all() and np.diff(cu).max() <= 64


def _tiny_llm_cfg(**kw):
    base = dict(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                intermediate_size=512, vocab_size=1024, mrope_section=[8, 12, 12], rope_theta=10000.0)
    base.update(kw)
    return LLMConfig(**base)


def _run_llm(model, ids_list, pages=8):
    """Prefill all sequences in one flattened batch, then decode 3 tokens greedily."""
    B = len(ids_list)
    caches = model.alloc_kv_cache(pages)
    lens = [len(x) for x in ids_list]
    bt = torch.zeros(B, 2, dtype=torch.int32)
    for s in range(B):
        bt[s, 0], bt[s, 1] = 1 + 2 * s, 2 + 2 * s
    flat = torch.tensor([t for x in ids_list for t in x], dtype=torch.int32)
    pos = torch.cat([torch.arange(n) for n in lens]).int()
    slots = torch.cat([bt[s, 0] * 128 + torch.arange(lens[s]) for s in range(B)]).int()
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    m = BatchMeta(flat, pos[None].expand(3, -1).contiguous(), slots, cu, torch.tensor(lens, dtype=torch.int32), bt,
                  (cu[1:] - 1).int(), max(lens))
    outs = []
    tok, _ = model(m, caches)
    outs.append(tok.clone())
    cur = list(lens)
    for _ in range(3):
        pos = torch.tensor(cur, dtype=torch.int32)
        slots = torch.tensor([int(bt[s, 0]) * 128 + cur[s] for s in range(B)], dtype=torch.int32)
        cur = [c + 1 for c in cur]
        m = BatchMeta(tok.int(), pos[None].expand(3, -1).contiguous(), slots, torch.arange(B + 1, dtype=torch.int32),
                      torch.tensor(cur, dtype=torch.int32), bt, torch.arange(B, dtype=torch.int32), 1, True)
        tok, _ = model(m, caches)
        outs.append(tok.clone())
    return torch.stack(outs, 1)


def test_llm_matches_hf_qwen2():
    tr = pytest.importorskip("transformers")
    cfg = _tiny_llm_cfg(mrope_section=None)
    hf_cfg = tr.Qwen2Config(hidden_size=256, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                            intermediate_size=512, vocab_size=1024, rope_theta=10000.0, rms_norm_eps=1e-6,
                            max_position_embeddings=512, tie_word_embeddings=False)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    ref = tr.Qwen2ForCausalLM(hf_cfg).float().eval()
    for n, p in ref.named_parameters():
        if "norm" not in n:
            torch.nn.init.normal_(p, 0, 0.08)
    mine = QwenLLM(cfg, device="cpu").float()
    loaded = mine.load_weights(ref.state_dict().items())
    assert len(loaded) == len(ref.state_dict())
    prompts = [list(range(5, 25)), list(range(100, 107))]
    got = _run_llm(mine, prompts)
    for s, p in enumerate(prompts):
        with torch.inference_mode():
            want = ref.generate(torch.tensor([p]), max_new_tokens=4, do_sample=False)[0, len(p):]
        assert got[s].tolist() == want.tolist()


def test_moe_llm_runs_and_is_deterministic():
    cfg = _tiny_llm_cfg(num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64, qk_norm=True,
                        attention_bias=False)
    torch.manual_seed(1)
    m = QwenLLM(cfg, device="cpu").float()
    a = _run_llm(m, [list(range(3, 30))])
    b = _run_llm(m, [list(range(3, 30))])
    assert torch.equal(a, b) and a.shape == (1, 4)
