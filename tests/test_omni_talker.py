"""Qwen3-Omni talker against the Hugging Face modules with shared random weights (CPU fp32): projections, the MoE decoder
with its gated shared expert, the code predictor, the assembly of the talker's input from the thinker's tokens, and the
frame-by-frame generation loop (greedy, driven through the Hugging Face modules' forward passes as the oracle)."""

from types import SimpleNamespace

import numpy as np
import pytest
import torch

hf = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeTalkerConfig  # noqa: E402

from cornserve.models.omni_talker import Talker, TalkerConfig  # noqa: E402

SPECIAL = {"im_start": 90, "system": 91, "user": 92, "assistant": 93, "multimodal": (95, 96, 97)}


def _tiny():
    text = dict(vocab_size=96, hidden_size=64, intermediate_size=48, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                head_dim=16, moe_intermediate_size=32, num_experts_per_tok=2, num_experts=8, shared_expert_intermediate_size=40,
                norm_topk_prob=True, rope_parameters={"rope_theta": 10000.0, "rope_type": "default", "mrope_section": [4, 2, 2],
                                                      "mrope_interleaved": True})
    cp = dict(vocab_size=64, hidden_size=64, intermediate_size=80, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
              head_dim=16, num_code_groups=4)
    cfg = Qwen3OmniMoeTalkerConfig(text_config=text, code_predictor_config=cp, num_code_groups=4, thinker_hidden_size=48,
                                   codec_eos_token_id=70, codec_nothink_id=71, codec_think_bos_id=72, codec_think_eos_id=73,
                                   codec_pad_id=74, codec_bos_id=75, accept_hidden_layer=1, speaker_id={"ethan": 80}, spatial_merge_size=2)
    cfg.text_config._attn_implementation = "eager"
    cfg.code_predictor_config._attn_implementation = "eager"
    torch.manual_seed(0)
    ref = hf.Qwen3OmniMoeTalkerForConditionalGeneration(cfg).float().eval()
    for n, p in ref.named_parameters():
        if p.dim() == 1 and "norm" in n:
            torch.nn.init.normal_(p, 1.0, 0.1)
        else:
            torch.nn.init.normal_(p, 0, 0.08)
    mine = Talker(TalkerConfig.from_hf(cfg.to_dict()), device="cpu").float()
    sd = {"talker." + k: v for k, v in ref.state_dict().items()}
    loaded = mine.load_weights(sd.items())
    assert loaded == set(sd), sorted(set(sd) - loaded)[:10]
    return cfg, ref, mine


def test_projections_and_decoder_match_hf():
    cfg, ref, mine = _tiny()
    x = torch.randn(9, 48)
    assert torch.allclose(mine.text_projection(x), ref.text_projection(x), atol=1e-4)
    assert torch.allclose(mine.hidden_projection(x), ref.hidden_projection(x), atol=1e-4)
    emb = torch.randn(1, 11, 64) * 0.5
    with torch.inference_mode():
        out = ref.model(inputs_embeds=emb, use_cache=False)
        want_h, want_logits = out.last_hidden_state[0], ref.codec_head(out.last_hidden_state)[0]
        from cornserve.models.omni_talker import _embeds_meta

        m = _embeds_meta(11, 0, [1], torch.device("cpu"), decode=False)
        m.mm_embeds, m.mm_index = emb[0], torch.arange(11, dtype=torch.int32)
        got_h = mine.decoder.forward_hidden(m, mine.decoder.alloc_kv_cache(2))
        got_logits = mine.decoder.compute_logits(got_h)
    assert torch.allclose(got_h, want_h, atol=2e-3, rtol=2e-3)
    assert torch.allclose(got_logits, want_logits, atol=2e-3, rtol=2e-3)


def _thinker_view(n_prompt_user=7, n_answer=6):
    """Token ids of `system ... user (text + 3 image tokens) ... assistant answer` plus thinker-side vectors."""
    ids = [90, 91, 5, 6, 90, 92, 7, 95, 95, 95, 8, 9][: 5 + n_prompt_user] + [90, 93, 10] + list(range(20, 20 + n_answer))
    ids = np.asarray(ids)
    g = torch.Generator().manual_seed(3)
    return ids, torch.randn(len(ids), 48, generator=g), torch.randn(len(ids), 48, generator=g), torch.randn(3, 48, generator=g)


def test_input_assembly_matches_hf():
    cfg, ref, mine = _tiny()
    ids, embeds, hidden, tts = _thinker_view()
    prefill, trailing, tts_pad = mine.build_inputs(ids, embeds, hidden, tts, SPECIAL, speaker=80)
    # the Hugging Face helpers are methods of the full model; drive them with a stand-in that has what they touch
    stub = SimpleNamespace(config=SimpleNamespace(talker_config=cfg, tts_pad_token_id=0), talker=ref)
    mm = torch.from_numpy(np.isin(ids, SPECIAL["multimodal"]))[None]
    bos, eos, pad = ref.text_projection(tts[None]).chunk(3, dim=1)
    user = hf.Qwen3OmniMoeForConditionalGeneration._get_talker_user_parts(stub, 4, 12, mm, hidden[None], embeds[None])
    asst, _, trail = hf.Qwen3OmniMoeForConditionalGeneration._get_talker_assistant_parts(stub, 12, len(ids), 80, embeds[None], pad, bos, eos)
    want = torch.cat([user, asst], dim=1)[0]
    assert prefill.shape == want.shape and torch.allclose(prefill, want, atol=1e-4)
    assert torch.allclose(trailing, trail[0], atol=1e-4) and torch.allclose(tts_pad, pad[0, 0], atol=1e-4)


def test_greedy_generation_matches_a_loop_over_the_hf_modules():
    cfg, ref, mine = _tiny()
    ids, embeds, hidden, tts = _thinker_view()
    prefill, trailing, tts_pad = mine.build_inputs(ids, embeds, hidden, tts, SPECIAL, speaker=80)
    frames = 5
    got = torch.stack(list(mine.generate(prefill, trailing, tts_pad, max_frames=frames, sample=False)))
    # oracle: the same loop with the Hugging Face modules doing the arithmetic (full re-computation, no cache)
    allowed = torch.zeros(96, dtype=torch.bool)
    allowed[:64] = True
    allowed[70] = True
    seq, want = prefill[None].clone(), []
    with torch.inference_mode():
        for f in range(frames):
            h = ref.model(inputs_embeds=seq, use_cache=False).last_hidden_state[:, -1:]
            c0 = int(ref.codec_head(h)[0, 0].masked_fill(~allowed, float("-inf")).argmax())
            if c0 == 70:
                break
            e0 = ref.model.codec_embedding(torch.tensor([[c0]]))
            codes, total, cp_in = [c0], e0.clone(), torch.cat([h, e0], dim=1)
            for gi in range(3):
                hp = ref.code_predictor.model(inputs_embeds=cp_in, use_cache=False).last_hidden_state[:, -1:]
                c = int(ref.code_predictor.lm_head[gi](hp)[0, 0].argmax())
                codes.append(c)
                e = ref.code_predictor.model.codec_embedding[gi](torch.tensor([[c]]))
                total = total + e
                cp_in = torch.cat([cp_in, e], dim=1)
            want.append(codes)
            nxt = total + (trailing[f] if f < trailing.shape[0] else tts_pad)
            seq = torch.cat([seq, nxt], dim=1)
    assert got.tolist() == want


def test_thinker_view_round_trip_in_bf16():
    from cornserve.models.omni_talker import pack_thinker_view, unpack_thinker_view

    ids = np.asarray([0, 255, 256, 65535, 65536, 151671, 151936 - 1], dtype=np.int64)
    emb = torch.randn(len(ids), 64).bfloat16()
    hid = torch.randn(len(ids), 64).bfloat16()
    tts = torch.randn(3, 64).bfloat16()
    rows = pack_thinker_view(ids, emb, hid, tts)
    assert rows.shape == (len(ids) + 3, 3 * 64) and rows.dtype == torch.bfloat16
    ids2, emb2, hid2, tts2 = unpack_thinker_view(rows)
    assert ids2.tolist() == ids.tolist() and torch.equal(emb2, emb) and torch.equal(hid2, hid) and torch.equal(tts2, tts)


@pytest.mark.gpu
def test_talker_on_gpu_matches_cpu():
    """The same talker (bf16 on the GPU through the paged-KV kernels and the fused expert path, fp32 on the CPU): the
    decoder's hidden states of a prefill agree, and generation yields frames of valid codes."""
    from cornserve.models.omni_talker import _embeds_meta
    from cornserve.utils.hub import load_config

    cfg = TalkerConfig.from_hf(load_config("cornserve-b200/tiny-omni")["talker_config"])
    torch.manual_seed(3)
    cpu = Talker(cfg, device="cpu").float()
    gpu = Talker(cfg, device="cuda")
    gpu.load_state_dict({k: v.to(torch.bfloat16) for k, v in cpu.state_dict().items()})
    x = torch.randn(40, cfg.text.hidden_size) * 0.5
    with torch.inference_mode():
        outs = []
        for m, dev in ((cpu, "cpu"), (gpu, "cuda")):
            meta = _embeds_meta(40, 0, [1], torch.device(dev), decode=False)
            meta.mm_embeds, meta.mm_index = x.to(dev, m.dtype), torch.arange(40, dtype=torch.int32, device=dev)
            outs.append(m.decoder.forward_hidden(meta, m.decoder.alloc_kv_cache(2)).float().cpu())
        cos = torch.nn.functional.cosine_similarity(outs[0].flatten(), outs[1].flatten(), dim=0).item()
        assert cos > 0.99, cos
        pre = (torch.randn(20, cfg.text.hidden_size) * 0.5).to("cuda", torch.bfloat16)
        trail = (torch.randn(5, cfg.text.hidden_size) * 0.5).to("cuda", torch.bfloat16)
        frames = list(gpu.generate(pre, trail, trail[0], max_frames=6, sample=False, min_frames=6))
    from cornserve import ops

    ops.check_error("talker on the GPU")
    assert len(frames) == 6 and all(f.shape == (cfg.num_code_groups,) and int(f.max()) < cfg.predictor.vocab_size for f in frames)
