"""Encoder towers of the model registry against the Hugging Face modules with shared random weights (CPU fp32)."""

import numpy as np
import pytest
import torch


def _cos(a, b):
    return torch.nn.functional.cosine_similarity(a.flatten().float(), b.flatten().float(), dim=0).item()


def _randomise(module, std=0.05):
    for n, p in module.named_parameters():
        if p.dim() == 1 and ("norm" in n or "ln_" in n) and n.endswith("weight"):
            torch.nn.init.normal_(p, 1.0, 0.1)
        else:
            torch.nn.init.normal_(p, 0, std)


def _pooled(out):
    out = getattr(out, "pooler_output", out)
    return out[0] if isinstance(out, tuple) else out


def test_qwen2_vl_vision_matches_hf():
    hf = pytest.importorskip("transformers.models.qwen2_vl.modeling_qwen2_vl")
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig

    from cornserve.models.qwen2_vl import Qwen2VisionConfig, Qwen2VisionTransformer

    hf_cfg = Qwen2VLVisionConfig(depth=2, embed_dim=128, num_heads=4, hidden_size=192, mlp_ratio=4)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    ref = hf.Qwen2VisionTransformerPretrainedModel(hf_cfg).float().eval()
    _randomise(ref)
    cfg = Qwen2VisionConfig.from_hf(hf_cfg.to_dict())
    mine = Qwen2VisionTransformer(cfg, device="cpu").float()
    assert mine.load_weights(ref.state_dict().items()) == set(ref.state_dict())
    grids = [[1, 8, 12], [2, 4, 6]]
    pix = [torch.randn(g[0] * g[1] * g[2], cfg.patch_dim) for g in grids]
    with torch.inference_mode():
        want = _pooled(ref(torch.cat(pix), torch.tensor(grids)))
        got = torch.cat(mine("image", None, {"pixel_values": pix, "image_grid_thw": grids}))
    assert got.shape == want.shape and _cos(got, want) > 0.999
    assert torch.allclose(got, want, atol=3e-3, rtol=3e-3)


def test_qwen3_vl_vision_matches_hf():
    hf = pytest.importorskip("transformers.models.qwen3_vl.modeling_qwen3_vl")
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig

    from cornserve.models.qwen3_vl import Qwen3VisionConfig, Qwen3VisionTransformer

    hf_cfg = Qwen3VLVisionConfig(depth=3, hidden_size=128, num_heads=4, intermediate_size=256, out_hidden_size=160,
                                 num_position_embeddings=36, deepstack_visual_indexes=[0, 2], patch_size=16)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(0)
    ref = hf.Qwen3VLVisionModel(hf_cfg).float().eval()
    _randomise(ref)
    cfg = Qwen3VisionConfig.from_hf(hf_cfg.to_dict())
    mine = Qwen3VisionTransformer(cfg, device="cpu").float()
    assert mine.load_weights(ref.state_dict().items()) == set(ref.state_dict())
    grids = [[1, 8, 12], [2, 4, 6]]
    pix = [torch.randn(g[0] * g[1] * g[2], cfg.patch_dim) for g in grids]
    with torch.inference_mode():
        out = ref(torch.cat(pix), torch.tensor(grids))
        want = torch.cat([out.pooler_output, *out.deepstack_features], dim=1)
        got = torch.cat(mine("image", None, {"pixel_values": pix, "image_grid_thw": grids}))
    assert got.shape == want.shape == (8 * 12 // 4 + 2 * 4 * 6 // 4, 160 * 3)
    assert _cos(got, want) > 0.999 and torch.allclose(got, want, atol=3e-3, rtol=3e-3)


def test_qwen2_5_omni_audio_and_vision_match_hf():
    hf = pytest.importorskip("transformers.models.qwen2_5_omni.modeling_qwen2_5_omni")
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import (Qwen2_5OmniAudioEncoderConfig,
                                                                            Qwen2_5OmniVisionEncoderConfig)

    from cornserve.models.omni_audio import AudioEncoder, AudioEncoderConfig
    from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer

    torch.manual_seed(0)
    a_cfg = Qwen2_5OmniAudioEncoderConfig(num_mel_bins=16, d_model=64, encoder_layers=2, encoder_attention_heads=4,
                                          encoder_ffn_dim=128, max_source_positions=100, n_window=10, output_dim=48)
    a_cfg._attn_implementation = "eager"
    ref = hf.Qwen2_5OmniAudioEncoder(a_cfg).float().eval()
    _randomise(ref)
    mine = AudioEncoder(AudioEncoderConfig.from_hf(a_cfg.to_dict(), conv2d_stem=False), device="cpu").float()
    loaded = mine.load_weights(ref.state_dict().items())
    assert set(ref.state_dict()) - loaded == {"audio_bos_eos_token.weight"}
    lens = [47, 20, 31]
    mels = [torch.randn(16, n) for n in lens]
    with torch.inference_mode():
        fl = torch.tensor(lens)
        after = (fl - 1) // 2 + 1
        want = ref(torch.cat(mels, dim=1), feature_lens=fl, aftercnn_lens=after).last_hidden_state
        got = mine("audio", None, {"input_features": mels})
    assert [g.shape[0] for g in got] == [int(a) // 2 for a in after]
    got = torch.cat(got)
    assert got.shape == want.shape and _cos(got, want) > 0.999 and torch.allclose(got, want, atol=3e-3, rtol=3e-3)

    v_cfg = Qwen2_5OmniVisionEncoderConfig(depth=2, hidden_size=128, num_heads=4, intermediate_size=256, out_hidden_size=96,
                                           fullatt_block_indexes=[1], window_size=112)
    v_cfg._attn_implementation = "eager"
    vref = hf.Qwen2_5OmniVisionEncoder(v_cfg).float().eval()
    _randomise(vref)
    vmine = Qwen25VisionTransformer(Qwen25VisionConfig.from_hf(v_cfg.to_dict()), device="cpu").float()
    assert vmine.load_weights(vref.state_dict().items()) == set(vref.state_dict())
    grids = [[1, 16, 24], [1, 10, 8]]
    pix = [torch.randn(g[1] * g[2], vmine.cfg.patch_dim) for g in grids]
    with torch.inference_mode():
        want = _pooled(vref(torch.cat(pix), torch.tensor(grids)))
        got = torch.cat(vmine("image", None, {"pixel_values": pix, "image_grid_thw": grids}))
    assert got.shape == want.shape and _cos(got, want) > 0.999


def test_qwen3_omni_audio_matches_hf():
    hf = pytest.importorskip("transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe")
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeAudioEncoderConfig

    from cornserve.models.omni_audio import AudioEncoder, AudioEncoderConfig

    torch.manual_seed(0)
    a_cfg = Qwen3OmniMoeAudioEncoderConfig(num_mel_bins=16, d_model=64, encoder_layers=2, encoder_attention_heads=4,
                                           encoder_ffn_dim=128, max_source_positions=100, n_window=50, output_dim=48,
                                           downsample_hidden_size=24, n_window_infer=200, conv_chunksize=4)
    a_cfg._attn_implementation = "eager"
    ref = hf.Qwen3OmniMoeAudioEncoder(a_cfg).float().eval()
    _randomise(ref)
    mine = AudioEncoder(AudioEncoderConfig.from_hf(a_cfg.to_dict(), conv2d_stem=True), device="cpu").float()
    assert mine.load_weights(ref.state_dict().items()) == set(ref.state_dict())
    # the HF module's eager attention path ignores its own window boundaries, so exact agreement is checked on an
    # audio that fits one attention window (<= n_window_infer frames); longer inputs are checked for their shape
    mel = torch.randn(16, 137)
    with torch.inference_mode():
        want = ref(mel, feature_lens=torch.tensor([137])).last_hidden_state
        got = torch.cat(mine("audio", None, {"input_features": [mel]}))
    assert got.shape == want.shape == (18, 48)
    assert _cos(got, want) > 0.9999 and torch.allclose(got, want, atol=3e-3, rtol=3e-3)
    lens = [250, 100, 137]
    outs = mine("audio", None, {"input_features": [torch.randn(16, n) for n in lens]})
    assert [o.shape[0] for o in outs] == [33, 13, 18]


def test_omni_encoder_routes_modalities():
    from cornserve.models.qwen_omni import OmniEncoderConfig, Qwen3OmniEncoder

    cfg = OmniEncoderConfig.from_hf({"model_type": "qwen3_omni_moe", "thinker_config": {
        "vision_config": {"depth": 1, "hidden_size": 64, "num_heads": 2, "intermediate_size": 128, "out_hidden_size": 48,
                          "num_position_embeddings": 16, "deepstack_visual_indexes": [0]},
        "audio_config": {"num_mel_bins": 16, "d_model": 64, "encoder_layers": 1, "encoder_attention_heads": 2,
                         "encoder_ffn_dim": 64, "max_source_positions": 100, "n_window": 50, "output_dim": 48,
                         "downsample_hidden_size": 8, "n_window_infer": 200}}})
    m = Qwen3OmniEncoder(cfg, device="cpu").float()
    out = m("audio", None, {"input_features": [torch.randn(16, 120)]})
    assert out[0].shape[1] == 48
    img = m("image", None, {"pixel_values": [torch.randn(16, m.visual.cfg.patch_dim)], "image_grid_thw": [[1, 4, 4]]})
    assert img[0].shape == (4, 96)


def test_gemma3_encoder_matches_hf_and_shares_the_tower():
    hf = pytest.importorskip("transformers.models.gemma3.modeling_gemma3")
    from transformers.models.gemma3.configuration_gemma3 import Gemma3Config
    from transformers.models.siglip.modeling_siglip import SiglipVisionModel

    from cornserve.models.siglip import Gemma3VisionConfig, Gemma3VisionEncoder

    torch.manual_seed(0)
    vis = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2, image_size=112, patch_size=14,
               vision_use_head=False)
    hf_cfg = Gemma3Config(vision_config=vis, text_config=dict(hidden_size=96, num_hidden_layers=1, num_attention_heads=2,
                                                              num_key_value_heads=1, intermediate_size=64, vocab_size=64),
                          mm_tokens_per_image=16)
    hf_cfg.vision_config._attn_implementation = "eager"
    tower = SiglipVisionModel(hf_cfg.vision_config).float().eval()
    proj = hf.Gemma3MultiModalProjector(hf_cfg).float().eval()
    _randomise(tower)
    _randomise(proj)
    cfg = Gemma3VisionConfig.from_hf(hf_cfg.to_dict())
    mine = Gemma3VisionEncoder(cfg, device="cpu", model_id="google/gemma-3-4b-it").float()
    sd = {"vision_tower." + k: v for k, v in tower.state_dict().items()}
    sd.update({"multi_modal_projector." + k: v for k, v in proj.state_dict().items()})
    assert mine.load_weights(sd.items()) == set(sd)
    pix = [torch.randn(1, 3, 112, 112), torch.randn(2, 3, 112, 112)]
    with torch.inference_mode():
        want = proj(tower(torch.cat(pix)).last_hidden_state)
        got = mine("image", "google/gemma-3-4b-it", {"pixel_values": pix, "num_crops": [torch.tensor([0]), torch.tensor([1])]})
    assert [g.shape for g in got] == [(16, 96), (32, 96)]
    assert _cos(torch.cat(got), want.flatten(0, 1)) > 0.9999
    # a second LLM size shares the tower through its own projector
    big = dict(hf_cfg.to_dict(), text_config=dict(hidden_size=160))
    proj2 = hf.Gemma3MultiModalProjector(Gemma3Config(vision_config=vis, text_config=dict(hidden_size=160), mm_tokens_per_image=16)).float()
    _randomise(proj2)
    mine.add_adapter("google/gemma-3-12b-it", big, proj2.state_dict().items())
    with torch.inference_mode():
        got2 = mine("image", "google/gemma-3-12b-it", {"pixel_values": pix[:1], "num_crops": [torch.tensor([0])]})
        want2 = proj2(tower(pix[0]).last_hidden_state)
    assert got2[0].shape == (16, 160) and _cos(got2[0], want2[0]) > 0.9999


def test_llava_onevision_encoder_matches_hf():
    hf = pytest.importorskip("transformers.models.llava_onevision.modeling_llava_onevision")
    from transformers.models.llava_onevision.configuration_llava_onevision import LlavaOnevisionConfig

    from cornserve.models.siglip import LlavaOnevisionEncoder, LlavaOnevisionVisionConfig

    torch.manual_seed(0)
    S = 56
    hf_cfg = LlavaOnevisionConfig(
        vision_config=dict(model_type="siglip_vision_model", hidden_size=64, intermediate_size=128, num_hidden_layers=3,
                           num_attention_heads=2, image_size=S, patch_size=14, vision_use_head=False),
        text_config=dict(model_type="qwen2", hidden_size=96, num_hidden_layers=1, num_attention_heads=2, num_key_value_heads=1,
                         intermediate_size=64, vocab_size=64),
        image_grid_pinpoints=[[S, S], [S, 2 * S], [2 * S, S], [2 * S, 2 * S], [S, 3 * S]], vision_feature_layer=-1,
        vision_feature_select_strategy="full")
    hf_cfg.vision_config._attn_implementation = "eager"
    ref = hf.LlavaOnevisionModel(hf_cfg).float().eval()
    _randomise(ref)
    mine = LlavaOnevisionEncoder(LlavaOnevisionVisionConfig.from_hf(hf_cfg.to_dict()), device="cpu").float()
    sd = {k: v for k, v in ref.state_dict().items() if not k.startswith("language_model")}
    loaded = mine.load_weights(sd.items())
    assert {k for k in sd if "vision_model.head" not in k} <= loaded
    sizes = [(50, 120), (100, 90)]           # (height, width): a wide image (1x3 tiles -> pinpoint [S, 3S]) and a 2x2 one
    tiles = [1 + 3, 1 + 4]
    pix = [torch.randn(n, 3, S, S) for n in tiles]
    with torch.inference_mode():
        out = ref.get_image_features(torch.cat(pix), torch.tensor(sizes), vision_feature_layer=-1,
                                     vision_feature_select_strategy="full", vision_aspect_ratio="anyres_max_9")
        want = out.pooler_output
        got = mine("image", None, {"pixel_values": pix, "image_sizes": [torch.tensor(s) for s in sizes]})
    for g, w in zip(got, want):
        assert g.shape == w.shape and _cos(g, w) > 0.9999


def test_internvl_encoder_matches_restatement():
    """InternViT + pixel shuffle + projector against a plain PyTorch restatement that uses the checkpoint's names."""
    import torch.nn.functional as F

    from cornserve.models.internvl import InternVLEncoder, InternVLVisionConfig, pixel_shuffle

    torch.manual_seed(0)
    cfg = InternVLVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=3, num_attention_heads=4, image_size=56,
                               patch_size=14, qk_normalization=True, norm_type="rms_norm", llm_hidden_size=96, select_layer=-1)
    H, L, heads = cfg.hidden_size, cfg.num_hidden_layers, cfg.num_attention_heads
    r = lambda *s, std=0.1: torch.randn(*s) * std  # noqa: E731
    w = {"vision_model.embeddings.class_embedding": r(1, 1, H), "vision_model.embeddings.position_embedding": r(1, 17, H),
         "vision_model.embeddings.patch_embedding.weight": r(H, 3, 14, 14, std=0.05), "vision_model.embeddings.patch_embedding.bias": r(H),
         "mlp1.0.weight": 1 + r(4 * H), "mlp1.0.bias": r(4 * H), "mlp1.1.weight": r(96, 4 * H), "mlp1.1.bias": r(96),
         "mlp1.3.weight": r(96, 96), "mlp1.3.bias": r(96)}
    for i in range(L):
        p = f"vision_model.encoder.layers.{i}."
        w.update({p + "norm1.weight": 1 + r(H), p + "norm2.weight": 1 + r(H), p + "attn.qkv.weight": r(3 * H, H), p + "attn.qkv.bias": r(3 * H),
                  p + "attn.q_norm.weight": 1 + r(H), p + "attn.k_norm.weight": 1 + r(H), p + "attn.proj.weight": r(H, H),
                  p + "attn.proj.bias": r(H), p + "mlp.fc1.weight": r(128, H), p + "mlp.fc1.bias": r(128), p + "mlp.fc2.weight": r(H, 128),
                  p + "mlp.fc2.bias": r(H), p + "ls1": 0.5 + r(H), p + "ls2": 0.5 + r(H)})
    mine = InternVLEncoder(cfg, device="cpu").float()
    assert mine.load_weights(w.items()) == set(w)

    def rms(x, wt):
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * wt

    pix = torch.randn(3, 3, 56, 56)
    x = F.conv2d(pix, w["vision_model.embeddings.patch_embedding.weight"], w["vision_model.embeddings.patch_embedding.bias"], stride=14)
    x = x.flatten(2).transpose(1, 2)
    x = torch.cat([w["vision_model.embeddings.class_embedding"].expand(3, -1, -1), x], dim=1) + w["vision_model.embeddings.position_embedding"]
    for i in range(L):
        p = f"vision_model.encoder.layers.{i}."
        h = rms(x, w[p + "norm1.weight"])
        q, k, v = F.linear(h, w[p + "attn.qkv.weight"], w[p + "attn.qkv.bias"]).chunk(3, dim=-1)
        q, k = rms(q, w[p + "attn.q_norm.weight"]), rms(k, w[p + "attn.k_norm.weight"])
        sp = lambda t: t.view(3, 17, heads, H // heads).transpose(1, 2)  # noqa: E731
        a = F.scaled_dot_product_attention(sp(q), sp(k), sp(v)).transpose(1, 2).reshape(3, 17, H)
        x = x + F.linear(a, w[p + "attn.proj.weight"], w[p + "attn.proj.bias"]) * w[p + "ls1"]
        h = rms(x, w[p + "norm2.weight"])
        h = F.linear(F.gelu(F.linear(h, w[p + "mlp.fc1.weight"], w[p + "mlp.fc1.bias"])), w[p + "mlp.fc2.weight"], w[p + "mlp.fc2.bias"])
        x = x + h * w[p + "ls2"]
    x = pixel_shuffle(x[:, 1:].reshape(3, 4, 4, H), 0.5, "v2").reshape(3, 4, 4 * H)
    x = F.layer_norm(x, (4 * H,), w["mlp1.0.weight"], w["mlp1.0.bias"])
    want = F.linear(F.gelu(F.linear(x, w["mlp1.1.weight"], w["mlp1.1.bias"])), w["mlp1.3.weight"], w["mlp1.3.bias"])
    got = mine("image", None, {"pixel_values": [pix[:1], pix[1:]]})
    assert [g.shape for g in got] == [(4, 96), (8, 96)]
    assert _cos(torch.cat(got), want.flatten(0, 1)) > 0.9999


@pytest.mark.parametrize("model_id,modality,adapter,width", [
    ("cornserve-b200/tiny-qwen2-vl", "image", None, 96),
    ("cornserve-b200/tiny-qwen3-vl", "video", None, 192),
    ("cornserve-b200/tiny-qwen3-omni", "audio", None, 96),
    ("cornserve-b200/tiny-qwen2.5-omni", "audio", None, 96),
    ("cornserve-b200/tiny-qwen2.5-omni", "image", None, 96),
    ("cornserve-b200/tiny-gemma3", "image", "cornserve-b200/tiny-gemma3-large", 512),
    ("cornserve-b200/tiny-llava-onevision", "image", None, 96),
    ("cornserve-b200/tiny-internvl", "image", None, 96),
])
def test_every_registered_encoder_runs_through_the_worker(model_id, modality, adapter, width, monkeypatch, tmp_path):
    """Registry entry -> worker -> preprocessing recipe -> forward, on raw decoded inputs, for each model family."""
    from cornserve.task_executors.eric.config import EricConfig, ModelConfig
    from cornserve.task_executors.eric.schema import Batch, Modality
    from cornserve.task_executors.eric.worker import Worker

    monkeypatch.setenv("CORNSERVE_DEVICE", "cpu")
    monkeypatch.setenv("CORNSERVE_TEST_DUMP_TENSOR_DIR", str(tmp_path))
    cfg = EricConfig(model=ModelConfig(id=model_id, modality=Modality(modality), adapter_model_ids=[adapter] if adapter else []))
    w = Worker(cfg)
    rng = np.random.default_rng(0)
    if modality == "audio":
        data = {"raw_audio": [torch.from_numpy(rng.standard_normal(16000 * 2).astype(np.float32) * 0.1)]}
    elif modality == "video":
        data = {"raw_videos": [torch.from_numpy(rng.integers(0, 256, (4, 64, 96, 3), dtype=np.uint8))]}
    else:
        data = {"raw_images": [torch.from_numpy(rng.integers(0, 256, (70, 120, 3), dtype=np.uint8))]}
    w.execute_model(Batch(Modality(modality), adapter or model_id, ["r"], ["d0"], [None], data))
    out = torch.load(tmp_path / "d0.pt")
    assert out.dim() == 2 and out.shape[1] == width and out.shape[0] > 0 and torch.isfinite(out.float()).all()
