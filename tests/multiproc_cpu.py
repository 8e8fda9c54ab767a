"""Two-rank (gloo, CPU) checks of the host-side parallel logic: weight sharding, head / token ownership, index tables
and the order of the collectives.  Launched by ``test_parallel_cpu.py`` once per rank; prints ``MULTIPROC_CPU_OK``."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from cornserve.parallel.state import init_distributed, single_group  # noqa: E402


def cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


def sp_dit(g):
    from test_geri_models import dit_weights

    from cornserve.models.qwen_image import QwenImageDiT, QwenImageDiTConfig

    cfg = QwenImageDiTConfig(in_channels=16, out_channels=4, num_layers=2, attention_head_dim=64, num_attention_heads=4,
                             joint_attention_dim=64, axes_dims_rope=(8, 28, 28))
    w = dit_weights(cfg)
    P, rank = g.size, g.rank
    sp = QwenImageDiT(cfg, group=g)
    sp.load_weights(w.items())
    one = QwenImageDiT(cfg, group=single_group())
    one.load_weights(w.items())
    gen = torch.Generator().manual_seed(3)
    for B, (h, wd), n_txt, txt_len in ((2, (4, 6), 8, [8, 8]), (2, (4, 4), 8, [8, 5]), (1, (6, 4), 4, [1])):
        n_img = h * wd
        lat = torch.randn(B * n_img, cfg.in_channels, generator=gen).bfloat16()
        prompt = torch.randn(B * n_txt, cfg.joint_attention_dim, generator=gen).bfloat16()
        t = torch.linspace(0.8, 0.2, B)
        want = one(lat, prompt, t, one.make_layout(B, txt_len, n_txt, (h, wd)))
        shard = lambda x, n: x.view(B, P, n // P, -1)[:, rank].reshape(B * (n // P), -1).contiguous()  # noqa: E731
        lay = sp.make_layout(B, txt_len, n_txt, (h, wd))
        assert lay.fused is None and lay.sp == P
        got = sp(shard(lat, n_img), shard(prompt, n_txt), t, lay)
        c = cos(got, shard(want, n_img))
        assert c > 0.995, f"sequence-parallel DiT differs from the single-process result (cos {c:.4f})"


def tp_llm(g):
    from multigpu_fused import hf_style_weights

    from cornserve.task_executors.llm.engine import EngineConfig, LLMEngine, SamplingParams, Sequence
    from cornserve.models.qwen_llm import LLMConfig, QwenLLM

    cfg = LLMConfig(hidden_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                    intermediate_size=256, vocab_size=512, eos_token_id=511)
    weights = hf_style_weights(cfg)
    outs = {}
    for name, group in (("tp", g), ("single", single_group())):
        model = QwenLLM(cfg, group=group, device="cpu")
        assert len(model.load_weights(weights.items())) == len(weights)
        eng = LLMEngine(model, EngineConfig(num_pages=16, max_batched_tokens=256, decode_burst=2, max_model_len=512))
        for i in range(2):
            eng.add_request(Sequence(f"s{i}", np.arange(3 + i, 40 + 9 * i, dtype=np.int32), SamplingParams(4, True), return_hidden=True))
        toks, hid = {}, {}
        while eng.has_work():
            for o in eng.step():
                toks.setdefault(o.seq_id, []).extend(o.new_token_ids)
                if o.hidden is not None:
                    hid[o.seq_id] = o.hidden
        outs[name] = (toks, hid)
    for sid in outs["single"][0]:
        c = cos(outs["tp"][1][sid], outs["single"][1][sid])
        assert c > 0.99, f"{sid}: tensor-parallel hidden states differ (cos {c:.4f})"
        assert outs["tp"][0][sid][0] == outs["single"][0][sid][0]


def tp_vit(g):
    from multigpu_fused import vit_weights

    from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer

    cfg = Qwen25VisionConfig(depth=2, hidden_size=128, num_heads=4, intermediate_size=256, out_hidden_size=64,
                             fullatt_block_indexes=[1], window_size=56)
    weights = vit_weights(cfg)
    tp = Qwen25VisionTransformer(cfg, group=g, device="cpu")
    tp.load_weights(weights.items())
    one = Qwen25VisionTransformer(cfg, group=single_group(), device="cpu")
    one.load_weights(weights.items())
    grid = np.asarray([[1, 8, 12], [2, 4, 4]])
    L = int(grid.prod(axis=1).sum())
    pix = (torch.randn(L, cfg.patch_dim, generator=torch.Generator().manual_seed(5)) * 0.5).bfloat16()
    c = cos(tp.encode(pix, grid), one.encode(pix, grid))
    assert c > 0.995, f"tensor-parallel vision tower differs (cos {c:.4f})"


def tp_encoder_families(g):
    """Every other encoder family of the registry, tensor parallel over two ranks against the single-process model
    (both loaded from one full checkpoint, so this checks the sharding of fused qkv, biases, MLP columns, layer
    scale, the all-head q/k norm of InternViT and the reductions)."""
    import torch.nn as nn
    from test_encoder_models import _randomise

    def compare(name, make, sd, call):
        tp, one = make(g), make(single_group())
        for m in (tp, one):
            m.float()
            m.load_weights(list(sd.items()))
        with torch.inference_mode():
            got, want = torch.cat(call(tp)), torch.cat(call(one))
        c = cos(got, want)
        assert got.shape == want.shape and c > 0.9995, f"{name}: tensor-parallel output differs (cos {c:.5f})"

    torch.manual_seed(0)
    # Qwen2-VL
    from transformers.models.qwen2_vl import modeling_qwen2_vl as hf2
    from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLVisionConfig

    from cornserve.models.qwen2_vl import Qwen2VisionConfig, Qwen2VisionTransformer

    hc = Qwen2VLVisionConfig(depth=2, embed_dim=128, num_heads=4, hidden_size=192, mlp_ratio=4)
    ref: nn.Module = hf2.Qwen2VisionTransformerPretrainedModel(hc).float()
    _randomise(ref)
    cfg2 = Qwen2VisionConfig.from_hf(hc.to_dict())
    grids = [[1, 8, 12], [2, 4, 6]]
    pix = [torch.randn(a * b * c, cfg2.patch_dim) for a, b, c in grids]
    compare("qwen2_vl", lambda grp: Qwen2VisionTransformer(cfg2, group=grp), ref.state_dict(),
            lambda m: m("image", None, {"pixel_values": pix, "image_grid_thw": grids}))
    # Qwen3-VL (deep-stack mergers, bilinear position table)
    from transformers.models.qwen3_vl import modeling_qwen3_vl as hf3
    from transformers.models.qwen3_vl.configuration_qwen3_vl import Qwen3VLVisionConfig

    from cornserve.models.qwen3_vl import Qwen3VisionConfig, Qwen3VisionTransformer

    hc = Qwen3VLVisionConfig(depth=3, hidden_size=128, num_heads=4, intermediate_size=256, out_hidden_size=160,
                             num_position_embeddings=36, deepstack_visual_indexes=[0, 2], patch_size=16)
    ref = hf3.Qwen3VLVisionModel(hc).float()
    _randomise(ref)
    cfg3 = Qwen3VisionConfig.from_hf(hc.to_dict())
    pix3 = [torch.randn(a * b * c, cfg3.patch_dim) for a, b, c in grids]
    compare("qwen3_vl", lambda grp: Qwen3VisionTransformer(cfg3, group=grp), ref.state_dict(),
            lambda m: m("image", None, {"pixel_values": pix3, "image_grid_thw": grids}))
    # Qwen2.5-Omni audio tower
    from transformers.models.qwen2_5_omni import modeling_qwen2_5_omni as hfo
    from transformers.models.qwen2_5_omni.configuration_qwen2_5_omni import Qwen2_5OmniAudioEncoderConfig

    from cornserve.models.omni_audio import AudioEncoder, AudioEncoderConfig

    ac = Qwen2_5OmniAudioEncoderConfig(num_mel_bins=16, d_model=64, encoder_layers=2, encoder_attention_heads=4,
                                       encoder_ffn_dim=128, max_source_positions=100, n_window=10, output_dim=48)
    ref = hfo.Qwen2_5OmniAudioEncoder(ac).float()
    _randomise(ref)
    acfg = AudioEncoderConfig.from_hf(ac.to_dict(), conv2d_stem=False)
    mels = [torch.randn(16, n) for n in (47, 20, 31)]
    compare("qwen2_5_omni audio", lambda grp: AudioEncoder(acfg, group=grp), ref.state_dict(),
            lambda m: m("audio", None, {"input_features": mels}))
    # Gemma-3 (SigLIP tower + projector)
    from transformers.models.gemma3 import modeling_gemma3 as hfg
    from transformers.models.gemma3.configuration_gemma3 import Gemma3Config
    from transformers.models.siglip.modeling_siglip import SiglipVisionModel

    from cornserve.models.siglip import Gemma3VisionConfig, Gemma3VisionEncoder

    vis = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=2, image_size=112, patch_size=14,
               vision_use_head=False)
    gc = Gemma3Config(vision_config=vis, text_config=dict(hidden_size=96, num_hidden_layers=1, num_attention_heads=2,
                                                          num_key_value_heads=1, intermediate_size=64, vocab_size=64),
                      mm_tokens_per_image=16)
    tower, proj = SiglipVisionModel(gc.vision_config).float(), hfg.Gemma3MultiModalProjector(gc).float()
    _randomise(tower)
    _randomise(proj)
    sd = {"vision_tower." + k: v for k, v in tower.state_dict().items()}
    sd.update({"multi_modal_projector." + k: v for k, v in proj.state_dict().items()})
    gcfg = Gemma3VisionConfig.from_hf(gc.to_dict())
    gpix = [torch.randn(1, 3, 112, 112), torch.randn(2, 3, 112, 112)]
    compare("gemma3", lambda grp: Gemma3VisionEncoder(gcfg, group=grp, model_id="google/gemma-3-4b-it"), sd,
            lambda m: m("image", "google/gemma-3-4b-it", {"pixel_values": gpix, "num_crops": [torch.tensor([0]), torch.tensor([1])]}))
    # InternVL (layer scale, q/k norm over all heads)
    from cornserve.models.internvl import InternVLEncoder, InternVLVisionConfig

    icfg = InternVLVisionConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, image_size=56,
                                patch_size=14, qk_normalization=True, norm_type="rms_norm", llm_hidden_size=96, select_layer=-1)
    H = icfg.hidden_size
    r = lambda *s, std=0.1: torch.randn(*s) * std  # noqa: E731
    w = {"vision_model.embeddings.class_embedding": r(1, 1, H), "vision_model.embeddings.position_embedding": r(1, 17, H),
         "vision_model.embeddings.patch_embedding.weight": r(H, 3, 14, 14, std=0.05), "vision_model.embeddings.patch_embedding.bias": r(H),
         "mlp1.0.weight": 1 + r(4 * H), "mlp1.0.bias": r(4 * H), "mlp1.1.weight": r(96, 4 * H), "mlp1.1.bias": r(96),
         "mlp1.3.weight": r(96, 96), "mlp1.3.bias": r(96)}
    for i in range(icfg.num_hidden_layers):
        p = f"vision_model.encoder.layers.{i}."
        w.update({p + "norm1.weight": 1 + r(H), p + "norm2.weight": 1 + r(H), p + "attn.qkv.weight": r(3 * H, H), p + "attn.qkv.bias": r(3 * H),
                  p + "attn.q_norm.weight": 1 + r(H), p + "attn.k_norm.weight": 1 + r(H), p + "attn.proj.weight": r(H, H),
                  p + "attn.proj.bias": r(H), p + "mlp.fc1.weight": r(128, H), p + "mlp.fc1.bias": r(128), p + "mlp.fc2.weight": r(H, 128),
                  p + "mlp.fc2.bias": r(H), p + "ls1": 0.5 + r(H), p + "ls2": 0.5 + r(H)})
    dist.broadcast_object_list(box := [w], src=0)   # the dict was drawn after rank-dependent work above: share rank 0's
    w = box[0]
    ipix = torch.randn(3, 3, 56, 56, generator=torch.Generator().manual_seed(9))
    compare("internvl", lambda grp: InternVLEncoder(icfg, group=grp), w, lambda m: m("image", None, {"pixel_values": [ipix[:1], ipix[1:]]}))


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    torch.set_num_threads(2)
    g = init_distributed(rank, world, master_port=port, backend="gloo", timeout_s=120, with_fabric=False)
    assert g.size == world and g.fabric is None
    for fn in (sp_dit, tp_vit, tp_encoder_families, tp_llm):
        fn(g)
        dist.barrier()
    if rank == 0:
        print("MULTIPROC_CPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
