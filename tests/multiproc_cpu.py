"""Two-rank (gloo, CPU) checks of the host-side parallel logic: weight sharding, head / token ownership, index tables
and the order of the collectives.  Launched by ``test_parallel_cpu.py`` once per rank; prints ``MULTIPROC_CPU_OK``."""

import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))

from cornserve_b200.parallel.state import init_distributed, single_group  # noqa: E402


def cos(a, b):
    return torch.nn.functional.cosine_similarity(a.float().flatten(), b.float().flatten(), dim=0).item()


def sp_dit(g):
    from test_geri_models import dit_weights

    from cornserve_b200.models.qwen_image import QwenImageDiT, QwenImageDiTConfig

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

    from cornserve_b200.executors.llm.engine import EngineConfig, LLMEngine, SamplingParams, Sequence
    from cornserve_b200.models.qwen_llm import LLMConfig, QwenLLM

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

    from cornserve_b200.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer

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


def main():
    rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
    torch.set_num_threads(2)
    g = init_distributed(rank, world, master_port=port, backend="gloo", timeout_s=120, with_fabric=False)
    assert g.size == world and g.fabric is None
    for fn in (sp_dit, tp_vit, tp_llm):
        fn(g)
        dist.barrier()
    if rank == 0:
        print("MULTIPROC_CPU_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
