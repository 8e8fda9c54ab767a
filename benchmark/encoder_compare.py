"""Encoder forward pass: this package's Qwen2.5-VL vision tower against the reference's own module on one GPU.

    python -m benchmark.encoder_compare --images 7 --iters 5
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 -m benchmark.encoder_compare   # both at TP=2

The reference's LLM executor and control plane cannot run offline, but its encoder executor's model code can: when the
reference package is installed under ``baseline/_ref`` its ``Qwen2_5_VisionTransformer`` (reference:
python/cornserve/task_executors/eric/models/qwen2_5_vl.py:262-486; torch ``Linear`` on cuBLAS, flash-attn var-len
attention, eager norms and rotary) is built unmodified with random bf16 weights of the 7B tower (32 layers, hidden 1280,
16 heads, window attention with full attention at layers 7 / 15 / 23 / 31, 2x2 merger to 3584) and run through its own
``forward`` on the same synthetic batch of 1280x720 images as this package's tower.  Both are timed with CUDA events
after warm-up; one JSON line reports images per second of each and the ratio.  Under ``torchrun`` both towers are
tensor parallel over all ranks: the reference with its own column / row parallel layers over NCCL, this package with the
exchanges inside its GEMM and norm kernels over peer memory; times are the maximum over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import numpy as np
import torch

VISION_7B = dict(depth=32, hidden_size=1280, num_heads=16, intermediate_size=3420, out_hidden_size=3584,
                 fullatt_block_indexes=[7, 15, 23, 31], window_size=112, patch_size=14, spatial_merge_size=2,
                 temporal_patch_size=2, hidden_act="silu", in_channels=3)
# Qwen2-VL-7B tower: LayerNorm, quick-GELU MLP of ratio 4, full attention in every layer
VISION_QWEN2 = dict(depth=32, embed_dim=1280, hidden_size=3584, num_heads=16, mlp_ratio=4, in_channels=3, in_chans=3,
                    patch_size=14, spatial_merge_size=2, temporal_patch_size=2, hidden_act="quick_gelu")


def _time(fn, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters / 1e3


def _max_over_ranks(seconds: float, world: int) -> float:
    if world == 1:
        return seconds
    import torch.distributed as dist

    t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_ours(model: str, pixels: list[torch.Tensor], grids: list[list[int]], iters: int, warmup: int, rank: int, world: int) -> float:
    from cornserve import ops
    from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer
    from cornserve.parallel.state import init_distributed

    group = init_distributed(rank, world, master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"),
                             master_port=int(os.environ.get("MASTER_PORT", "29511")), local_device=int(os.environ.get("LOCAL_RANK", rank)))
    torch.manual_seed(0)
    if model == "qwen2_vl":
        from cornserve.models.qwen2_vl import Qwen2VisionConfig, Qwen2VisionTransformer

        tower = Qwen2VisionTransformer(Qwen2VisionConfig(), group=group, device=group.device)
    else:
        tower = Qwen25VisionTransformer(Qwen25VisionConfig(), group=group, device=group.device)
    pv, grid = torch.cat(pixels), np.asarray(grids)
    with torch.inference_mode():
        secs = _time(lambda: tower.encode(pv, grid), iters, warmup)
    ops.check_error("encoder_compare")
    return _max_over_ranks(secs, world)


def time_reference(model: str, pixels: list[torch.Tensor], grids: list[list[int]], iters: int, warmup: int, rank: int, world: int) -> float | str:
    """Runs in a process of its own whose import path holds the reference package and not this repository (both are
    called ``cornserve``); see :func:`reference_in_subprocess`."""
    try:
        from cornserve.task_executors.eric.distributed import parallel

        if model == "qwen2_vl":
            from cornserve.task_executors.eric.models import qwen2_vl as ref_mod
            from transformers.models.qwen2_vl.configuration_qwen2_vl import Qwen2VLConfig

            build = lambda: ref_mod.Qwen2VisionTransformer(Qwen2VLConfig(vision_config=VISION_QWEN2))  # noqa: E731
        else:
            from cornserve.task_executors.eric.models import qwen2_5_vl as ref_mod
            from transformers.models.qwen2_5_vl.configuration_qwen2_5_vl import Qwen2_5_VLConfig

            build = lambda: ref_mod.Qwen2_5_VisionTransformer(Qwen2_5_VLConfig(vision_config=VISION_7B))  # noqa: E731
        Modality = ref_mod.Modality
    except Exception as e:  # noqa: BLE001
        return f"the reference encoder does not import here: {type(e).__name__}: {e}"
    parallel.init_distributed(world_size=world, rank=rank, init_method=f"tcp://{os.environ.get('MASTER_ADDR', '127.0.0.1')}:"
                                                                       f"{int(os.environ.get('MASTER_PORT', '29511')) + 7}")
    torch.manual_seed(0)
    tower = build().to(device="cuda", dtype=torch.bfloat16).eval()
    batch = {"pixel_values": pixels, "image_grid_thw": [torch.tensor([g]) for g in grids]}
    with torch.inference_mode():
        secs = _time(lambda: tower(Modality.IMAGE, "", batch), iters, warmup)
    return _max_over_ranks(secs, world)


def reference_in_subprocess(a: argparse.Namespace) -> float | str:
    """The reference arm, one child process per rank: started with ``-P`` and a ``PYTHONPATH`` that holds
    ``baseline/_ref`` (the unmodified reference) and not this repository."""
    import subprocess

    repo = Path(__file__).resolve().parents[1]
    root = repo / "baseline" / "_ref"
    if not (root / "cornserve").is_dir():
        return "the reference package is not installed under baseline/_ref"
    keep = [p for p in os.environ.get("PYTHONPATH", "").split(os.pathsep) if p and Path(p).resolve() != repo]
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([str(root), *keep]))
    r = subprocess.run([sys.executable, "-P", str(Path(__file__).resolve()), "--arm", "reference", "--model", a.model, "--images", str(a.images),
                        "--iters", str(a.iters), "--warmup", str(a.warmup)], env=env, cwd="/", capture_output=True, text=True, timeout=900)
    if r.returncode != 0:
        return f"the reference arm failed: {r.stderr.strip().splitlines()[-1] if r.stderr.strip() else r.returncode}"
    out = json.loads(r.stdout.strip().splitlines()[-1])
    return out.get("unavailable") or float(out["seconds_per_pass"])


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="qwen2_5_vl", choices=["qwen2_5_vl", "qwen2_vl"], help="which 7B vision tower")
    ap.add_argument("--images", type=int, default=7, help="1280x720 images per forward pass")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--arm", default="both", choices=["both", "reference"], help="reference: only that arm, for the child process")
    a = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("encoder_compare needs a CUDA device")
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    gen = torch.Generator(device="cuda").manual_seed(1)
    grid = [1, 52, 92]   # 1280x720 -> 728 x 1288 after rounding to 28-pixel cells: 52 x 92 patches
    pixels = [torch.randn(grid[1] * grid[2], 3 * 2 * 14 * 14, device="cuda", generator=gen).bfloat16() for _ in range(a.images)]
    grids = [grid] * a.images
    if a.arm == "reference":
        ref = time_reference(a.model, pixels, grids, a.iters, a.warmup, rank, world)
        print(json.dumps({"unavailable": ref} if isinstance(ref, str) else {"seconds_per_pass": ref}))
        return
    ref = reference_in_subprocess(a)   # first, and finished before this package touches the GPU
    ours = time_ours(a.model, pixels, grids, a.iters, a.warmup, rank, world)
    out = {"metric": "encoder_images_per_second", "model": a.model, "n_gpus": world, "parallelism": f"tp{world}", "dtype": "bf16",
           "images_per_pass": a.images, "data": "synthetic (random patches, random-init weights)",
           "ours": {"seconds_per_pass": ours, "images_per_second": a.images / ours}}
    if isinstance(ref, str):
        out["reference"] = {"unavailable": ref}
    else:
        out["reference"] = {"seconds_per_pass": ref, "images_per_second": a.images / ref}
        out["ours_over_reference"] = ref / ours
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
