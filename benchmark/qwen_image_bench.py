"""Qwen-Image text-to-image throughput (images/s) on N GPUs of one node, the second headline workload.

Full-size architecture with random-init weights and synthetic conditioning: MMDiT with 60 dual-stream blocks (hidden
3072, 24 heads of 128), 1024 x 1024 output (4096 image tokens) plus 256 text tokens, 50 flow-matching steps with
classifier-free guidance (two denoiser passes per step), 16-channel VAE decode to RGB8.  With N > 1 the denoiser runs
Ulysses sequence parallel over all ranks (token shards outside attention, head shards inside), the exchanges done by the
GEMM epilogues and peer-store kernels of this library (``--library-a2a`` switches to the NCCL all-to-all twin).

    python -m benchmark.qwen_image_bench --images 2 --warmup 1
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m benchmark.qwen_image_bench --images 2

Timed on the device (CUDA events on the launching stream, barrier + synchronize on both sides, maximum over ranks); rank
0 prints one JSON line.
"""

from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv: list[str] | None = None) -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--images", type=int, default=2, help="timed images (one at a time, batch 1)")
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--size", type=int, default=1024)
    ap.add_argument("--text-tokens", type=int, default=256)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-cfg", action="store_true")
    ap.add_argument("--library-a2a", action="store_true")
    ap.add_argument("--tiny", action="store_true", help="small architecture (CPU smoke run)")
    a = ap.parse_args(argv)

    from cornserve import ops
    from cornserve.models.qwen_image import QwenImageDiTConfig, QwenImageModel, QwenImagePipelineConfig
    from cornserve.models.qwen_image_vae import QwenImageVAEConfig
    from cornserve.parallel.state import init_distributed, single_group

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    cuda = torch.cuda.is_available()
    if world > 1:
        group = init_distributed(rank, world, master_addr=os.environ.get("MASTER_ADDR", "127.0.0.1"),
                                 master_port=int(os.environ.get("MASTER_PORT", "29500")),
                                 local_device=int(os.environ.get("LOCAL_RANK", rank)) if cuda else None)
    else:
        if cuda:
            torch.cuda.set_device(0)
        group = single_group("cuda:0" if cuda else "cpu")
    dev = group.device
    if a.tiny:
        cfg = QwenImagePipelineConfig(dit=QwenImageDiTConfig(in_channels=64, out_channels=16, num_layers=2, attention_head_dim=64,
                                                             num_attention_heads=4, joint_attention_dim=128, axes_dims_rope=(8, 28, 28)),
                                      vae=QwenImageVAEConfig(base_dim=16, z_dim=16, dim_mult=[1, 2, 4, 4], num_res_blocks=1))
    else:
        cfg = QwenImagePipelineConfig()
    torch.manual_seed(0)
    model = QwenImageModel(cfg, group=group, device=dev)
    if not cuda:
        model.dit.float()
        model.vae.float()
    model.dit.fused_exchange = not a.library_a2a
    gen = torch.Generator().manual_seed(1)
    emb = [torch.randn(a.text_tokens, model.embedding_dim, generator=gen).to(model.dtype) for _ in range(a.batch)]
    neg = None if a.no_cfg else [torch.randn(a.text_tokens, model.embedding_dim, generator=gen).to(model.dtype) for _ in range(a.batch)]

    def one():
        return model.generate_rgb(emb, a.size, a.size, a.steps, negative_embeds=neg)

    def fence():
        if cuda:
            torch.cuda.synchronize()
        if world > 1:
            dist.barrier()

    for _ in range(a.warmup):
        one()
    fence()
    launches0 = ops.kernel_launches()
    if cuda:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
    import time

    t0 = time.perf_counter()
    for _ in range(a.images):
        img = one()
    if cuda:
        e1.record()
    fence()
    secs = (e0.elapsed_time(e1) / 1e3) if cuda else (time.perf_counter() - t0)
    if cuda:
        ops.check_error("qwen-image bench")
    t = torch.tensor([secs], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        d = cfg.dit
        print(json.dumps({
            "metric": "images_per_second", "value": a.images * a.batch / t.item(), "unit": "img/s", "n_gpus": world,
            "seconds_per_image": t.item() / (a.images * a.batch), "images": a.images, "warmup": a.warmup, "dtype": "bf16" if cuda else "fp32",
            "data": "synthetic (random conditioning, random-init weights)",
            "config": {"model": "Qwen-Image" if not a.tiny else "tiny", "blocks": d.num_layers, "hidden": d.inner_dim, "size": a.size,
                       "text_tokens": a.text_tokens, "steps": a.steps, "cfg": not a.no_cfg, "batch": a.batch,
                       "parallelism": f"ulysses sp{world}" + (" (NCCL all-to-all)" if a.library_a2a and world > 1 else ""),
                       "output": list(img.shape)},
            "gpu_launches": (ops.kernel_launches() - launches0) * world}))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
