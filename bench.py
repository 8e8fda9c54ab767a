#!/usr/bin/env python
"""Headline benchmark: Qwen2.5-VL-7B multimodal-LLM serving throughput (requests/s).

One *step* serves a fixed batch of synthetic requests to completion on every GPU: each request has
1-4 uniform-random 1280x720 RGB images, 128 random prompt tokens and 256 greedy output tokens
(``ignore_eos``).  The step runs image preprocessing, the 32-layer vision tower, chunked prefill and
256 decode steps of the 28-layer LLM with this repository's kernels (bf16, random-init weights of the
real architecture, synthetic data).

  python bench.py --gpus N --steps K --warmup W          # N > 1: launched with torch.distributed.run
  python bench.py --impl reference ...                   # reference arm: prints why it cannot run here

Rank 0 prints one JSON line.  ``value`` is timed on the device (CUDA events, max over ranks) with the
inputs already resident; ``e2e.value`` is the same work through ``MLLMPipeline.generate`` with the
images copied from pinned host memory every step and the generated tokens read back.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

METRIC = "requests_per_second"
MODEL = "Qwen2.5-VL-7B"
REF_UNAVAILABLE = (
    "the reference's LLM executor is an empty git submodule (third_party/vllm) and its request path needs "
    "Kubernetes pods; only its Eric encoder modules import offline, so the MLLM request metric cannot be "
    "produced by unmodified reference code (the encoder module alone is timed by python -m benchmark.encoder_compare)"
)


def parse_args() -> argparse.Namespace:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--requests-per-gpu", type=int, default=128)
    ap.add_argument("--output-tokens", type=int, default=256)
    ap.add_argument("--prompt-tokens", type=int, default=128)
    ap.add_argument("--prefill-tokens", type=int, default=18944, help="token budget of one prefill step (148 SMs x 128 rows)")
    ap.add_argument("--vit-patches", type=int, default=34000, help="patch budget of one vision-tower call (7 images of 1280x720)")
    ap.add_argument("--small", action="store_true", help="tiny model/config for smoke runs (not a valid number)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200"], stdout=f, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, gpu_index: int = 0) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                p = [x.strip() for x in line.split(",")]
                if len(p) < 9 or not p[0].isdigit() or int(p[0]) != gpu_index:
                    continue
                sm.append(float(p[1])); mx.append(float(p[2]))
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        # samples under load = upper half of the clock readings taken while kernels ran
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def main() -> None:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": REF_UNAVAILABLE}))
        return

    import numpy as np
    import torch
    import torch.distributed as dist

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from cornserve import ops
    from cornserve.task_executors.llm.engine import EngineConfig
    from cornserve.models.qwen2_5_vl import Qwen25VisionConfig, Qwen25VisionTransformer
    from cornserve.models.qwen_llm import LLMConfig, QwenLLM
    from cornserve.pipelines import MLLMPipeline, MLLMRequest

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    R, out_tok, prompt_tok = args.requests_per_gpu, args.output_tokens, args.prompt_tokens
    if args.small:
        vcfg = Qwen25VisionConfig(depth=2, hidden_size=256, num_heads=4, intermediate_size=512, out_hidden_size=512,
                                  fullatt_block_indexes=[1])
        lcfg = LLMConfig(hidden_size=512, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         head_dim=128, intermediate_size=1024, vocab_size=152064)
        img_hw = (224, 224)
    else:
        vcfg = Qwen25VisionConfig()  # 32 layers, hidden 1280, 16 heads, window attention, merger -> 3584
        lcfg = LLMConfig()           # 28 layers, hidden 3584, 28/4 heads, MLP 18944, vocab 152064, M-RoPE
        img_hw = (720, 1280)
    torch.manual_seed(1234 + rank)
    vision = Qwen25VisionTransformer(vcfg, device=dev)
    llm = QwenLLM(lcfg, device=dev)
    tokens_per_img = 1196 if not args.small else 64
    pages = R * (-(-(4 * (tokens_per_img + 2) + prompt_tok + out_tok + 2) // 128) + 1) + 8
    # 148 SMs x 128-row tiles: with 18944 tokens per prefill step every GEMM of the decoder has a whole number of tile
    # waves (14, 18 and 74 column tiles per row tile); 7 images of 4784 patches do the same for the vision tower
    # (262 row tiles x 5 / 14 / 15 column tiles = 8.85 / 24.8 / 26.6 waves, against 10.1 / 28.3 / 30.3 for 8 images)
    pipe = MLLMPipeline(vision, llm, EngineConfig(num_pages=pages, max_batched_tokens=args.prefill_tokens,
                                                  max_num_seqs=max(R, 1), decode_burst=16, max_model_len=8192),
                        max_patches_per_encode=args.vit_patches)

    rng = np.random.default_rng(rank)
    n_imgs = [1 + (i % 4) for i in range(R)]
    host_imgs = [[torch.from_numpy(rng.integers(0, 256, (*img_hw, 3), dtype=np.uint8)).pin_memory()
                  for _ in range(n)] for n in n_imgs]
    dev_imgs = [[im.to(dev) for im in ims] for ims in host_imgs]
    prompts = [rng.integers(1000, 100000, prompt_tok).astype(np.int32) for _ in range(R)]

    def make_requests(images, step):
        return [MLLMRequest(f"r{step}-{i}", prompts[i], images[i], max_tokens=out_tok, ignore_eos=True)
                for i in range(R)]

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def run_steps(images, n, tag):
        for s in range(n):
            res = pipe.generate(make_requests(images, f"{tag}{s}"))
            assert all(len(v) == out_tok for v in res.values())

    # ---- device-timed arm (inputs resident on the GPU) ------------------------------------------------
    run_steps(dev_imgs, args.warmup, "w")
    ops.check_error("warm-up")
    sampler = ClockSampler()
    barrier()
    if rank == 0:
        sampler.start()
    ops.reset_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    run_steps(dev_imgs, args.steps, "t")
    e1.record()
    barrier()
    clocks = sampler.stop(local_rank) if rank == 0 else {}
    launches = ops.kernel_launches()
    dev_ms = e0.elapsed_time(e1)
    ops.check_error("timed region")

    # ---- end-to-end arm (pinned host inputs copied every step, tokens read back) ---------------------------
    run_steps(host_imgs, 1, "ew")
    pipe.h2d_bytes = pipe.d2h_bytes = 0
    barrier()
    t0 = time.perf_counter()
    run_steps(host_imgs, args.steps, "e")
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    ops.check_error("e2e region")

    times = torch.tensor([dev_ms, e2e_s * 1000.0], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = times.tolist()
    if rank == 0:
        total_req = R * world * args.steps
        avg_prompt = int(sum(n * (tokens_per_img + 2) for n in n_imgs) / R + prompt_tok)
        line = {
            "metric": METRIC, "value": total_req / (dev_ms / 1e3), "unit": "req/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic (uniform-random images and token ids, random-init weights)",
            "config": {
                "model": MODEL if not args.small else "tiny-smoke", "global_batch": R * world,
                "seq_len": avg_prompt + out_tok, "parallelism": f"dp{world} (one monolithic encoder+LLM replica per GPU)",
                "images_per_request": "1-4 (mean 2.5) of 1280x720", "prompt_tokens": prompt_tok,
                "output_tokens": out_tok, "requests_per_gpu_per_step": R,
                "l2_policy": "inputs larger than L2: every step streams 16.6 GB of weights plus the KV cache",
            },
            "clocks": clocks,
            "e2e": {"value": total_req / (e2e_ms / 1e3), "unit": "req/s", "ms_per_step": e2e_ms / args.steps,
                    # whole job, like `value`: every rank copies its own batch (the ranks' batches have the same shape)
                    "h2d_bytes_per_step": world * pipe.h2d_bytes // args.steps,
                    "d2h_bytes_per_step": world * pipe.d2h_bytes // args.steps,
                    "api": "cornserve.pipelines.MLLMPipeline.generate"},
            "gpu_launches": launches * world,
            "output_tokens_per_second": total_req * out_tok / (dev_ms / 1e3),
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
