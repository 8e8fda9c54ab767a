"""Times one kernel of the library on one shape (CUDA events, warm-up, L2 flushed between iterations).

  python -m cornserve.ops.microbench gemm 16384 3584 3584
  python -m cornserve.ops.microbench swiglu 19136 3424 1280
  python -m cornserve.ops.microbench skinny 64 3584 18944
  python -m cornserve.ops.microbench attn-window 4 [1]        # Qwen2.5-VL windows of 4 1280x720 images (1: packed tiles)
  python -m cornserve.ops.microbench attn-full 16 80 4784 0   # heads, head_dim, length, causal
  python -m cornserve.ops.microbench attn-decode 48 3500      # sequences, context
  python -m cornserve.ops.microbench norm 19136 1280
  python -m cornserve.ops.microbench adaln 8192 3072          # LayerNorm + AdaLN modulation (two samples)
  python -m cornserve.ops.microbench qk-norm-rope 8704 24     # per-head RMSNorm + rotation of q and k, d = 128
  python -m cornserve.ops.microbench sample 128 152064 50     # rows, vocabulary, top-k (temperature 1, top-p 0.9)
  python -m cornserve.ops.microbench gemm-fp8 16384 3584 3584 # e4m3 with 1x128 / 128x128 block scales
  python -m cornserve.ops.microbench moe 128 128 8 2048 768   # tokens, experts, top-k, hidden, expert FFN width
  python -m cornserve.ops.microbench push 8573952             # the sidecar's copy kernel, bytes
  python -m cornserve.ops.microbench tp-chain 19136 1280 3424 # fused TP half-block on one rank (loopback fabric)
  python -m cornserve.ops.microbench ulysses-qkv 4352 3072 24 # q|k|v GEMM with the all-to-all epilogue (loopback)

``--graph`` (gemm / skinny / swiglu) times the launches inside one CUDA graph over rotating weight copies, which is how
the decode path runs them; without it a kernel of a few microseconds is dominated by the host's launch path.

Each line printed gives the time per launch, the achieved rate and the fraction of the measured peak
(``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s and 1.59 PFLOP/s).  The same
commands, with ``--iters 1 --warmup 1``, are what the ncu summaries under ``profiles/`` were captured on.
"""

from __future__ import annotations

import argparse
import json
import math
from pathlib import Path

import numpy as np
import torch

from cornserve import ops


def peaks() -> tuple[float, float, str]:
    p = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]) * 1e9, float(d["bf16_tflops"]) * 1e12, "of measured"
    return 6.65e12, 1.59e15, "of fallback"


class Timer:
    def __init__(self, iters: int, warmup: int, flush: bool):
        self.iters, self.warmup = iters, warmup
        self.flush_buf = torch.empty(256 << 20, device="cuda", dtype=torch.uint8) if flush else None

    def __call__(self, fn) -> float:
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(self.iters):
            if self.flush_buf is not None:
                ops.l2_flush(self.flush_buf)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        ops.check_error("microbench")
        return total / self.iters * 1e-3


def graph_time(launch, weights: list[torch.Tensor], replays: int = 5) -> float:
    """Device time per launch with the host out of the picture: one CUDA graph of ``len(weights)`` launches, each on
    its own copy of the weight (together larger than L2, so every launch streams its weight from HBM as a decode step
    does), replayed ``replays`` times between two events."""
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for w in weights[:2]:
            launch(w)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for w in weights:
            launch(w)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    ops.check_error("microbench")
    return e0.elapsed_time(e1) * 1e-3 / (replays * len(weights))


def report(name: str, secs: float, flops: float = 0.0, nbytes: float = 0.0) -> None:
    bw, fl, tag = peaks()
    parts = [f"{name}: {secs * 1e6:.1f} us"]
    if flops:
        parts.append(f"{flops / secs / 1e12:.1f} TFLOP/s ({flops / secs / fl:.2f} {tag} bf16 burst)")
    if nbytes:
        parts.append(f"{nbytes / secs / 1e9:.0f} GB/s ({nbytes / secs / bw:.2f} {tag} copy bandwidth)")
    print("  ".join(parts), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel")
    ap.add_argument("args", nargs="*", type=int)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--splits", type=int, default=0, help="K splits of the weight-streaming kernel (0 = its own choice)")
    ap.add_argument("--graph", action="store_true",
                    help="gemm / skinny / swiglu: time inside a CUDA graph over rotating weight copies (no host time)")
    ap.add_argument("--cublas", action="store_true", help="with --graph: the same shape through torch's cuBLAS call")
    a = ap.parse_args()
    t = Timer(a.iters, a.warmup, not a.no_flush)
    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, std=1.0: (torch.randn(*s, device=dev, generator=g) * std).bfloat16()  # noqa: E731
    k = a.kernel
    if k in ("gemm", "swiglu", "skinny") and a.graph:
        M, N, K = a.args[:3]
        x = rnd(M, K)
        rows = 2 * N if k == "swiglu" else N
        copies = max(2, min(64, -(-(300 << 20) // (rows * K * 2))))
        weights = [rnd(rows, K, std=K ** -0.5) for _ in range(copies)]
        out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        if a.cublas:
            if k == "swiglu":
                def launch(w):
                    y = torch.nn.functional.linear(x, w)
                    torch.mul(torch.nn.functional.silu(y[:, :N]), y[:, N:], out=out)
            else:
                def launch(w):
                    torch.matmul(x, w.t(), out=out)
        elif k == "swiglu":
            def launch(w):
                ops.swiglu_linear(x, w, bn=a.bn, skinny=True if a.splits else None, splits=a.splits)
        else:
            def launch(w):
                ops.linear(x, w, out=out, bn=a.bn, skinny=(k == "skinny"), splits=a.splits)
        secs = graph_time(launch, weights)
        mult = 2.0 if k == "swiglu" else 1.0
        report(f"{'cublas ' if a.cublas else ''}{k} {M}x{N}x{K} (graph of {copies} launches, splits={a.splits}, bn={a.bn})", secs,
               2.0 * mult * M * N * K, 2.0 * (M * K + rows * K + M * N))
    elif k in ("gemm", "swiglu", "skinny"):
        M, N, K = a.args[:3]
        x = rnd(M, K)
        if k == "swiglu":
            w = rnd(2 * N, K, std=K ** -0.5)
            secs = t(lambda: ops.swiglu_linear(x, w, bn=a.bn, skinny=True if a.splits else None, splits=a.splits))
            report(f"swiglu {M}x{N}x{K}", secs, 4.0 * M * N * K, 2.0 * (M * K + 2 * N * K + M * N))
        else:
            w = rnd(N, K, std=K ** -0.5)
            out = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
            secs = t(lambda: ops.linear(x, w, out=out, bn=a.bn, skinny=(k == "skinny"), splits=a.splits))
            report(f"{k} {M}x{N}x{K}", secs, 2.0 * M * N * K, 2.0 * (M * K + N * K + M * N))
    elif k == "attn-window":
        from cornserve.models.qwen2_5_vl import pack_windows, window_index

        n = a.args[0] if a.args else 4
        packed = len(a.args) > 1 and a.args[1] == 1   # second argument 1: windows packed into shared 128-row tiles
        grid = np.array([[1, 52, 92]] * n)
        _, cu = window_index(grid, 112, 2, 14)
        bounds = None
        lens = np.diff(cu).astype(np.float64)
        if packed:
            cu, lo, hi = pack_windows(cu)
            bounds = (torch.from_numpy(lo).cuda(), torch.from_numpy(hi).cuda())
        T, H, d = 4784 * n, 16, 80
        qkv = rnd(T, 3 * H * d)
        q, kk, v = (qkv[:, i * H * d:(i + 1) * H * d].view(T, H, d) for i in range(3))
        cu_d = torch.from_numpy(cu).cuda()
        mx = int(np.diff(cu).max())
        secs = t(lambda: ops.attention_varlen(q, kk, v, cu_d, cu_d, mx, row_bounds=bounds))
        report(f"attn-window {n} images ({len(lens)} windows{', packed' if packed else ''})", secs, 4.0 * H * d * float((lens ** 2).sum()),
               2.0 * 4 * T * H * d)
    elif k == "attn-full":
        H, d, L, causal = (a.args + [16, 80, 4784, 0][len(a.args):])[:4]
        q, kk, v = rnd(L, H, d), rnd(L, H, d), rnd(L, H, d)
        cu = torch.tensor([0, L], device=dev, dtype=torch.int32)
        secs = t(lambda: ops.attention_varlen(q, kk, v, cu, cu, L, causal=bool(causal)))
        report(f"attn-full H={H} d={d} L={L} causal={causal}", secs, 4.0 * H * d * L * L * (0.5 if causal else 1.0))
    elif k == "attn-decode":
        B, ctx = (a.args + [48, 3500][len(a.args):])[:2]
        Hq, Hkv, d = 28, 4, 128
        blocks = -(-ctx // 128)
        cache = rnd(B * blocks, 2, Hkv, 128, d)
        bt = torch.arange(B * blocks, device=dev, dtype=torch.int32).view(B, blocks)
        kv_len = torch.full((B,), ctx, device=dev, dtype=torch.int32)
        cu = torch.arange(B + 1, device=dev, dtype=torch.int32)
        q = rnd(B, Hq, d)
        secs = t(lambda: ops.attention_paged(q, cache, bt, kv_len, cu, 1, causal=True, pack_gqa=True))
        report(f"attn-decode B={B} ctx={ctx}", secs, 4.0 * B * Hq * d * ctx, 2.0 * 2 * B * Hkv * ctx * d)
    elif k == "norm":
        rows, H = a.args[:2]
        x, r, w = rnd(rows, H), rnd(rows, H), rnd(H)
        secs = t(lambda: ops.rms_norm(x, w, 1e-6, residual=r))
        report(f"rms_norm+residual {rows}x{H}", secs, 0.0, 2.0 * 4 * rows * H)
    elif k == "adaln":
        rows, H = a.args[:2]
        x, mod = rnd(rows, H), rnd(2, 2 * H, std=0.1)
        secs = t(lambda: ops.layer_norm(x, None, None, 1e-6, scale=mod[:, :H], shift=mod[:, H:], rows_per_batch=rows // 2))
        report(f"modulated layer_norm {rows}x{H}", secs, 0.0, 2.0 * 2 * rows * H)
    elif k == "qk-norm-rope":
        T, heads = a.args[:2]
        d = 128
        qkv, ws = rnd(T, 3 * heads * d), [rnd(d) for _ in range(4)]
        cs = torch.randn(T, 2, d // 2, device=dev, generator=g)
        secs = t(lambda: ops.qk_norm_rope_(qkv, heads, d, heads * d, ws[0], ws[1], 1e-6, cs, wq2=ws[2], wk2=ws[3],
                                           seg=T // 2, n_first=T // 34))
        report(f"q/k head norm + rotation {T} tokens x {heads} heads", secs, 0.0, 2.0 * 2 * 2 * T * heads * d + 4.0 * T * d)
    elif k == "sample":
        rows, V = (a.args + [128, 152064][len(a.args):])[:2]
        top_k = a.args[2] if len(a.args) > 2 else 0
        logits = torch.randn(rows, V, device=dev, generator=g) * 3
        f = lambda v, dt: torch.full((rows,), v, device=dev, dtype=dt)  # noqa: E731
        args = (f(1.0, torch.float32), f(0.9, torch.float32), f(top_k, torch.int32),
                torch.arange(rows, device=dev, dtype=torch.int64), torch.zeros(rows, device=dev, dtype=torch.int32))
        secs = t(lambda: ops.sample_rows(logits, *args))
        report(f"sample (temperature 1, top_p 0.9, top_k {top_k}) {rows}x{V}", secs, 0.0, 4.0 * rows * V)
        secs = t(lambda: ops.argmax(logits))
        report(f"argmax {rows}x{V}", secs, 0.0, 4.0 * rows * V)
    elif k == "gemm-fp8":
        M, N, K = a.args[:3]
        x = rnd(M, K)
        wq, ws = ops.quantize_fp8_weight(rnd(N, K, std=K ** -0.5))
        xq = ops.quantize_fp8_rows(x)
        secs = t(lambda: ops.linear_fp8(x, wq, ws, xq=xq))
        report(f"gemm-fp8 {M}x{N}x{K} (operands already quantised)", secs, 2.0 * M * N * K, 1.0 * (M * K + N * K) + 2.0 * M * N)
        secs = t(lambda: ops.quantize_fp8_rows(x))
        report(f"quantise rows {M}x{K}", secs, 0.0, 3.0 * M * K)
    elif k == "moe":
        from cornserve.parallel.moe import FusedMoE
        from cornserve.parallel.state import single_group

        T, E, kk, H, I = (a.args + [128, 128, 8, 2048, 768][len(a.args):])[:5]
        layer = FusedMoE(single_group(dev), E, kk, H, I, max(T, 1024))
        x, logits = rnd(T, H), torch.randn(T, E, device=dev, generator=g)
        wgu, wd = rnd(E, 2 * I, H, std=H ** -0.5), rnd(E, H, I, std=I ** -0.5)
        secs = t(lambda: layer.forward(x, logits, wgu, wd))
        touched = min(E, T * kk)  # experts whose weights must be read (upper bound when tokens collide)
        report(f"moe layer T={T} E={E} top{kk} H={H} I={I} (row tile {layer.tile_rows_for(T)})", secs, 6.0 * T * kk * H * I,
               2.0 * (touched * 3 * H * I + 2 * T * kk * (H + I) + 2 * T * H))
    elif k == "push":
        nbytes = (a.args[0] if a.args else 1196 * 3584 * 2)
        src = torch.randint(0, 255, (nbytes,), device=dev, dtype=torch.uint8)
        dst = torch.empty_like(src)
        secs = t(lambda: ops.push_bytes_(dst, src))
        report(f"sidecar push kernel {nbytes} bytes (same GPU)", secs, 0.0, 2.0 * nbytes)
    elif k == "tp-chain":
        # the tensor-parallel MLP half-block (norm -> all-gather -> gate/up GEMM -> down GEMM -> reduce-scatter ->
        # residual + norm) with one rank: every push, counter and wait of the fused kernels runs, against this GPU's memory
        from cornserve.parallel.fabric import Fabric
        from cornserve.parallel.fused import FusedEncoderTP

        S, H, I = (a.args + [19136, 1280, 3424][len(a.args):])[:3]
        fab = Fabric.loopback(dev)
        tp = FusedEncoderTP(fab.group, H, S)
        xs, nw = rnd(S, H), rnd(H)
        wgu, wdn = rnd(2 * I, H, std=H ** -0.5), rnd(H, I, std=I ** -0.5)
        state = {}

        def stage(name):
            def run():
                tp.begin(S)
                if name in ("all", "norm+push"):
                    tp.reduce_norm_push(bias=None, residual=xs, dst=1, reduce=False, norm_w=nw, eps=1e-6)
                if name in ("all", "gathered gemm"):
                    state["h"] = tp.gemm_gathered(1, wgu, None, act="silu", swiglu=True)
                if name in ("all", "push gemm"):
                    tp.gemm_push(state["h"], wdn)
                if name in ("all", "reduce+norm+push"):
                    tp.reduce_norm_push(bias=None, residual=xs, dst=0, norm_w=nw, eps=1e-6)
            return run

        stage("all")()
        torch.cuda.synchronize()
        report(f"tp-chain (one rank, loopback) S={S} H={H} I={I}: whole half-block", t(stage("all")), 6.0 * S * H * I,
               2.0 * (3 * I * H + 6 * S * H + 2 * S * I))
        # a stage alone starts a pass with fresh counters, so its waits pass at once: this is its own time
        report("  norm + push (all-gather store)", t(stage("norm+push")), 0.0, 2.0 * 2 * S * H)
        report("  gate/up GEMM on the gathered operand (SwiGLU epilogue)", t(stage("gathered gemm")), 4.0 * S * H * I)
        report("  down GEMM with the reduce-scatter in its epilogue", t(stage("push gemm")), 2.0 * S * H * I)
        report("  reduce + residual + norm + push", t(stage("reduce+norm+push")), 0.0, 2.0 * 4 * S * H)
    elif k == "ulysses-qkv":
        from cornserve.parallel.fabric import Fabric
        from cornserve.parallel.fused import FusedUlysses

        rows, D, heads = (a.args + [4352, 3072, 24][len(a.args):])[:3]
        fab = Fabric.loopback(dev)
        fu = FusedUlysses(fab.group, D, heads, D // heads, rows)
        x, w, b = rnd(rows, D), rnd(3 * D, D, std=D ** -0.5), rnd(3 * D)
        secs = t(lambda: fu.qkv_scatter(x, w, b, 0, rows, rows, rows))
        report(f"ulysses q|k|v projection with the all-to-all in its epilogue (one rank, loopback) {rows}x{3 * D}x{D}", secs,
               6.0 * rows * D * D, 2.0 * (rows * D + 3 * D * D + 3 * rows * D))
    else:
        raise SystemExit(f"unknown kernel {k}")


if __name__ == "__main__":
    main()
