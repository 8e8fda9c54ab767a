"""The fused compute + collective kernels on ONE GPU: with a one-rank loopback fabric every push, arrival counter and
wait of the tensor-parallel chain and of the Ulysses projection runs against the GPU's own memory, so their code path
and numerics are checked (against fp32 restatements) without a second GPU."""

import pytest
import torch

from cornserve import ops

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).bfloat16()


def _rms(x, w, eps=1e-6):
    x = x.float()
    return (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float())


@pytest.mark.parametrize("S,H,I", [(700, 1280, 1712), (384, 3584, 1024), (130, 2048, 256)])
def test_tensor_parallel_half_block_chain_in_loopback(S, H, I):
    """norm -> (all-gather store) -> gate/up GEMM with SwiGLU -> down GEMM (reduce-scatter store) -> reduce + residual +
    norm, twice in a row (the second pass uses the other set of counters)."""
    from cornserve.parallel.fabric import Fabric
    from cornserve.parallel.fused import FusedEncoderTP

    torch.manual_seed(S)
    tp = FusedEncoderTP(Fabric.loopback(DEV).group, H, S)
    nw1, nw2 = 1 + _rand(H, scale=0.1), 1 + _rand(H, scale=0.1)
    wgu, wdn, bias = _rand(2 * I, H, scale=H ** -0.5), _rand(H, I, scale=I ** -0.5), _rand(H, scale=0.1)
    for attempt in range(2):
        xs = _rand(S, H)
        tp.begin(S)
        tp.reduce_norm_push(bias=None, residual=xs, dst=1, reduce=False, norm_w=nw1, eps=1e-6)
        h = tp.gemm_gathered(1, wgu, None, act="silu", swiglu=True)
        tp.gemm_push(h, wdn)
        x_new = tp.reduce_norm_push(bias=bias, residual=xs, dst=0, norm_w=nw2, eps=1e-6)
        torch.cuda.synchronize()
        ops.check_error(f"chain pass {attempt}")
        xn = _rms(xs, nw1).bfloat16().float()
        gu = xn @ wgu.float().t()
        hh = (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]).bfloat16().float()
        want = (hh @ wdn.float().t()).bfloat16().float() + bias.float() + xs.float()
        err = (x_new.float() - want).abs().max().item()
        assert err < 0.08 and torch.nn.functional.cosine_similarity(x_new.float().flatten(), want.flatten(), dim=0) > 0.999, err
        got_norm = tp.gather[0].local[: S * H].view(S, H).float()
        want_norm = _rms(x_new, nw2)
        assert (got_norm - want_norm).abs().max().item() < 0.06


def test_ulysses_projection_epilogue_in_loopback():
    """The q|k|v projection whose epilogue is the tokens -> heads all-to-all: with one rank every head tile lands in
    this GPU's own buffer, in the order (sample, rank, row in segment)."""
    from cornserve.parallel.fabric import Fabric
    from cornserve.parallel.fused import FusedUlysses

    torch.manual_seed(1)
    rows, D, heads = 520, 1024, 8
    fu = FusedUlysses(Fabric.loopback(DEV).group, D, heads, D // heads, rows)
    x, w, b = _rand(rows, D), _rand(3 * D, D, scale=D ** -0.5), _rand(3 * D, scale=0.1)
    fu.begin_pass()
    fu.qkv_scatter(x, w, b, 0, rows, rows, rows)
    got = fu.gathered_qkv(rows)
    torch.cuda.synchronize()
    ops.check_error("ulysses loopback")
    want = x.float() @ w.float().t() + b.float()
    assert got.shape == (rows, 3 * D)
    assert (got.float() - want).abs().max().item() < 0.08
    o = _rand(rows, D)
    back = fu.push_heads(o, rows)
    torch.cuda.synchronize()
    ops.check_error("ulysses return")
    assert torch.equal(back, o)
