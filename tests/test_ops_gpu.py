"""Numerics of the sm_100a kernels against the fp32 PyTorch restatements (GPU only)."""

import math

import pytest
import torch

from cornserve import ops
from cornserve.ops import reference as ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0, dtype=torch.bfloat16):
    return (torch.randn(*shape, device=DEV, dtype=torch.float32) * scale).to(dtype)


def _close(a, b, atol, rtol, name=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    bad = (err > tol).float().mean().item()
    cos = torch.nn.functional.cosine_similarity(a.flatten(), b.flatten(), dim=0).item()
    assert bad < 1e-3 and cos > 0.999, f"{name}: max err {err.max().item():.4g}, frac bad {bad:.4g}, cos {cos:.6f}"


@pytest.fixture(autouse=True)
def _no_kernel_error():
    yield
    torch.cuda.synchronize()
    ops.check_error("after test")


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 256), (300, 200, 136), (4784, 3840, 1280),
                                   (1000, 1280, 1712), (8, 4608, 3584), (64, 3584, 18944)])
@pytest.mark.parametrize("bn", [0, 32, 64, 128, 256])
def test_gemm_plain(M, N, K, bn):
    torch.manual_seed(0)
    x, w = _rand(M, K), _rand(N, K, scale=K ** -0.5)
    y = ops.linear(x, w, bn=bn)
    _close(y, ref.linear(x, w, out_dtype=torch.float32), 2e-2, 2e-2, f"gemm {M}x{N}x{K} bn={bn}")


@pytest.mark.parametrize("act", ["none", "gelu", "gelu_tanh", "silu", "quick_gelu"])
def test_gemm_epilogues(act):
    torch.manual_seed(1)
    M, N, K = 515, 1280, 320
    x, w, b, r = _rand(M, K), _rand(N, K, scale=K ** -0.5), _rand(N), _rand(M, N)
    y = ops.linear(x, w, b, act=act, residual=r)
    _close(y, ref.linear(x, w, b, act, r, out_dtype=torch.float32), 3e-2, 2e-2, f"epilogue {act}")
    g = _rand(5, N)
    y = ops.linear(x, w, b, act=act, residual=r, gate=g, gate_rows_per_batch=103)
    _close(y, ref.linear(x, w, b, act, r, g, 103, out_dtype=torch.float32), 3e-2, 2e-2, f"gated {act}")
    y32 = ops.linear(x, w, b, out_dtype=torch.float32)
    assert y32.dtype == torch.float32
    _close(y32, ref.linear(x, w, b, out_dtype=torch.float32), 1e-2, 1e-2, "fp32 out")


@pytest.mark.parametrize("M,I,K,bn", [(700, 1712, 1280, 0), (64, 512, 256, 128), (4784, 3424, 1280, 256), (9, 96, 64, 64)])
def test_gemm_swiglu(M, I, K, bn):
    torch.manual_seed(2)
    x, w, b = _rand(M, K), _rand(2 * I, K, scale=K ** -0.5), _rand(2 * I, scale=0.1)
    y = ops.swiglu_linear(x, w, b, bn=bn)
    _close(y, ref.swiglu_linear(x.float(), w.float(), b.float()), 3e-2, 2e-2, "swiglu")


@pytest.mark.parametrize("H", [1280, 3584, 5120, 128])
def test_norms(H):
    torch.manual_seed(3)
    x, r, w, b = _rand(77, H), _rand(77, H), _rand(H), _rand(H)
    _close(ops.rms_norm(x, w, 1e-6), ref.rms_norm(x.float(), w, 1e-6), 2e-2, 1e-2, "rms")
    y, nr = ops.rms_norm(x, w, 1e-6, residual=r)
    y0, nr0 = ref.rms_norm(x, w, 1e-6, residual=r)
    _close(y, y0, 3e-2, 2e-2, "rms+res")
    _close(nr, nr0, 1e-2, 1e-2, "res out")
    _close(ops.rms_norm(x, w, 1e-6, gemma=True), ref.rms_norm(x.float(), w, 1e-6, gemma=True), 3e-2, 1e-2, "gemma")
    _close(ops.layer_norm(x, w, b, 1e-5), ref.layer_norm(x.float(), w, b, 1e-5), 3e-2, 1e-2, "ln")
    sc, sh = _rand(7, H, scale=0.2), _rand(7, H, scale=0.2)
    _close(ops.layer_norm(x, None, None, 1e-6, sc, sh, 11), ref.layer_norm(x.float(), None, None, 1e-6, sc, sh, 11),
           3e-2, 1e-2, "adaln")


@pytest.mark.parametrize("H,rows", [(3072, 2304), (4096, 2050), (2560, 4100), (1280, 3000)])
def test_norms_many_rows_take_the_warp_per_row_kernels(H, rows):
    """With thousands of rows the norms run one warp per row (up to 2048 columns for every mode, up to 4096 for
    LayerNorm); same restatement as the block-per-row kernel."""
    torch.manual_seed(33)
    x, r, w, b = _rand(rows, H), _rand(rows, H), _rand(H), _rand(H)
    sc, sh = _rand(2, H, scale=0.2), _rand(2, H, scale=0.2)
    rpb = (rows + 1) // 2
    _close(ops.layer_norm(x, None, None, 1e-6, sc, sh, rpb), ref.layer_norm(x.float(), None, None, 1e-6, sc, sh, rpb),
           3e-2, 1e-2, "adaln")
    _close(ops.layer_norm(x, w, b, 1e-5), ref.layer_norm(x.float(), w, b, 1e-5), 3e-2, 1e-2, "ln")
    y, nr = ops.layer_norm(x, w, b, 1e-5, residual=r)
    y0, nr0 = ref.layer_norm(x, w, b, 1e-5, residual=r)
    _close(y, y0, 3e-2, 2e-2, "ln+res")
    _close(nr, nr0, 1e-2, 1e-2, "res out")
    y, nr = ops.rms_norm(x, w, 1e-6, residual=r)
    y0, nr0 = ref.rms_norm(x, w, 1e-6, residual=r)
    _close(y, y0, 3e-2, 2e-2, "rms+res")
    _close(nr, nr0, 1e-2, 1e-2, "rms res out")


def test_rope_and_tables():
    torch.manual_seed(4)
    T, H, d = 333, 16, 80
    qkv = _rand(T, 3 * H * d)
    cs = torch.stack([torch.randn(T, d // 2, device=DEV).cos(), torch.randn(T, d // 2, device=DEV).sin()], 1).contiguous()
    q = qkv[:, : H * d].view(T, H, d)
    want = ref.rope(q.clone(), cs)
    ops.rope_(q, cs)
    _close(q, want, 1e-2, 1e-2, "rope")
    pos = torch.randint(0, 4000, (3, T), device=DEV, dtype=torch.int32)
    t = ops.mrope_table(pos, 64, 1e6, [16, 24, 24])
    _close(t, ref.mrope_table(pos.cpu(), 64, 1e6, [16, 24, 24]).to(DEV), 2e-3, 0, "mrope table")


@pytest.mark.parametrize("H,d,lens,causal", [
    (16, 80, [64, 64, 48, 64, 17], False),
    (16, 80, [1000, 300], False),
    (4, 128, [257, 128, 5], True),
    (2, 64, [130], False),
    (3, 72, [200, 9], False),
])
def test_attention_varlen(H, d, lens, causal):
    torch.manual_seed(5)
    T = sum(lens)
    qkv = _rand(T, 3 * H * d)
    q, k, v = (qkv[:, i * H * d: (i + 1) * H * d].view(T, H, d) for i in range(3))
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device=DEV, dtype=torch.int32)
    o = ops.attention_varlen(q, k, v, cu, cu, max(lens), causal=causal)
    want = ref.attention_varlen(q.float(), k.float(), v.float(), cu.cpu(), cu.cpu(), 1 / math.sqrt(d), causal)
    _close(o, want, 2e-2, 2e-2, f"attn H={H} d={d}")


@pytest.mark.parametrize("q_lens,ctx", [([1, 1, 1], [300, 128, 1]), ([200, 77], [200, 500]), ([1] * 9, [1000] * 9)])
@pytest.mark.parametrize("pack", [False, True])
@pytest.mark.parametrize("kv_splits", [1, 0, 3])
def test_attention_paged(q_lens, ctx, pack, kv_splits):
    torch.manual_seed(6)
    Hq, Hkv, d, page = 28, 4, 128, 128
    B = len(q_lens)
    nblk = [(c + page - 1) // page for c in ctx]
    pages = sum(nblk) + 2
    cache = torch.zeros(pages, 2, Hkv, page, d, device=DEV, dtype=torch.bfloat16)
    perm = torch.randperm(pages - 1)[: sum(nblk)] + 1
    bt = torch.zeros(B, max(nblk), dtype=torch.int32)
    p = 0
    for s in range(B):
        bt[s, : nblk[s]] = perm[p: p + nblk[s]].int()
        p += nblk[s]
    bt = bt.to(DEV)
    for s in range(B):
        n = ctx[s]
        kv = _rand(2, n, Hkv, d)
        for j in range(nblk[s]):
            m = min(page, n - j * page)
            cache[bt[s, j], :, :, :m] = kv[:, j * page: j * page + m].permute(0, 2, 1, 3)
    Tq = sum(q_lens)
    q = _rand(Tq, Hq, d)
    cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), device=DEV, dtype=torch.int32)
    kv_len = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    o = ops.attention_paged(q, cache, bt, kv_len, cu, max(q_lens), causal=True, pack_gqa=pack, kv_splits=kv_splits)
    want = ref.attention_paged(q.cpu().float(), cache.cpu().float(), bt.cpu(), kv_len.cpu(), cu.cpu(),
                               1 / math.sqrt(d), True)
    _close(o, want.to(DEV), 2e-2, 2e-2, "paged attn")


def test_rope_kv_write():
    torch.manual_seed(7)
    T, Hq, Hkv, d, page = 150, 28, 4, 128, 128
    qkv = _rand(T, (Hq + 2 * Hkv) * d)
    pos = torch.arange(T, device=DEV, dtype=torch.int32)[None].expand(3, -1).contiguous()
    cs = ops.mrope_table(pos, d // 2, 1e6, [16, 24, 24])
    cache = torch.zeros(4, 2, Hkv, page, d, device=DEV, dtype=torch.bfloat16)
    slot = (torch.arange(T, device=DEV, dtype=torch.int32) + 128)
    slot[3] = -1
    cache_ref = cache.clone().cpu()
    q_ref = ref.rope_kv_write(qkv.clone().cpu(), Hq, Hkv, d, cs.cpu(), cache_ref, slot.cpu(), page)
    q = ops.rope_kv_write_(qkv, Hq, Hkv, d, cs, cache, slot)
    _close(q, q_ref.to(DEV), 2e-2, 1e-2, "q rope")
    _close(cache, cache_ref.to(DEV), 2e-2, 1e-2, "cache")


def test_misc_kernels():
    torch.manual_seed(8)
    gu = _rand(33, 2 * 3424)
    _close(ops.act_mul(gu), ref.act_mul(gu.float()), 2e-2, 1e-2, "act_mul")
    src = _rand(100, 1280)
    idx = torch.randperm(100, device=DEV)[:60].int()
    assert torch.equal(ops.gather_rows(src, idx), src[idx.long()])
    dst = torch.zeros(100, 1280, device=DEV, dtype=torch.bfloat16)
    ops.scatter_rows_(dst, idx, src[:60])
    assert torch.equal(dst[idx.long()], src[:60])
    logits = _rand(7, 152064)
    assert torch.equal(ops.argmax(logits).long(), logits.float().argmax(-1))
    lf = logits.float()
    assert torch.equal(ops.argmax(lf).long(), lf.argmax(-1))
    x = torch.randn(64, 64, device=DEV)
    c, u = _rand(64, 64), _rand(64, 64)
    want = ref.flow_step(x.clone(), c, u, 4.0, -0.02, True)
    ops.flow_step_(x, c, u, 4.0, -0.02, True)
    _close(x, want, 1e-4, 1e-4, "flow step")
    w = torch.rand(1000, device=DEV) * 2.4 - 1.2
    assert (ops.pcm16(w).int() - ref.pcm16(w).int()).abs().max() <= 1


@pytest.mark.parametrize("M,N,K", [(1, 256, 128), (16, 3584, 3584), (64, 3584, 18944), (7, 4608, 3584), (128, 1000, 1352),
                                   (100, 152064, 512)])
@pytest.mark.parametrize("splits", [0, 1, 3, 6])   # 6: more CTAs than SMs for the wide shapes (the last split reduces alone)
def test_gemm_skinny(M, N, K, splits):
    if N > 100000 and splits > 1:
        pytest.skip("split-K scratch is sized for decoder projections, not for a forced split of the vocabulary")
    torch.manual_seed(9)
    x, w, b, r = _rand(M, K), _rand(N, K, scale=K ** -0.5), _rand(N), _rand(M, N)
    for _ in range(2):  # twice: the split-K counters must be back at zero after a call
        y = ops.linear(x, w, b, act="gelu", residual=r, skinny=True, splits=splits)
        _close(y, ref.linear(x, w, b, "gelu", r, out_dtype=torch.float32), 3e-2, 2e-2, f"skinny {M}x{N}x{K}")
    y32 = ops.linear(x, w, out_dtype=torch.float32, splits=splits)
    _close(y32, ref.linear(x, w, out_dtype=torch.float32), 1e-2, 1e-2, "skinny fp32")


@pytest.mark.parametrize("M,I,K", [(16, 18944, 3584), (3, 96, 64), (128, 1712, 1280)])
@pytest.mark.parametrize("splits", [0, 1, 2])
def test_gemm_skinny_swiglu(M, I, K, splits):
    torch.manual_seed(10)
    x, w, b = _rand(M, K), _rand(2 * I, K, scale=K ** -0.5), _rand(2 * I, scale=0.1)
    y = ops.swiglu_linear(x, w, b, skinny=True, splits=splits)
    _close(y, ref.swiglu_linear(x.float(), w.float(), b.float()), 3e-2, 2e-2, "skinny swiglu")


# ------------------------------------------------------------------------------------------------
# generator kernels
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("d,heads", [(64, 5), (128, 24), (256, 2)])
@pytest.mark.parametrize("with_norm,with_rope", [(True, True), (True, False), (False, True)])
def test_head_norm_rope(d, heads, with_norm, with_rope):
    torch.manual_seed(10)
    T = 77
    buf = _rand(T, 3 * heads * d)
    x = buf[:, heads * d: 2 * heads * d].view(T, heads, d)  # a strided view, as q/k inside a fused qkv buffer
    w = (1 + 0.2 * torch.randn(d, device=DEV)).bfloat16() if with_norm else None
    ang = torch.rand(T, d // 2, device=DEV) * 6.28
    cs = torch.stack([ang.cos(), ang.sin()], dim=1).contiguous() if with_rope else None
    want = ref.head_norm_rope(x.clone(), w, 1e-6, cs)
    before = buf.clone()
    ops.head_norm_rope_(x, w, 1e-6, cs)
    _close(x, want, 2e-2, 2e-2, "head_norm_rope")
    assert torch.equal(buf[:, : heads * d], before[:, : heads * d]) and torch.equal(buf[:, 2 * heads * d:], before[:, 2 * heads * d:])


@pytest.mark.parametrize("heads,two_streams", [(24, True), (6, False), (3, True), (2, True)])
def test_qk_norm_rope_one_launch(heads, two_streams):
    """q and k parts of a fused projection in one launch (d = 128) against the per-part fp32 restatement."""
    torch.manual_seed(14)
    T, d, seg, n_first = 93, 128, 31, 7
    D = heads * d
    buf = _rand(T, 3 * D + 8)[:, :3 * D]     # row stride wider than the columns
    ws = [(1 + 0.2 * torch.randn(d, device=DEV)).bfloat16() for _ in range(4)]
    ang = torch.rand(T, d // 2, device=DEV) * 6.28
    cs = torch.stack([ang.cos(), ang.sin()], dim=1).contiguous()
    first = (torch.arange(T, device=DEV) % seg) < n_first
    want = buf.clone()
    for part, (w, w2) in enumerate(((ws[0], ws[2]), (ws[1], ws[3]))):
        x = buf[:, part * D:(part + 1) * D].reshape(T, heads, d)
        a = ref.head_norm_rope(x.clone(), w, 1e-6, cs)
        b = ref.head_norm_rope(x.clone(), w2, 1e-6, cs) if two_streams else a
        want[:, part * D:(part + 1) * D] = torch.where(first[:, None, None], a, b).reshape(T, D).to(want.dtype)
    kw = dict(wq2=ws[2], wk2=ws[3], seg=seg, n_first=n_first) if two_streams else {}
    ops.qk_norm_rope_(buf, heads, d, D, ws[0], ws[1], 1e-6, cs, **kw)
    _close(buf[:, :2 * D], want[:, :2 * D], 2e-2, 2e-2, "qk_norm_rope")
    assert torch.equal(buf[:, 2 * D:], want[:, 2 * D:])


def _sample_args(rows, temp, top_p, top_k, seed0=0):
    f = lambda v, dt: torch.full((rows,), v, device=DEV, dtype=dt)  # noqa: E731
    return (f(temp, torch.float32), f(top_p, torch.float32), f(top_k, torch.int32),
            torch.arange(seed0, seed0 + rows, device=DEV, dtype=torch.int64), torch.zeros(rows, device=DEV, dtype=torch.int32))


def test_sample_rows_degenerate_cases_are_the_argmax():
    torch.manual_seed(20)
    logits = torch.randn(37, 152064, device=DEV) * 3
    want = logits.argmax(-1).int()
    for temp, top_p, top_k in ((0.0, 1.0, 0), (0.7, 1.0, 1), (1.0, 1e-6, 0)):
        args = _sample_args(37, temp, top_p, top_k)
        assert torch.equal(ops.sample_rows(logits, *args), want), (temp, top_p, top_k)
        assert int(args[4].min()) == 1 and int(args[4].max()) == 1     # the draw index advanced once


@pytest.mark.parametrize("V,temp,top_p,top_k", [(1000, 0.9, 0.8, 25), (152064, 1.0, 0.9, 0), (152064, 1.3, 1.0, 50),
                                                (5000, 0.6, 0.95, 200), (777, 1.0, 1.0, 0)])
def test_sample_rows_cutoffs_distribution_and_streams(V, temp, top_p, top_k):
    """Every draw lies inside the set that the fp32 restatement keeps, follows the renormalised probabilities, and is a
    function of (seed, draw index) alone."""
    torch.manual_seed(21)
    rows = 4096
    base = torch.randn(V, device=DEV) * 2.5
    logits = base[None].repeat(rows, 1).contiguous()
    keep, _ = ref.sample_kept_mask(base, temp, top_p, top_k)
    keep = torch.from_numpy(keep).to(DEV)
    args = _sample_args(rows, temp, top_p, top_k)
    toks = ops.sample_rows(logits, *args)
    assert int(toks.min()) >= 0 and int(toks.max()) < V
    inside = keep[toks.long()].float().mean().item()
    assert inside >= 0.999, inside          # a logit that ties the cut-off to the last bit may fall either way
    probs = torch.softmax(base.double() / temp, -1) * keep
    probs = probs / probs.sum()
    freq = torch.bincount(toks.long(), minlength=V).double() / rows
    assert (freq - probs).abs().max().item() < 0.03
    again = _sample_args(rows, temp, top_p, top_k)
    assert torch.equal(ops.sample_rows(logits, *again), toks)                    # same seeds, same draw index
    nxt = ops.sample_rows(logits, *args)                                         # draw index 1 of the same streams
    assert (nxt != toks).float().mean().item() > 0.2 or int(keep.sum()) < 3
    # the restatement on the CPU (same hash, same fixed-point weights) picks the same token almost everywhere
    n = 64
    cpu = ref.sample_rows(logits[:n].cpu(), *[a[:n].cpu() for a in _sample_args(rows, temp, top_p, top_k)])
    assert (cpu.to(DEV) == toks[:n]).float().mean().item() >= 0.9


def test_sample_rows_mixed_rows():
    torch.manual_seed(22)
    V, rows = 4096, 64
    logits = torch.randn(rows, V, device=DEV) * 2
    temp = torch.where(torch.arange(rows, device=DEV) % 2 == 0, 0.0, 1.0).float()
    args = (temp, torch.ones(rows, device=DEV), torch.zeros(rows, device=DEV, dtype=torch.int32),
            torch.arange(rows, device=DEV, dtype=torch.int64), torch.zeros(rows, device=DEV, dtype=torch.int32))
    toks = ops.sample_rows(logits, *args)
    assert torch.equal(toks[0::2], logits[0::2].argmax(-1).int())
    assert (toks[1::2] != logits[1::2].argmax(-1).int()).float().mean().item() > 0.5


def test_softmax_rows():
    torch.manual_seed(11)
    x = _rand(300, 1032, scale=4.0)
    _close(ops.softmax_rows(x, 0.37), ref.softmax_rows(x, 0.37), 2e-3, 2e-2, "softmax")


@pytest.mark.parametrize("up,silu", [(1, False), (2, True), (1, True)])
def test_im2col3x3_and_conv(up, silu):
    torch.manual_seed(12)
    B, H, W, C, Co = 2, 7, 9, 24, 40
    x = _rand(B * H * W, C)
    assert torch.equal(ops.im2col3x3(x, B, H, W, up, silu), ref.im2col3x3(x, B, H, W, up, silu)) or \
        (ops.im2col3x3(x, B, H, W, up, silu).float() - ref.im2col3x3(x, B, H, W, up, silu).float()).abs().max() < 2e-2
    w, b = _rand(Co, 9 * C, scale=(9 * C) ** -0.5), _rand(Co)
    y = ops.conv3x3(x, w, b, B, H, W, up=up, silu=silu)
    # the same convolution through torch (NCHW)
    img = x.float().view(B, H, W, C).permute(0, 3, 1, 2)
    if silu:
        img = torch.nn.functional.silu(img)
    if up == 2:
        img = torch.nn.functional.interpolate(img, scale_factor=2.0, mode="nearest")
    w4 = w.float().view(Co, 3, 3, C).permute(0, 3, 1, 2)
    want = torch.nn.functional.conv2d(img, w4, b.float(), padding=1).permute(0, 2, 3, 1).reshape(-1, Co)
    _close(y, want, 3e-2, 3e-2, "conv3x3")


def test_conv1d_family():
    torch.manual_seed(13)
    B, T, C, Co = 2, 37, 16, 24
    x = _rand(B * T, C)
    alpha, beta = torch.randn(C, device=DEV) * 0.3, torch.randn(C, device=DEV) * 0.3
    for k, dil in ((7, 1), (7, 3), (1, 1)):
        w, b = _rand(Co, k * C, scale=(k * C) ** -0.5), _rand(Co)
        y = ops.conv1d_causal(x, w, b, B, T, k, dil, alpha=alpha, beta=beta)
        xin = ref.snake_beta(x.float().view(B, T, C), alpha, beta).transpose(1, 2)
        w3 = w.float().view(Co, k, C).permute(0, 2, 1)
        want = torch.nn.functional.conv1d(torch.nn.functional.pad(xin, ((k - 1) * dil, 0)), w3, b.float(), dilation=dil)
        _close(y, want.transpose(1, 2).reshape(B * T, Co), 3e-2, 3e-2, f"conv1d k={k} dil={dil}")
    # transposed convolutions: kernel == stride, and kernel == 2 * stride with both ends trimmed by stride
    for s, k in ((2, 2), (3, 6)):
        wt, bt = _rand(C, Co, k, scale=C ** -0.5), _rand(Co)
        wk = wt.permute(2, 1, 0)
        w2d = torch.cat([wk[:s].reshape(s * Co, C)] + ([wk[s:].reshape(s * Co, C)] if k == 2 * s else []), dim=1).contiguous()
        y, To = ops.conv_transpose1d_causal(x, w2d, bt.repeat(s), B, T, s, k)
        full = torch.nn.functional.conv_transpose1d(x.float().view(B, T, C).transpose(1, 2), wt.float(), bt.float(), stride=s)
        pad = k - s
        want = full[..., pad: full.shape[-1] - pad] if pad else full
        assert To == want.shape[-1]
        _close(y, want.transpose(1, 2).reshape(B * To, Co), 3e-2, 3e-2, f"convT s={s} k={k}")
    wd, bd = _rand(C, 7, scale=0.4), _rand(C)
    _close(ops.dwconv1d(x, wd, bd, B, T), ref.dwconv1d(x, wd, bd, B, T), 2e-2, 2e-2, "dwconv1d")


def test_to_rgb8():
    x = _rand(1000, 8)
    got, want = ops.to_rgb8(x), ref.to_rgb8(x)
    assert got.dtype == torch.uint8 and (got.int() - want.int()).abs().max().item() <= 1


@pytest.mark.parametrize("window", [6, 72, 200])
def test_attention_sliding_window(window):
    torch.manual_seed(14)
    H, d, lens = 4, 64, [325, 40]
    T = sum(lens)
    q, k, v = _rand(T, H, d), _rand(T, H, d), _rand(T, H, d)
    cu = torch.tensor([0, lens[0], T], device=DEV, dtype=torch.int32)
    got = ops.attention_varlen(q, k, v, cu, cu, max(lens), causal=True, window=window)
    want = ref.attention_varlen(q, k, v, cu, cu, 1 / math.sqrt(d), True, window)
    _close(got, want, 2e-2, 2e-2, f"sliding window {window}")


@pytest.mark.parametrize("Hq,Hkv", [(28, 4), (16, 16), (32, 2), (8, 2)])
@pytest.mark.parametrize("ctx,kv_splits", [([1, 127, 128, 129, 700], 0), ([3500, 40, 2049], 1), ([3500, 40, 2049], 3),
                                           ([5, 9], 4)])
def test_attention_decode_swapped_operands(Hq, Hkv, ctx, kv_splits):
    """The decode kernel (keys on the 128-row side, grouped query heads on the other) against the fp32 restatement;
    the stale rows beyond kv_len in the last page hold large values and must not leak in."""
    torch.manual_seed(15)
    d, page = 128, 128
    B = len(ctx)
    nblk = [(c + page - 1) // page for c in ctx]
    pages = sum(nblk) + 3
    cache = (torch.randn(pages, 2, Hkv, page, d, device=DEV) * 30).bfloat16()  # garbage everywhere, overwritten below
    perm = torch.randperm(pages - 1)[: sum(nblk)] + 1
    bt = torch.zeros(B, max(nblk) + 1, dtype=torch.int32)
    p = 0
    for s in range(B):
        bt[s, : nblk[s]] = perm[p: p + nblk[s]].int()
        p += nblk[s]
    bt = bt.to(DEV)
    for s in range(B):
        kv = _rand(2, ctx[s], Hkv, d)
        for j in range(nblk[s]):
            m = min(page, ctx[s] - j * page)
            cache[bt[s, j], :, :, :m] = kv[:, j * page: j * page + m].permute(0, 2, 1, 3)
    qkv = _rand(B, (Hq + 2 * Hkv) * d)
    q = qkv[:, : Hq * d].view(B, Hq, d)  # strided view, as the engine passes it
    cu = torch.arange(B + 1, device=DEV, dtype=torch.int32)
    kv_len = torch.tensor(ctx, device=DEV, dtype=torch.int32)
    o = ops.attention_paged(q, cache, bt, kv_len, cu, 1, causal=True, pack_gqa=True, kv_splits=kv_splits)
    want = ref.attention_paged(q.cpu().float(), cache.cpu().float(), bt.cpu(), kv_len.cpu(), cu.cpu(), 1 / math.sqrt(d), True)
    _close(o, want.to(DEV), 2e-2, 2e-2, f"decode attn Hq={Hq} Hkv={Hkv}")


def test_strided_tap_gathers_and_bilinear_embed():
    torch.manual_seed(16)
    B, H, W, C = 2, 9, 12, 16
    x = _rand(B * H * W, C)
    got, want = ops.im2col3x3(x, B, H, W, stride=2), ref.im2col3x3(x, B, H, W, stride=2)
    assert got.shape == want.shape == (B * 5 * 6, 9 * C) and torch.equal(got, want)
    T = 41
    s = _rand(B * T, C)
    To = (T - 1) // 2 + 1
    assert torch.equal(ops.im2col1d(s, B, T, To, 3, -1, stride=2), ref.im2col1d(s, B, T, To, 3, -1, 1, stride=2))
    table = _rand(36, 64)
    L = 77
    idx = torch.randint(0, 36, (4, L), device=DEV, dtype=torch.int32)
    wgt = torch.rand(4, L, device=DEV)
    xe = _rand(L, 64)
    want = (xe.float() + (table.float()[idx.long()] * wgt[:, :, None]).sum(0))
    ops.bilinear_embed_add_(xe, table, idx, wgt)
    _close(xe, want, 2e-2, 2e-2, "bilinear embed")


@pytest.mark.parametrize("model_id,modality", [("cornserve-b200/tiny-qwen3-vl", "image"), ("cornserve-b200/tiny-qwen3-omni", "audio"),
                                               ("cornserve-b200/tiny-internvl", "image"), ("cornserve-b200/tiny-llava-onevision", "image")])
def test_encoder_families_cuda_vs_cpu(model_id, modality, monkeypatch):
    """The same random weights on the CUDA kernels and on the fp32 reference path give the same embeddings."""
    import numpy as np

    from cornserve.task_executors.eric.config import EricConfig, ModelConfig
    from cornserve.task_executors.eric.schema import Batch, Modality
    from cornserve.task_executors.eric.worker import Worker

    rng = np.random.default_rng(0)
    if modality == "audio":
        data = {"raw_audio": [torch.from_numpy(rng.standard_normal(16000 * 2).astype(np.float32) * 0.1)]}
    else:
        data = {"raw_images": [torch.from_numpy(rng.integers(0, 256, (70, 120, 3), dtype=np.uint8))]}
    outs = {}
    for dev in ("cpu", "cuda"):
        monkeypatch.setenv("CORNSERVE_DEVICE", dev)
        monkeypatch.setenv("CORNSERVE_SEED", "0")
        w = Worker(EricConfig(model=ModelConfig(id=model_id, modality=Modality(modality))))
        if dev == "cuda":
            w.model.load_state_dict(outs["state"])
            w.model.bfloat16()
        else:
            outs["state"] = {k: v.clone() for k, v in w.model.state_dict().items()}
        with torch.inference_mode():
            y = w.model(modality, model_id, w.prepare(Batch(Modality(modality), model_id, ["r"], ["d"], [None], dict(data))))
        outs[dev] = torch.cat(y).float().cpu()
    cos = torch.nn.functional.cosine_similarity(outs["cpu"].flatten(), outs["cuda"].flatten(), dim=0).item()
    assert outs["cpu"].shape == outs["cuda"].shape and cos > 0.98, cos


# ------------------------------------------------------------------------------------------------
# mixture of experts: route -> layout -> dispatch -> grouped GEMMs -> combine, no host round trip
# ------------------------------------------------------------------------------------------------
def _moe_reference(x, logits, wgu, wd, k, norm):
    """fp32 restatement on the CPU (bf16 rounding of the intermediate activations as the kernels do)."""
    x, logits, wgu, wd = x.float().cpu(), logits.float().cpu(), wgu.float().cpu(), wd.float().cpu()
    I = wd.shape[2]
    p = torch.softmax(logits, dim=-1)
    w, idx = torch.topk(p, k, dim=-1)
    if norm:
        w = w / w.sum(-1, keepdim=True)
    out = torch.zeros_like(x)
    for e in range(wgu.shape[0]):
        tok, slot = (idx == e).nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        h = (torch.nn.functional.silu(xe @ wgu[e, :I].t()) * (xe @ wgu[e, I:].t())).bfloat16().float()
        y = (h @ wd[e].t()).bfloat16().float()
        out.index_add_(0, tok, y * w[tok, slot, None])
    return out, idx


@pytest.mark.parametrize("T,E,k,H,I", [(1, 128, 8, 2048, 768), (37, 128, 8, 2048, 768), (700, 32, 4, 512, 256),
                                       (3000, 8, 2, 256, 128), (64, 16, 16, 256, 64)])
def test_fused_moe_layer_matches_reference(T, E, k, H, I):
    from cornserve.parallel.moe import FusedMoE
    from cornserve.parallel.state import single_group

    g = torch.Generator(device="cuda").manual_seed(T + E)
    x = torch.randn(T, H, device="cuda", generator=g).bfloat16()
    logits = torch.randn(T, E, device="cuda", generator=g) * 2
    wgu = (torch.randn(E, 2 * I, H, device="cuda", generator=g) * H ** -0.5).bfloat16()
    wd = (torch.randn(E, H, I, device="cuda", generator=g) * I ** -0.5).bfloat16()
    layer = FusedMoE(single_group("cuda"), E, k, H, I, max_tokens=4096)
    want, idx = _moe_reference(x, logits, wgu, wd, k, True)
    for _ in range(2):  # the second call runs on the advanced epoch and reused buffers
        got = layer.forward(x, logits, wgu, wd).float().cpu()
        ops.check_error("fused moe")
        assert torch.equal(layer.topk_e[: T * k].view(T, k).cpu().sort(-1).values.long(), idx.sort(-1).values)
        err = (got - want).abs().max().item()
        assert err < 0.03 * want.abs().max().item() + 0.02, err
    assert int(layer.epoch.item()) == 2 and int(layer.overflow.item()) == 0


def test_fused_moe_layer_replays_from_a_cuda_graph():
    from cornserve.parallel.moe import FusedMoE
    from cornserve.parallel.state import single_group

    T, E, k, H, I = 48, 64, 4, 512, 256
    x = torch.randn(T, H, device="cuda").bfloat16()
    logits = torch.randn(T, E, device="cuda")
    wgu = (torch.randn(E, 2 * I, H, device="cuda") * H ** -0.5).bfloat16()
    wd = (torch.randn(E, H, I, device="cuda") * I ** -0.5).bfloat16()
    layer = FusedMoE(single_group("cuda"), E, k, H, I, max_tokens=1024)
    eager = layer.forward(x, logits, wgu, wd).clone()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = layer.forward(x, logits, wgu, wd)
    for _ in range(3):
        x.copy_(torch.randn(T, H, device="cuda").bfloat16())
        graph.replay()
    torch.cuda.synchronize()
    ops.check_error("fused moe graph")
    want, _ = _moe_reference(x, logits, wgu, wd, k, True)
    assert (out.float().cpu() - want).abs().max().item() < 0.03 * want.abs().max().item() + 0.02
    assert eager.shape == out.shape


def test_kv_page_copy_is_byte_exact():
    L, pages, hkv, d = 3, 40, 2, 64
    src = torch.randn(L, pages, 2, hkv, 128, d, device="cuda").bfloat16()
    dst = torch.zeros(L, 24, 2, hkv, 128, d, device="cuda", dtype=torch.bfloat16)
    sp = torch.tensor([7, 39, 1, 18, 2], device="cuda", dtype=torch.int32)
    dp = torch.tensor([23, 0, 5, 6, 11], device="cuda", dtype=torch.int32)
    ops.kv_copy_pages(dst, src, sp, dp)
    torch.cuda.synchronize()
    ops.check_error("kv copy")
    want = torch.zeros_like(dst)
    want[:, dp.long()] = src[:, sp.long()]
    assert torch.equal(dst.view(torch.int16), want.view(torch.int16))
    # a page number outside the cache is refused by the kernel (error status), nothing is written
    before = dst.clone()
    ops.kv_copy_pages(dst, src, torch.tensor([40], device="cuda", dtype=torch.int32), torch.tensor([1], device="cuda", dtype=torch.int32))
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError):
        ops.check_error("kv copy with a bad page")
    assert torch.equal(dst.view(torch.int16), before.view(torch.int16))


# ------------------------------------------------------------------------------------------------
# fp8 block-scaled GEMM
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(5, 256, 512), (128, 384, 1024), (300, 200, 256), (1000, 3584, 3584)])
def test_fp8_blockscaled_linear(M, N, K):
    g = torch.Generator(device="cuda").manual_seed(M + N)
    x = (torch.randn(M, K, device="cuda", generator=g) * (1 + 3 * torch.rand(M, 1, device="cuda", generator=g))).bfloat16()
    w = (torch.randn(N, K, device="cuda", generator=g) * K ** -0.5).bfloat16()
    bias = torch.randn(N, device="cuda", generator=g).bfloat16()
    wq, ws = ops.quantize_fp8_weight(w)
    xq, xs = ops.quantize_fp8_rows(x)
    # the quantiser against its restatement on the CPU
    xq_c, xs_c = ops.quantize_fp8_rows(x.cpu())
    assert torch.allclose(xs.cpu(), xs_c, rtol=1e-6, atol=0)
    assert (xq.float().cpu() - xq_c.float()).abs().max().item() <= 32.0  # at most one e4m3 step at the top of the range
    assert (xq.float().cpu() != xq_c.float()).float().mean().item() < 1e-3
    got = ops.linear_fp8(x, wq, ws, bias, xq=(xq, xs)).float().cpu()
    torch.cuda.synchronize()
    ops.check_error("fp8 gemm")
    # exact oracle: the same quantised operands, dequantised and multiplied in fp32 on the CPU
    want = ops.linear_fp8(x.cpu(), wq.cpu(), ws.cpu(), bias.cpu(), xq=(xq.cpu(), xs.cpu()))
    err = (got - want).abs().max().item()
    assert err < 0.01 * want.abs().max().item() + 0.02, err
    # and it is a faithful 8-bit approximation of the bf16 layer
    ref = x.float().cpu() @ w.float().cpu().t() + bias.float().cpu()
    rel = (got - ref).norm().item() / ref.norm().item()
    assert rel < 0.06, rel


@pytest.mark.parametrize("layer_norm", [False, True])
def test_reduce_norm_push_kernel_single_rank(layer_norm):
    """The reduce + bias + residual + norm kernel of the tensor-parallel encoder chain with one rank playing the whole
    group: two partial-sum slots are summed, the new residual is stored, and the normalised rows (RMSNorm or LayerNorm)
    land in the operand buffer with their arrival counters."""
    import ctypes

    from cornserve.ops import _lib
    from cornserve.parallel import fused  # noqa: F401  (declares the entry point's signature)

    rows, H = 256, 1280
    g = torch.Generator(device="cuda").manual_seed(7)
    part = torch.randn(1, rows, H, device="cuda", generator=g).bfloat16()
    bias, res = torch.randn(H, device="cuda", generator=g).bfloat16(), torch.randn(rows, H, device="cuda", generator=g).bfloat16()
    w, b = (1 + 0.1 * torch.randn(H, device="cuda", generator=g)).bfloat16(), torch.randn(H, device="cuda", generator=g).bfloat16()
    flags = torch.full((rows // 128,), 5, device="cuda", dtype=torch.int32)       # "all tiles have arrived"
    x_out = torch.empty(rows, H, device="cuda", dtype=torch.bfloat16)
    gathered = torch.zeros(rows, H, device="cuda", dtype=torch.bfloat16)
    gflags = torch.zeros(rows // 128, device="cuda", dtype=torch.int32)
    gp, fp = (ctypes.c_void_p * 1)(gathered.data_ptr()), (ctypes.c_void_p * 1)(gflags.data_ptr())
    lib = _lib.load()
    rc = lib.cs_tp_reduce_norm_push(rows, H, 1, 0, rows, part.data_ptr(), H, flags.data_ptr(), 5, bias.data_ptr(), res.data_ptr(), H,
                                    x_out.data_ptr(), H, w.data_ptr(), 1e-6, b.data_ptr() if layer_norm else None, int(layer_norm),
                                    ctypes.cast(gp, ctypes.c_void_p), ctypes.cast(fp, ctypes.c_void_p), H, 128,
                                    torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    ops.check_error("reduce norm push")
    want_x = (part[0].float() + bias.float() + res.float()).bfloat16()
    assert torch.equal(x_out, want_x)
    xf = want_x.float()
    if layer_norm:
        want = torch.nn.functional.layer_norm(xf, (H,), w.float(), b.float(), 1e-6)
    else:
        want = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert torch.allclose(gathered.float(), want, atol=3e-2, rtol=3e-2)
    assert gflags.tolist() == [128, 128]


def test_packed_attention_windows_match_unpacked():
    """Several short windows sharing one 128-row tile (per-token key bounds) against one window per tile."""
    import numpy as np

    from cornserve.models.qwen2_5_vl import pack_windows, window_index

    grid = np.array([[1, 52, 92], [1, 16, 24], [2, 20, 28]])
    _, cu = window_index(grid, 112, 2, 14)
    T, H, d = int(cu[-1]), 4, 80
    g = torch.Generator(device="cuda").manual_seed(4)
    q, k, v = (torch.randn(T, H, d, device="cuda", generator=g).bfloat16() for _ in range(3))
    cu_d = torch.from_numpy(cu).cuda()
    want = ops.attention_varlen(q, k, v, cu_d, cu_d, int(np.diff(cu).max()))
    cu_p, lo, hi = pack_windows(cu)
    assert len(cu_p) < len(cu) and int(np.diff(cu_p).max()) <= 128 and cu_p[-1] == cu[-1]
    cu_pd = torch.from_numpy(cu_p).cuda()
    got = ops.attention_varlen(q, k, v, cu_pd, cu_pd, int(np.diff(cu_p).max()),
                               row_bounds=(torch.from_numpy(lo).cuda(), torch.from_numpy(hi).cuda()))
    torch.cuda.synchronize()
    ops.check_error("packed windows")
    assert torch.allclose(got.float(), want.float(), atol=2e-2, rtol=2e-2)
    # and the CPU restatement of the bounded form agrees with the plain CPU path
    qc, kc, vc = q[:400].float().cpu(), k[:400].float().cpu(), v[:400].float().cpu()
    n = int(np.searchsorted(cu, 400, side="right")) - 1
    cu_c = torch.from_numpy(cu[: n + 1])
    Tn = int(cu[n])
    plain = ops.attention_varlen(qc[:Tn], kc[:Tn], vc[:Tn], cu_c, cu_c, 64)
    one = torch.tensor([0, Tn], dtype=torch.int32)
    bounded = ops.attention_varlen(qc[:Tn], kc[:Tn], vc[:Tn], one, one, Tn, row_bounds=(torch.from_numpy(lo[:Tn]), torch.from_numpy(hi[:Tn])))
    assert torch.allclose(plain, bounded, atol=1e-4)


@pytest.mark.parametrize("nbytes,src_off,dst_off", [(1196 * 3584 * 2, 0, 0), (4096 + 5, 0, 0), (777, 16, 32), (100_003, 3, 0),
                                                    (64 << 20, 0, 256), (15, 0, 0)])
def test_push_bytes_is_an_exact_copy(nbytes, src_off, dst_off):
    """The sidecar's copy kernel: vector path, ragged tail and misaligned pointers, bit for bit; bytes around the
    destination stay untouched."""
    g = torch.Generator(device=DEV).manual_seed(nbytes)
    src_buf = torch.randint(0, 256, (nbytes + src_off + 64,), device=DEV, dtype=torch.uint8, generator=g)
    dst_buf = torch.full((nbytes + dst_off + 64,), 0xAB, device=DEV, dtype=torch.uint8)
    src, dst = src_buf[src_off: src_off + nbytes], dst_buf[dst_off: dst_off + nbytes]
    ops.push_bytes_(dst, src)
    torch.cuda.synchronize()
    assert torch.equal(dst, src)
    assert bool((dst_buf[:dst_off] == 0xAB).all()) and bool((dst_buf[dst_off + nbytes:] == 0xAB).all())


def test_penalties_and_token_counts_match_the_restatement():
    torch.manual_seed(5)
    rows, V = 37, 152064
    logits = torch.randn(rows, V + 64, device=DEV)[:, :V]            # a strided view, as the padded lm_head gives
    counts = torch.zeros(rows, V, device=DEV, dtype=torch.int32)
    idx = torch.randint(0, V, (rows, 50), device=DEV)
    counts.scatter_add_(1, idx, torch.ones_like(idx, dtype=torch.int32))
    freq = torch.rand(rows, device=DEV) * 2
    pres = torch.rand(rows, device=DEV) * 3
    freq[3] = pres[3] = 0.0
    want = ops.apply_penalties_(logits.cpu().clone(), counts.cpu(), freq.cpu(), pres.cpu())
    got = ops.apply_penalties_(logits, counts, freq, pres)
    torch.testing.assert_close(got.cpu(), want, rtol=1e-6, atol=1e-6)
    toks = torch.randint(0, V, (rows,), device=DEV, dtype=torch.int32)
    active = (torch.arange(rows, device=DEV) % 3 != 0).to(torch.int32)
    want_c = ops.count_tokens_(counts.cpu().clone(), toks.cpu(), active.cpu())
    ops.count_tokens_(counts, toks, active)
    assert torch.equal(counts.cpu(), want_c)
