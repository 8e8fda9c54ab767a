"""Plain PyTorch fp32 restatements of every op in ``cornserve.ops``.

They are the numerics oracle for the CUDA kernels and the execution path for CPU tensors
(CPU-only plumbing runs and unit tests).  Inputs of any float dtype are computed in fp32 and
cast back to the input dtype.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F

ACTS = {"none": 0, "gelu": 1, "gelu_tanh": 2, "silu": 3, "quick_gelu": 4, "relu": 5}


def act_fn(x: torch.Tensor, act: str | None) -> torch.Tensor:
    if act in (None, "none"):
        return x
    if act == "gelu":
        return F.gelu(x)
    if act == "gelu_tanh":
        return F.gelu(x, approximate="tanh")
    if act == "silu":
        return F.silu(x)
    if act == "quick_gelu":
        return x * torch.sigmoid(1.702 * x)
    if act == "relu":
        return F.relu(x)
    raise ValueError(f"unknown activation {act}")


def linear(x, w, bias=None, act=None, residual=None, gate=None, gate_rows_per_batch=1, out_dtype=None):
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    y = act_fn(y, act)
    if gate is not None:
        g = gate.float().repeat_interleave(gate_rows_per_batch, dim=0)[: y.shape[0]]
        y = y * g
    if residual is not None:
        y = y + residual.float()
    return y.to(out_dtype or x.dtype)


def swiglu_linear(x, w, bias=None, act="silu"):
    n = w.shape[0] // 2
    y = x.float() @ w.float().t()
    if bias is not None:
        y = y + bias.float()
    return (act_fn(y[:, :n], act) * y[:, n:]).to(x.dtype)


def rms_norm(x, w, eps, residual=None, gemma=False):
    xf = x.float()
    new_res = None
    if residual is not None:
        new_res = (xf + residual.float()).to(x.dtype)
        xf = new_res.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if w is not None:
        y = y * ((1.0 + w.float()) if gemma else w.float())
    y = y.to(x.dtype)
    return (y, new_res) if residual is not None else y


def layer_norm(x, w, b, eps, scale=None, shift=None, rows_per_batch=1, residual=None):
    xf = x.float()
    new_res = None
    if residual is not None:
        new_res = (xf + residual.float()).to(x.dtype)
        xf = new_res.float()
    y = F.layer_norm(xf, (x.shape[-1],), None if w is None else w.float(), None if b is None else b.float(), eps)
    if scale is not None:
        sc = scale.float().repeat_interleave(rows_per_batch, dim=0)[: y.shape[0]]
        sh = shift.float().repeat_interleave(rows_per_batch, dim=0)[: y.shape[0]]
        y = y * (1.0 + sc) + sh
    y = y.to(x.dtype)
    return (y, new_res) if residual is not None else y


def rope(x, cs, rot=None):
    """x: [T, heads, d]; cs: [T, 2, rot/2] (cos, sin).  Rotate-half convention; returns a new tensor."""
    d = x.shape[-1]
    rot = rot or d
    half = rot // 2
    cos = cs[:, 0].float()[:, None, :]
    sin = cs[:, 1].float()[:, None, :]
    xf = x.float()
    a, b = xf[..., :half], xf[..., half:rot]
    out = xf.clone()
    out[..., :half] = a * cos - b * sin
    out[..., half:rot] = b * cos + a * sin
    return out.to(x.dtype)


def mrope_table(positions, half, theta, sections):
    """positions: [3, T] int; returns [T, 2, half] fp32 with the section-wise choice of position row."""
    T = positions.shape[1]
    i = torch.arange(half, dtype=torch.float32, device=positions.device)
    inv = theta ** (-(2.0 * i) / (2.0 * half))
    which = torch.zeros(half, dtype=torch.long, device=positions.device)
    which[sections[0]: sections[0] + sections[1]] = 1
    which[sections[0] + sections[1]:] = 2
    pos = positions.float()[which, :].t()  # [T, half]
    ang = pos * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], dim=1).contiguous().view(T, 2, half)


def attention_varlen(q, k, v, cu_q, cu_k, scale, causal=False, window=0):
    """q: [Tq, Hq, d]; k, v: [Tk, Hkv, d]; packed sequences; returns [Tq, Hq, d]."""
    Hq, Hkv = q.shape[1], k.shape[1]
    rep = Hq // Hkv
    out = torch.zeros_like(q, dtype=torch.float32)
    cu_q = cu_q.tolist()
    cu_k = cu_k.tolist()
    for s in range(len(cu_q) - 1):
        qs = q[cu_q[s]: cu_q[s + 1]].float().transpose(0, 1)  # [Hq, Lq, d]
        ks = k[cu_k[s]: cu_k[s + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vs = v[cu_k[s]: cu_k[s + 1]].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        Lq, Lk = qs.shape[1], ks.shape[1]
        if Lq == 0:
            continue
        if Lk == 0:
            continue
        sc = (qs @ ks.transpose(1, 2)) * scale
        if causal:
            qi = torch.arange(Lq, device=q.device)[:, None] + (Lk - Lq)
            kj = torch.arange(Lk, device=q.device)[None, :]
            sc = sc.masked_fill(kj > qi, float("-inf"))
            if window > 0:
                sc = sc.masked_fill(kj <= qi - window, float("-inf"))
        pr = torch.softmax(sc, dim=-1)
        pr = torch.nan_to_num(pr, nan=0.0)
        out[cu_q[s]: cu_q[s + 1]] = (pr @ vs).transpose(0, 1)
    return out.to(q.dtype)


def gather_paged_kv(cache, block_table, kv_len, seq):
    """cache: [pages, 2, Hkv, page, d] -> (k, v) of shape [kv_len, Hkv, d] for sequence `seq`."""
    page = cache.shape[3]
    n = int(kv_len[seq])
    nblk = (n + page - 1) // page
    ids = block_table[seq, :nblk].long()
    k = cache[ids, 0].permute(0, 2, 1, 3).reshape(-1, cache.shape[2], cache.shape[4])[:n]
    v = cache[ids, 1].permute(0, 2, 1, 3).reshape(-1, cache.shape[2], cache.shape[4])[:n]
    return k, v


def attention_paged(q, cache, block_table, kv_len, cu_q, scale, causal=True):
    out = torch.zeros_like(q, dtype=torch.float32)
    cu = cu_q.tolist()
    for s in range(len(cu) - 1):
        if cu[s + 1] == cu[s]:
            continue
        k, v = gather_paged_kv(cache, block_table, kv_len, s)
        qq = q[cu[s]: cu[s + 1]]
        o = attention_varlen(
            qq, k, v,
            torch.tensor([0, qq.shape[0]]), torch.tensor([0, k.shape[0]]), scale, causal,
        )
        out[cu[s]: cu[s + 1]] = o.float()
    return out.to(q.dtype)


def rope_kv_write(qkv, Hq, Hkv, d, cs, cache, slot, page):
    """Returns rotated q [T, Hq, d] and writes rotated k / plain v into the paged cache (in place)."""
    T = qkv.shape[0]
    q = qkv[:, : Hq * d].reshape(T, Hq, d)
    k = qkv[:, Hq * d: (Hq + Hkv) * d].reshape(T, Hkv, d)
    v = qkv[:, (Hq + Hkv) * d:].reshape(T, Hkv, d)
    q = rope(q, cs)
    k = rope(k, cs)
    slot = slot.long()
    ok = slot >= 0
    pg = torch.div(slot[ok], page, rounding_mode="floor")
    off = slot[ok] % page
    cache[pg, 0, :, off] = k[ok].to(cache.dtype)
    cache[pg, 1, :, off] = v[ok].to(cache.dtype)
    return q


def act_mul(gu, act="silu"):
    n = gu.shape[-1] // 2
    return (act_fn(gu[..., :n].float(), act) * gu[..., n:].float()).to(gu.dtype)


def argmax(logits):
    return logits.float().argmax(dim=-1).to(torch.int32)


_M64 = (1 << 64) - 1


def _mix64(z: int) -> int:
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M64
    return z ^ (z >> 31)


def sample_kept_mask(logits_row, temperature: float, top_p: float, top_k: int):
    """Which tokens of one row survive top-k then top-p (ties at a cut-off are kept), and their weights
    (probabilities relative to the maximum, in 2^-36 fixed point, as the CUDA kernel counts them)."""
    import numpy as np

    x = logits_row.detach().float().cpu().numpy()
    V = x.shape[0]
    mx = np.float32(x.max())
    inv = np.float32(1.4426950408889634) / np.float32(temperature)
    w = np.floor(np.exp2((x - mx) * inv, dtype=np.float32).astype(np.float64) * float(1 << 36)).astype(np.uint64)
    keep = np.ones(V, dtype=bool)
    if 0 < top_k < V:
        keep &= x >= np.sort(x)[V - top_k]
    if 0.0 < top_p < 1.0:
        idx = np.nonzero(keep)[0]
        order = idx[np.argsort(-x[idx], kind="stable")]
        cum = np.cumsum(w[order], dtype=np.uint64)
        target = max(1, int(float(int(cum[-1])) * float(np.float32(top_p))))
        pos = int(np.searchsorted(cum, np.uint64(target), side="left"))   # first prefix whose weight reaches the target
        keep &= x >= x[order[min(pos, len(order) - 1)]]
    return keep, w


def sample_rows(logits, temperature, top_p, top_k, seed, draws):
    """Temperature / top-k / top-p sampling of one token per row; ``draws`` (int32, the index of this draw in every
    row's random stream) is advanced in place.  Rows with ``temperature <= 0`` take the arg-max."""
    import numpy as np

    rows = logits.shape[0]
    out = torch.empty(rows, dtype=torch.int32)
    for r in range(rows):
        t = float(temperature[r])
        d = int(draws[r])
        draws[r] = d + 1
        if not t > 0.0:
            out[r] = int(logits[r].float().argmax())
            continue
        keep, w = sample_kept_mask(logits[r], t, float(top_p[r]), int(top_k[r]))
        cum = np.cumsum(np.where(keep, w, np.uint64(0)), dtype=np.uint64)
        total = int(cum[-1])
        rnd = _mix64(_mix64(int(seed[r]) & _M64) ^ ((0x9E3779B97F4A7C15 * (d + 1)) & _M64))
        target = (rnd * total) >> 64
        out[r] = min(int(np.searchsorted(cum, np.uint64(target), side="right")), logits.shape[1] - 1)
    return out.to(logits.device)


def flow_step(x, cond, uncond, cfg, dt, norm_rescale=False):
    c = cond.float()
    v = c
    if uncond is not None:
        u = uncond.float()
        v = u + cfg * (c - u)
        if norm_rescale:
            nc = c.norm(dim=-1, keepdim=True)
            nv = v.norm(dim=-1, keepdim=True).clamp_min(1e-12)
            v = v * (nc / nv)
    return x + dt * v


def pcm16(x):
    return (x.float().clamp(-1, 1) * 32767.0).round().to(torch.int16)


def softmax_scale(d: int) -> float:
    return 1.0 / math.sqrt(d)


def head_norm_rope(x, w, eps, cs):
    """x: [T, heads, d]; per-head RMSNorm with weight ``w`` [d] (or None), then rotate-half RoPE (or None)."""
    y = x
    if w is not None:
        y = rms_norm(y, w, eps)
    if cs is not None:
        y = rope(y, cs)
    return y


def softmax_rows(x, scale=1.0):
    return torch.softmax(x.float() * scale, dim=-1).to(x.dtype)


def im2col3x3(x, B, H, W, up=1, silu=False, stride=1):
    """x: [B*H*W, C] channels-last -> [B*Ho*Wo, 9*C] (tap-major: ky, kx, c), zero padding 1."""
    C = x.shape[-1]
    img = x.float().view(B, H, W, C)
    if silu:
        img = F.silu(img)
    if up == 2:
        img = img.repeat_interleave(2, dim=1).repeat_interleave(2, dim=2)
    Hu, Wu = H * up, W * up
    p = F.pad(img, (0, 0, 1, 1, 1, 1))
    taps = [p[:, ky: ky + Hu: stride, kx: kx + Wu: stride, :] for ky in range(3) for kx in range(3)]
    out = torch.stack(taps, dim=3)
    return out.reshape(-1, 9 * C).to(x.dtype)


def snake_beta(x, alpha, beta):
    a, b = alpha.float().exp(), beta.float().exp()
    xf = x.float()
    return xf + torch.sin(xf * a).pow(2) / (b + 1e-9)


def im2col1d(x, B, T, To, taps, first, dilation, alpha=None, beta=None, stride=1):
    """x: [B*T, C] -> [B*To, taps*C]; row t, tap j reads time ``t + first + j*dilation`` (zero outside)."""
    C = x.shape[-1]
    xf = x.float().view(B, T, C)
    if alpha is not None:
        xf = snake_beta(xf, alpha, beta)
    out = torch.zeros(B, To, taps, C, dtype=torch.float32, device=x.device)
    t = torch.arange(To, device=x.device)
    for j in range(taps):
        ts = t * stride + first + j * dilation
        ok = (ts >= 0) & (ts < T)
        out[:, ok, j, :] = xf[:, ts[ok], :]
    return out.reshape(B * To, taps * C).to(x.dtype)


def dwconv1d(x, w, bias, B, T):
    """Depth-wise causal conv: x [B*T, C], w [C, k]."""
    C, k = w.shape
    xf = x.float().view(B, T, C).transpose(1, 2)
    y = F.conv1d(F.pad(xf, (k - 1, 0)), w.float().unsqueeze(1), None if bias is None else bias.float(), groups=C)
    return y.transpose(1, 2).reshape(B * T, C).to(x.dtype)


def to_rgb8(x):
    v = (x[..., :3].float() * 0.5 + 0.5).clamp(0, 1)
    return (v * 255.0).round().to(torch.uint8)
