"""Generator models against plain PyTorch restatements of the published architectures.

The restatements below follow the checkpoint's own conventions (interleaved-pair complex rotary embedding,
separate q/k/v projections, NCHW convolutions), so they also check the weight re-layouts done at load time.
They run on CPU (ops -> fp32 reference path) and, marked ``gpu``, on the CUDA kernels.
"""

import base64
import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

from cornserve.models.qwen_image import (QwenImageDiT, QwenImageDiTConfig, QwenImageModel, QwenImagePipelineConfig,
                                              flow_match_sigmas, pack_latents, timestep_embedding, unpack_latents)
from cornserve.models.qwen_image_vae import QwenImageVAEConfig, QwenImageVAEDecoder

DEVICES = ["cpu", pytest.param("cuda", marks=pytest.mark.gpu)]


# ------------------------------------------------------------------------------------------------
# MMDiT
# ------------------------------------------------------------------------------------------------
def dit_weights(cfg: QwenImageDiTConfig, seed=0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    D, J = cfg.inner_dim, cfg.joint_attention_dim
    r = lambda *s, std=0.05: (torch.randn(*s, generator=g) * std).bfloat16()  # noqa: E731
    w = {"txt_norm.weight": 1 + r(J), "img_in.weight": r(D, cfg.in_channels, std=0.2), "img_in.bias": r(D),
         "txt_in.weight": r(D, J, std=0.1), "txt_in.bias": r(D),
         "time_text_embed.timestep_embedder.linear_1.weight": r(D, 256), "time_text_embed.timestep_embedder.linear_1.bias": r(D),
         "time_text_embed.timestep_embedder.linear_2.weight": r(D, D), "time_text_embed.timestep_embedder.linear_2.bias": r(D),
         "norm_out.linear.weight": r(2 * D, D), "norm_out.linear.bias": r(2 * D),
         "proj_out.weight": r(cfg.patch_size ** 2 * cfg.out_channels, D), "proj_out.bias": r(cfg.patch_size ** 2 * cfg.out_channels)}
    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}."
        for s in ("img", "txt"):
            w[p + f"{s}_mod.1.weight"], w[p + f"{s}_mod.1.bias"] = r(6 * D, D), r(6 * D, std=0.2)
            w[p + f"{s}_mlp.net.0.proj.weight"], w[p + f"{s}_mlp.net.0.proj.bias"] = r(4 * D, D), r(4 * D)
            w[p + f"{s}_mlp.net.2.weight"], w[p + f"{s}_mlp.net.2.bias"] = r(D, 4 * D), r(D)
        for n in ("to_q", "to_k", "to_v", "add_q_proj", "add_k_proj", "add_v_proj", "to_out.0", "to_add_out"):
            w[p + f"attn.{n}.weight"], w[p + f"attn.{n}.bias"] = r(D, D, std=0.1), r(D)
        for n in ("norm_q", "norm_k", "norm_added_q", "norm_added_k"):
            w[p + f"attn.{n}.weight"] = 1 + r(cfg.attention_head_dim, std=0.2)
    return w


def rope_complex(cfg, h, w, n_txt):
    """Complex rotary factors as the checkpoint defines them: [tokens, d/2]."""
    def fr(pos, dim):
        inv = 1.0 / (cfg.rope_theta ** (torch.arange(0, dim, 2, dtype=torch.float64) / dim))
        return torch.outer(pos.double(), inv)
    a0, a1, a2 = cfg.axes_dims_rope
    hh = torch.cat([torch.arange(-(h - h // 2), 0), torch.arange(0, h // 2)])
    ww = torch.cat([torch.arange(-(w - w // 2), 0), torch.arange(0, w // 2)])
    img = torch.cat([fr(torch.zeros(1), a0)[:, None, None].expand(1, h, w, -1).reshape(h * w, -1),
                     fr(hh, a1)[:, None].expand(h, w, -1).reshape(h * w, -1),
                     fr(ww, a2)[None].expand(h, w, -1).reshape(h * w, -1)], dim=-1)
    tp = torch.arange(max(h // 2, w // 2), max(h // 2, w // 2) + n_txt)
    txt = torch.cat([fr(tp, a) for a in cfg.axes_dims_rope], dim=-1)
    return torch.polar(torch.ones_like(img), img), torch.polar(torch.ones_like(txt), txt)


def dit_reference(cfg, w, latents, prompt, t, h, wd):
    """fp32 restatement: latents [B, n_img, C], prompt [B, n_txt, J], t [B]."""
    W = {k: v.float() for k, v in w.items()}
    D, H, d = cfg.inner_dim, cfg.num_attention_heads, cfg.attention_head_dim
    B, n_img, _ = latents.shape
    n_txt = prompt.shape[1]
    lin = lambda x, n: F.linear(x, W[n + ".weight"], W.get(n + ".bias"))  # noqa: E731
    rms = lambda x, wt: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * wt  # noqa: E731
    temb = lin(F.silu(lin(timestep_embedding(t, 256), "time_text_embed.timestep_embedder.linear_1")),
               "time_text_embed.timestep_embedder.linear_2")
    img = lin(latents.float(), "img_in")
    txt = lin(rms(prompt.float(), W["txt_norm.weight"]), "txt_in")
    f_img, f_txt = rope_complex(cfg, h, wd, n_txt)

    def rot(x, f):  # x [B, T, H, d]
        xc = torch.view_as_complex(x.double().reshape(*x.shape[:-1], -1, 2))
        return torch.view_as_real(xc * f[None, :, None, :]).flatten(3).float()

    for i in range(cfg.num_layers):
        p = f"transformer_blocks.{i}."
        mi = lin(F.silu(temb), p + "img_mod.1")
        mt = lin(F.silu(temb), p + "txt_mod.1")

        def modulate(x, m):
            sh, sc, g = m.chunk(3, dim=-1)
            return F.layer_norm(x, (D,), eps=1e-6) * (1 + sc[:, None]) + sh[:, None], g[:, None]

        xi, gi1 = modulate(img, mi[:, :3 * D])
        xt, gt1 = modulate(txt, mt[:, :3 * D])
        hv = lambda x: x.view(B, -1, H, d)  # noqa: E731
        qi, ki, vi = hv(lin(xi, p + "attn.to_q")), hv(lin(xi, p + "attn.to_k")), hv(lin(xi, p + "attn.to_v"))
        qt, kt, vt = hv(lin(xt, p + "attn.add_q_proj")), hv(lin(xt, p + "attn.add_k_proj")), hv(lin(xt, p + "attn.add_v_proj"))
        qi, ki = rot(rms(qi, W[p + "attn.norm_q.weight"]), f_img), rot(rms(ki, W[p + "attn.norm_k.weight"]), f_img)
        qt, kt = rot(rms(qt, W[p + "attn.norm_added_q.weight"]), f_txt), rot(rms(kt, W[p + "attn.norm_added_k.weight"]), f_txt)
        q, k, v = torch.cat([qt, qi], 1), torch.cat([kt, ki], 1), torch.cat([vt, vi], 1)
        a = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
        a = a.reshape(B, n_txt + n_img, D)
        img = img + gi1 * lin(a[:, n_txt:], p + "attn.to_out.0")
        txt = txt + gt1 * lin(a[:, :n_txt], p + "attn.to_add_out")
        xi, gi2 = modulate(img, mi[:, 3 * D:])
        xt, gt2 = modulate(txt, mt[:, 3 * D:])
        img = img + gi2 * lin(F.gelu(lin(xi, p + "img_mlp.net.0.proj"), approximate="tanh"), p + "img_mlp.net.2")
        txt = txt + gt2 * lin(F.gelu(lin(xt, p + "txt_mlp.net.0.proj"), approximate="tanh"), p + "txt_mlp.net.2")
    sc, sh = lin(F.silu(temb), "norm_out.linear").chunk(2, dim=-1)
    x = F.layer_norm(img, (D,), eps=1e-6) * (1 + sc[:, None]) + sh[:, None]
    return lin(x, "proj_out")


TINY_DIT = QwenImageDiTConfig(in_channels=16, out_channels=4, num_layers=2, attention_head_dim=64, num_attention_heads=2,
                              joint_attention_dim=64, axes_dims_rope=(8, 28, 28))


@pytest.mark.parametrize("device", DEVICES)
def test_dit_matches_restatement(device):
    cfg = TINY_DIT
    w = dit_weights(cfg)
    model = QwenImageDiT(cfg, device=device)
    assert model.load_weights(w.items()) == set(w)
    B, h, wd, n_txt = 2, 4, 6, 8
    g = torch.Generator().manual_seed(1)
    lat = torch.randn(B, h * wd, cfg.in_channels, generator=g).bfloat16()
    prompt = torch.randn(B, n_txt, cfg.joint_attention_dim, generator=g).bfloat16()
    t = torch.tensor([0.9, 0.3])
    want = dit_reference(cfg, w, lat, prompt, t, h, wd)
    lay = model.make_layout(B, [n_txt] * B, n_txt, (h, wd))
    got = model(lat.reshape(B * h * wd, -1).to(device), prompt.reshape(B * n_txt, -1).to(device), t.to(device), lay)
    got = got.float().cpu().view(B, h * wd, -1)
    cos = F.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    assert cos > 0.995, cos
    assert (got - want).abs().max().item() < 0.08 * want.abs().max().item() + 0.02


@pytest.mark.parametrize("device", DEVICES)
def test_dit_masks_padded_prompt_rows(device):
    """A shorter prompt in a padded batch gives the same result as running it alone."""
    cfg = TINY_DIT
    model = QwenImageDiT(cfg, device=device)
    model.load_weights(dit_weights(cfg).items())
    h, wd = 4, 4
    g = torch.Generator().manual_seed(2)
    lat = torch.randn(2, h * wd, cfg.in_channels, generator=g).bfloat16().to(device)
    prompt = torch.randn(2, 8, cfg.joint_attention_dim, generator=g).bfloat16().to(device)
    t = torch.tensor([0.5, 0.5], device=device)
    lay = model.make_layout(2, [8, 5], 8, (h, wd))
    both = model(lat.reshape(-1, cfg.in_channels), prompt.reshape(-1, cfg.joint_attention_dim), t, lay).view(2, h * wd, -1)
    lay1 = model.make_layout(1, [5], 5, (h, wd))
    alone = model(lat[1].contiguous(), prompt[1, :5].contiguous(), t[1:], lay1)
    assert torch.allclose(both[1].float(), alone.float(), atol=3e-2, rtol=3e-2)


def test_sigmas_and_packing():
    s = flow_match_sigmas(50, 4096)
    assert s.shape == (51,) and s[0] == pytest.approx(1.0) and s[-1] == 0.0 and np.all(np.diff(s) < 0)
    assert s[-2] == pytest.approx(0.02, abs=1e-6)
    x = torch.randn(2, 16, 8, 12)
    assert torch.equal(unpack_latents(pack_latents(x), 4, 6), x)


# ------------------------------------------------------------------------------------------------
# VAE decoder
# ------------------------------------------------------------------------------------------------
def vae_weights(cfg: QwenImageVAEConfig, seed=0) -> dict[str, torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    mult = list(cfg.dim_mult)
    dims = [cfg.base_dim * u for u in [mult[-1]] + mult[::-1]]
    w: dict[str, torch.Tensor] = {}

    def conv3d(name, cin, cout, k=3):
        w[name + ".weight"] = (torch.randn(cout, cin, k, k, k, generator=g) / math.sqrt(cin * k * k)).bfloat16()
        w[name + ".bias"] = (torch.randn(cout, generator=g) * 0.05).bfloat16()

    def conv2d(name, cin, cout, k):
        w[name + ".weight"] = (torch.randn(cout, cin, k, k, generator=g) / math.sqrt(cin * k * k)).bfloat16()
        w[name + ".bias"] = (torch.randn(cout, generator=g) * 0.05).bfloat16()

    def gamma(name, dim, nd):
        w[name + ".gamma"] = (1 + 0.2 * torch.randn(dim, *([1] * nd), generator=g)).bfloat16()

    def res(name, cin, cout):
        gamma(name + ".norm1", cin, 3); conv3d(name + ".conv1", cin, cout)
        gamma(name + ".norm2", cout, 3); conv3d(name + ".conv2", cout, cout)
        if cin != cout:
            conv3d(name + ".conv_shortcut", cin, cout, 1)

    conv3d("post_quant_conv", cfg.z_dim, cfg.z_dim, 1)
    conv3d("decoder.conv_in", cfg.z_dim, dims[0])
    res("decoder.mid_block.resnets.0", dims[0], dims[0]); res("decoder.mid_block.resnets.1", dims[0], dims[0])
    gamma("decoder.mid_block.attentions.0.norm", dims[0], 2)
    conv2d("decoder.mid_block.attentions.0.to_qkv", dims[0], 3 * dims[0], 1)
    conv2d("decoder.mid_block.attentions.0.proj", dims[0], dims[0], 1)
    for i, (cin, cout) in enumerate(zip(dims[:-1], dims[1:])):
        if i > 0:
            cin //= 2
        for j in range(cfg.num_res_blocks + 1):
            res(f"decoder.up_blocks.{i}.resnets.{j}", cin if j == 0 else cout, cout)
        if i != len(mult) - 1:
            conv2d(f"decoder.up_blocks.{i}.upsamplers.0.resample.1", cout, cout // 2, 3)
    gamma("decoder.norm_out", dims[-1], 3)
    conv3d("decoder.conv_out", dims[-1], 3)
    return w


def vae_reference(cfg, w, latents):
    W = {k: v.float() for k, v in w.items()}
    mult = list(cfg.dim_mult)
    dims = [cfg.base_dim * u for u in [mult[-1]] + mult[::-1]]

    def conv(x, name):
        wt = W[name + ".weight"]
        if wt.dim() == 5:
            # one frame through a causal 3-D convolution: two zero frames are padded in front
            k = wt.shape[2]
            x5 = F.pad(x[:, :, None], (wt.shape[4] // 2,) * 2 + (wt.shape[3] // 2,) * 2 + (k - 1, 0))
            return F.conv3d(x5, wt, W[name + ".bias"])[:, :, 0]
        return F.conv2d(x, wt, W[name + ".bias"], padding=wt.shape[-1] // 2)

    def norm(x, name):
        return F.normalize(x, dim=1) * x.shape[1] ** 0.5 * W[name + ".gamma"].reshape(1, -1, 1, 1)

    def res(x, name):
        h = conv(x, name + ".conv_shortcut") if name + ".conv_shortcut.weight" in W else x
        y = conv(F.silu(norm(x, name + ".norm1")), name + ".conv1")
        return conv(F.silu(norm(y, name + ".norm2")), name + ".conv2") + h

    mean = torch.tensor(cfg.latents_mean).view(1, -1, 1, 1)
    std = torch.tensor(cfg.latents_std).view(1, -1, 1, 1)
    x = conv(latents.float() * std + mean, "post_quant_conv")
    x = conv(x, "decoder.conv_in")
    x = res(x, "decoder.mid_block.resnets.0")
    a = "decoder.mid_block.attentions.0"
    B, C, H, Wd = x.shape
    qkv = conv(norm(x, a + ".norm"), a + ".to_qkv").reshape(B, 1, 3 * C, H * Wd).permute(0, 1, 3, 2)
    q, k, v = qkv.chunk(3, dim=-1)
    o = F.scaled_dot_product_attention(q, k, v).squeeze(1).permute(0, 2, 1).reshape(B, C, H, Wd)
    x = x + conv(o, a + ".proj")
    x = res(x, "decoder.mid_block.resnets.1")
    for i in range(len(dims) - 1):
        for j in range(cfg.num_res_blocks + 1):
            x = res(x, f"decoder.up_blocks.{i}.resnets.{j}")
        if i != len(mult) - 1:
            x = F.interpolate(x, scale_factor=2.0, mode="nearest-exact")
            x = conv(x, f"decoder.up_blocks.{i}.upsamplers.0.resample.1")
    x = conv(F.silu(norm(x, "decoder.norm_out")), "decoder.conv_out")
    return x.clamp(-1, 1)


TINY_VAE = QwenImageVAEConfig(base_dim=16, z_dim=16, dim_mult=(1, 2, 4, 4), num_res_blocks=1)


@pytest.mark.parametrize("device", DEVICES)
def test_vae_decoder_matches_restatement(device):
    cfg = TINY_VAE
    w = vae_weights(cfg)
    vae = QwenImageVAEDecoder(cfg, device=device)
    assert vae.load_weights(w.items()) == set(w)
    lat = torch.randn(2, 16, 4, 6, generator=torch.Generator().manual_seed(3)) * 0.5
    want = vae_reference(cfg, w, lat)  # [B, 3, 32, 48]
    rgb = vae.decode_to_rgb8(lat.to(device)).cpu()
    assert rgb.shape == (2, 32, 48, 3) and rgb.dtype == torch.uint8
    want8 = ((want.permute(0, 2, 3, 1) * 0.5 + 0.5).clamp(0, 1) * 255).round()
    err = (rgb.float() - want8).abs()
    assert err.mean().item() < 3.0 and (err > 16).float().mean().item() < 0.01, (err.mean().item(), err.max().item())


# ------------------------------------------------------------------------------------------------
# pipeline
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("device", DEVICES)
def test_pipeline_generates_png(device):
    dit = QwenImageDiTConfig(in_channels=64, out_channels=16, num_layers=1, attention_head_dim=64, num_attention_heads=2,
                             joint_attention_dim=64, axes_dims_rope=(8, 28, 28))
    cfg = QwenImagePipelineConfig(dit=dit, vae=TINY_VAE)
    model = QwenImageModel(cfg, device=device, seed=7)
    emb = [torch.randn(6, cfg.dit.joint_attention_dim).bfloat16(), torch.randn(6, cfg.dit.joint_attention_dim).bfloat16()]
    neg = [torch.zeros_like(e) for e in emb]
    out = model.generate(emb, 64, 32, num_inference_steps=2, negative_embeds=neg, true_cfg_scale=4.0)
    assert len(out) == 2
    png = base64.b64decode(out[0])
    assert png[:8] == b"\x89PNG\r\n\x1a\n"
    from PIL import Image
    import io

    im = Image.open(io.BytesIO(png))
    assert im.size == (32, 64)


# ------------------------------------------------------------------------------------------------
# code-to-waveform vocoder against the Hugging Face module
# ------------------------------------------------------------------------------------------------
def _hf_code2wav(seed=0):
    from transformers.models.qwen3_omni_moe.configuration_qwen3_omni_moe import Qwen3OmniMoeCode2WavConfig
    from transformers.models.qwen3_omni_moe.modeling_qwen3_omni_moe import Qwen3OmniMoeCode2Wav

    hf_cfg = Qwen3OmniMoeCode2WavConfig(codebook_size=32, hidden_size=64, num_attention_heads=2, num_key_value_heads=2,
                                        sliding_window=6, intermediate_size=128, num_hidden_layers=2, num_quantizers=4,
                                        upsample_rates=(3, 2, 2, 2), upsampling_ratios=(2, 2), decoder_dim=128)
    hf_cfg._attn_implementation = "eager"
    torch.manual_seed(seed)
    hf = Qwen3OmniMoeCode2Wav(hf_cfg).float().eval()
    with torch.no_grad():
        for n, p in hf.named_parameters():
            if n.endswith("alpha") or n.endswith("beta"):
                p.copy_(torch.randn_like(p) * 0.3)
            elif n.endswith("gamma") or "layer_scale" in n:
                p.copy_(torch.rand_like(p) * 0.5 + 0.25)
            elif p.dim() >= 2:
                p.copy_(torch.randn_like(p) * (0.5 / math.sqrt(p[0].numel())))
            elif "norm" in n and n.endswith("weight"):
                p.copy_(1 + 0.1 * torch.randn_like(p))
            else:
                p.copy_(torch.randn_like(p) * 0.05)
            p.copy_(p.bfloat16().float())
    return hf, hf_cfg


@pytest.mark.parametrize("device", DEVICES)
def test_code2wav_matches_hf(device):
    from cornserve.models.code2wav import Code2Wav, Code2WavConfig

    hf, hf_cfg = _hf_code2wav()
    cfg = Code2WavConfig.from_hf(hf_cfg.to_dict())
    model = Code2Wav(cfg, device=device)
    sd = hf.state_dict()
    loaded = model.load_weights((k, v.bfloat16()) for k, v in sd.items())
    missing = set(sd) - loaded
    assert not missing, sorted(missing)[:10]
    codes = torch.randint(0, hf_cfg.codebook_size, (2, hf_cfg.num_quantizers, 11), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        want = hf(codes)[:, 0]
    got = model(codes).float().cpu()
    assert got.shape == want.shape == (2, model.output_length(11))
    cos = F.cosine_similarity(got.flatten(), want.flatten(), dim=0).item()
    assert cos > 0.98, cos
    # chunked streaming decode agrees with the module's own chunked decode
    with torch.no_grad():
        want_chunks = hf.chunked_decode(codes, chunk_size=4, left_context_size=2)[:, 0]
    pieces = [[], []]
    for out in model.generate([codes[0], codes[1, :, :7]], chunk_size=4, left_context_size=2):
        for i, o in enumerate(out):
            if o is not None:
                pieces[i].append(o.float().cpu())
    full = torch.cat(pieces[0])
    assert full.shape[0] == want_chunks.shape[1]
    assert F.cosine_similarity(full, want_chunks[0], dim=0).item() > 0.98
    assert len(pieces[1]) == 2  # the shorter request ends early


@pytest.mark.parametrize("device", DEVICES)
def test_batched_cfg_matches_two_passes(device):
    """Conditional and unconditional samples in one batch of 2B give the latents of two separate denoiser calls,
    also when the negative prompt is shorter (padded text rows are masked out of the joint attention)."""
    dit = QwenImageDiTConfig(in_channels=64, out_channels=16, num_layers=2, attention_head_dim=64, num_attention_heads=2,
                             joint_attention_dim=64, axes_dims_rope=(8, 28, 28))
    cfg = QwenImagePipelineConfig(dit=dit, vae=TINY_VAE)
    model = QwenImageModel(cfg, device=device, seed=3)
    g = torch.Generator().manual_seed(5)
    emb = [torch.randn(6, 64, generator=g).bfloat16(), torch.randn(4, 64, generator=g).bfloat16()]
    neg = [torch.randn(2, 64, generator=g).bfloat16(), torch.randn(6, 64, generator=g).bfloat16()]
    one = model.denoise(emb, 64, 32, 3, negative_embeds=neg, true_cfg_scale=3.0, batch_cfg=True).float().cpu()
    two = model.denoise(emb, 64, 32, 3, negative_embeds=neg, true_cfg_scale=3.0, batch_cfg=False).float().cpu()
    tol = 1e-4 if device == "cpu" else 0.06
    assert (one - two).abs().max().item() <= tol * max(1.0, two.abs().max().item())
