"""Resolving a model id to a local directory and reading Hugging Face checkpoints.

Checkpoint format = the Hugging Face layout, unchanged (reference loader:
python/cornserve/task_executors/utils.py:33-135): ``config.json``, ``model.safetensors`` or
``model.safetensors.index.json`` + shards, same tensor names.  There is no network here, so ids resolve
to (in order) an existing path, ``$CORNSERVE_MODEL_DIR/<id>``, the local HF cache, or a built-in
architecture table that yields the *configuration* of well-known models for random-weight runs.
"""

from __future__ import annotations

import json
import os
from collections.abc import Iterator
from pathlib import Path
from typing import Any

import torch

from ..logging import get_logger

logger = get_logger(__name__)

# Architecture-only configurations (no weights) for runs with random initialisation.
_QWEN25_VL_VISION = {"depth": 32, "hidden_size": 1280, "num_heads": 16, "intermediate_size": 3420, "patch_size": 14,
                     "temporal_patch_size": 2, "spatial_merge_size": 2, "window_size": 112,
                     "fullatt_block_indexes": [7, 15, 23, 31], "hidden_act": "silu", "in_channels": 3}
BUILTIN_CONFIGS: dict[str, dict[str, Any]] = {
    "Qwen/Qwen2.5-VL-7B-Instruct": {
        "model_type": "qwen2_5_vl", "hidden_size": 3584, "num_hidden_layers": 28, "num_attention_heads": 28,
        "num_key_value_heads": 4, "intermediate_size": 18944, "vocab_size": 152064, "rms_norm_eps": 1e-6,
        "rope_theta": 1000000.0, "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]},
        "tie_word_embeddings": False, "image_token_id": 151655, "video_token_id": 151656,
        "vision_start_token_id": 151652, "eos_token_id": 151645,
        "vision_config": {**_QWEN25_VL_VISION, "out_hidden_size": 3584},
    },
    "Qwen/Qwen2.5-VL-32B-Instruct": {
        "model_type": "qwen2_5_vl", "hidden_size": 5120, "num_hidden_layers": 64, "num_attention_heads": 40,
        "num_key_value_heads": 8, "intermediate_size": 27648, "vocab_size": 152064, "rms_norm_eps": 1e-6,
        "rope_theta": 1000000.0, "rope_scaling": {"type": "mrope", "mrope_section": [16, 24, 24]},
        "tie_word_embeddings": False, "image_token_id": 151655, "video_token_id": 151656,
        "vision_start_token_id": 151652, "eos_token_id": 151645,
        "vision_config": {**_QWEN25_VL_VISION, "out_hidden_size": 5120},
    },
    # tiny models for CPU plumbing runs and tests
    "cornserve-b200/tiny-vlm": {
        "model_type": "qwen2_5_vl", "hidden_size": 256, "num_hidden_layers": 2, "num_attention_heads": 4,
        "num_key_value_heads": 2, "intermediate_size": 512, "vocab_size": 1024, "rms_norm_eps": 1e-6,
        "rope_theta": 10000.0, "rope_scaling": {"type": "mrope", "mrope_section": [8, 12, 12]},
        "tie_word_embeddings": False, "image_token_id": 1000, "video_token_id": 1001,
        "vision_start_token_id": 1002, "eos_token_id": 1023, "torch_dtype": "float32",
        "vision_config": {"depth": 2, "hidden_size": 128, "num_heads": 4, "intermediate_size": 512, "patch_size": 14,
                          "temporal_patch_size": 2, "spatial_merge_size": 2, "window_size": 112,
                          "fullatt_block_indexes": [1], "out_hidden_size": 256, "hidden_act": "silu", "in_channels": 3},
    },
    "cornserve-b200/tiny-qwen2-vl": {"model_type": "qwen2_vl", "torch_dtype": "float32", "vision_config": {
        "depth": 1, "embed_dim": 64, "num_heads": 2, "hidden_size": 96, "mlp_ratio": 2}},
    "cornserve-b200/tiny-qwen3-vl": {"model_type": "qwen3_vl", "torch_dtype": "float32", "vision_config": {
        "depth": 2, "hidden_size": 64, "num_heads": 2, "intermediate_size": 128, "out_hidden_size": 96,
        "num_position_embeddings": 16, "deepstack_visual_indexes": [0], "patch_size": 16}},
    "cornserve-b200/tiny-qwen3-omni": {"model_type": "qwen3_omni_moe", "torch_dtype": "float32", "thinker_config": {
        "vision_config": {"depth": 1, "hidden_size": 64, "num_heads": 2, "intermediate_size": 128, "out_hidden_size": 96,
                          "num_position_embeddings": 16, "deepstack_visual_indexes": [0], "patch_size": 16},
        "audio_config": {"num_mel_bins": 128, "d_model": 64, "encoder_layers": 1, "encoder_attention_heads": 2,
                         "encoder_ffn_dim": 64, "max_source_positions": 200, "n_window": 50, "output_dim": 96,
                         "downsample_hidden_size": 8, "n_window_infer": 400}}},
    # thinker (MoE decoder + encoders) + talker + vocoder of a Qwen3-Omni-shaped model, small enough for CPU tests
    "cornserve-b200/tiny-omni": {
        "model_type": "qwen3_omni_moe", "torch_dtype": "float32", "tts_bos_token_id": 500, "tts_eos_token_id": 501,
        "tts_pad_token_id": 502,
        "thinker_config": {
            "text_config": {"model_type": "qwen3_omni_moe_text", "hidden_size": 128, "num_hidden_layers": 2, "num_attention_heads": 2,
                            "num_key_value_heads": 1, "head_dim": 64, "intermediate_size": 128, "vocab_size": 512, "num_experts": 4,
                            "num_experts_per_tok": 2, "moe_intermediate_size": 64, "rope_theta": 10000.0},
            "vision_config": {"depth": 1, "hidden_size": 64, "num_heads": 2, "intermediate_size": 128, "out_hidden_size": 128,
                              "num_position_embeddings": 16, "deepstack_visual_indexes": [0], "patch_size": 16},
            "audio_config": {"num_mel_bins": 128, "d_model": 64, "encoder_layers": 1, "encoder_attention_heads": 2,
                             "encoder_ffn_dim": 64, "max_source_positions": 200, "n_window": 50, "output_dim": 128,
                             "downsample_hidden_size": 8, "n_window_infer": 400}},
        "talker_config": {
            "thinker_hidden_size": 128, "accept_hidden_layer": 1, "num_code_groups": 4, "codec_eos_token_id": 70,
            "codec_nothink_id": 71, "codec_think_bos_id": 72, "codec_think_eos_id": 73, "codec_pad_id": 74, "codec_bos_id": 75,
            "speaker_id": {"ethan": 80},
            "text_config": {"vocab_size": 96, "hidden_size": 128, "intermediate_size": 64, "num_hidden_layers": 2,
                            "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 64, "moe_intermediate_size": 64,
                            "num_experts_per_tok": 2, "num_experts": 4, "shared_expert_intermediate_size": 64, "rope_theta": 10000.0},
            "code_predictor_config": {"vocab_size": 32, "hidden_size": 128, "intermediate_size": 128, "num_hidden_layers": 2,
                                      "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 64, "num_code_groups": 4,
                                      "rope_theta": 10000.0}},
        "code2wav_config": {"codebook_size": 32, "hidden_size": 64, "num_attention_heads": 2, "num_key_value_heads": 2,
                            "sliding_window": 6, "intermediate_size": 128, "num_hidden_layers": 2, "num_quantizers": 4,
                            "upsample_rates": [3, 2, 2, 2], "upsampling_ratios": [2, 2], "decoder_dim": 128}},
    "cornserve-b200/tiny-qwen2.5-omni": {"model_type": "qwen2_5_omni", "torch_dtype": "float32", "thinker_config": {
        "vision_config": {"depth": 1, "hidden_size": 64, "num_heads": 2, "intermediate_size": 128, "out_hidden_size": 96,
                          "fullatt_block_indexes": [0]},
        "audio_config": {"num_mel_bins": 128, "d_model": 64, "encoder_layers": 1, "encoder_attention_heads": 2,
                         "encoder_ffn_dim": 64, "max_source_positions": 200, "n_window": 50, "output_dim": 96}}},
    "cornserve-b200/tiny-gemma3": {"model_type": "gemma3", "torch_dtype": "float32", "mm_tokens_per_image": 4,
                                   "text_config": {"hidden_size": 256},
                                   "vision_config": {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 1,
                                                     "num_attention_heads": 2, "image_size": 56, "patch_size": 14}},
    "cornserve-b200/tiny-gemma3-large": {"model_type": "gemma3", "torch_dtype": "float32", "mm_tokens_per_image": 4,
                                         "text_config": {"hidden_size": 512},
                                         "vision_config": {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 1,
                                                           "num_attention_heads": 2, "image_size": 56, "patch_size": 14}},
    "cornserve-b200/tiny-llava-onevision": {"model_type": "llava_onevision", "torch_dtype": "float32",
                                            "text_config": {"hidden_size": 96},
                                            "image_grid_pinpoints": [[56, 56], [56, 112], [112, 56], [112, 112]],
                                            "vision_config": {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
                                                              "num_attention_heads": 2, "image_size": 56, "patch_size": 14}},
    "cornserve-b200/tiny-internvl": {"model_type": "internvl_chat", "torch_dtype": "float32", "llm_config": {"hidden_size": 96},
                                     "vision_config": {"hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
                                                       "num_attention_heads": 2, "image_size": 56, "patch_size": 14}},
}


def resolve_model_dir(model_id: str) -> Path | None:
    """Local directory that holds ``config.json`` for ``model_id`` or ``None``."""
    candidates = [Path(model_id)]
    if os.environ.get("CORNSERVE_MODEL_DIR"):
        candidates.append(Path(os.environ["CORNSERVE_MODEL_DIR"]) / model_id)
    cache = Path(os.environ.get("HF_HOME", Path.home() / ".cache" / "huggingface")) / "hub"
    snap = cache / ("models--" + model_id.replace("/", "--")) / "snapshots"
    if snap.is_dir():
        candidates.extend(sorted(snap.iterdir(), reverse=True))
    for c in candidates:
        if (c / "config.json").is_file() or (c / "model_index.json").is_file():
            return c
    return None


def load_config(model_id: str) -> dict[str, Any]:
    """``config.json`` of the model (from disk, else from the built-in architecture table)."""
    d = resolve_model_dir(model_id)
    if d is not None and (d / "config.json").is_file():
        return json.loads((d / "config.json").read_text())
    if model_id in BUILTIN_CONFIGS:
        return dict(BUILTIN_CONFIGS[model_id])
    raise FileNotFoundError(f"Model {model_id} was not found locally (set CORNSERVE_MODEL_DIR) and is not a built-in "
                            "architecture")


def has_weights(model_id: str) -> bool:
    d = resolve_model_dir(model_id)
    return d is not None and (any(d.glob("*.safetensors")) or (d / "model.safetensors.index.json").is_file())


def iter_safetensors(model_id: str, required_prefixes: list[str] | None = None, strip_prefixes: bool = True,
                     ignored_prefixes: list[str] | None = None) -> Iterator[tuple[str, torch.Tensor]]:
    """Yield ``(name, tensor)`` for every checkpoint tensor whose name starts with one of
    ``required_prefixes`` (the prefix is stripped when asked).  With an index file only the shards that
    contain matching tensors are opened."""
    from safetensors import safe_open

    d = resolve_model_dir(model_id)
    if d is None:
        raise FileNotFoundError(f"no checkpoint directory for {model_id}")
    prefixes = required_prefixes or [""]
    ignored = ignored_prefixes or []
    index = d / "model.safetensors.index.json"
    if index.is_file():
        weight_map = json.loads(index.read_text())["weight_map"]
        files = sorted({f for name, f in weight_map.items() if any(name.startswith(p) for p in prefixes)})
    else:
        files = sorted(p.name for p in d.glob("*.safetensors"))
    for fname in files:
        with safe_open(str(d / fname), framework="pt", device="cpu") as f:
            for name in f.keys():
                hit = next((p for p in prefixes if name.startswith(p)), None)
                if hit is None:
                    continue
                out = name[len(hit):] if strip_prefixes else name
                if any(out.startswith(i) for i in ignored):
                    continue
                yield out, f.get_tensor(name)


_BUFFER_SUFFIXES = ("inv_freq", "rotary_emb.inv_freq", "position_ids", "num_batches_tracked")


def load_model_weights(model: torch.nn.Module, model_id: str, required_prefixes: list[str], strict: bool = True,
                       ignored_prefixes: list[str] | None = None, strip_prefixes: bool = True) -> bool:
    """Load checkpoint tensors through ``model.load_weights``.  Returns ``False`` (leaving the random
    initialisation in place) when the model has no weights on disk and random init is allowed."""
    if not has_weights(model_id):
        # serving random weights is for benchmarks and tests, which ask for it; a mistyped model id must not do it
        if os.environ.get("CORNSERVE_ALLOW_RANDOM_INIT", "0") != "1":
            raise FileNotFoundError(f"No safetensors found for {model_id} (set CORNSERVE_ALLOW_RANDOM_INIT=1 to serve "
                                    "randomly initialised weights of its architecture)")
        logger.warning("No checkpoint for %s on this machine: keeping randomly initialised weights", model_id)
        return False
    seen: list[str] = []

    def counted():
        for name, t in iter_safetensors(model_id, required_prefixes, strip_prefixes, ignored_prefixes):
            seen.append(name)
            yield name, t

    loaded = set(model.load_weights(counted()))
    expected = {n for n, _ in model.named_parameters()}
    logger.info("Loaded %d checkpoint tensors into %d parameters of %s", len(loaded), len(expected), model_id)
    if strict and not loaded:
        raise RuntimeError(f"No tensor of {model_id} matched prefixes {required_prefixes}")
    # checkpoint tensors under the model's prefixes that the model did not take: a layout it does not know (stacked
    # experts, renamed projections) would otherwise leave those parameters at their random initialisation in silence
    skipped = [n for n in dict.fromkeys(seen) if n not in loaded and not n.endswith(_BUFFER_SUFFIXES)]
    if skipped:
        msg = (f"{len(skipped)} of {len(set(seen))} checkpoint tensors of {model_id} were not recognised by "
               f"{type(model).__name__}: {skipped[:12]}{' ...' if len(skipped) > 12 else ''}")
        if strict and os.environ.get("CORNSERVE_STRICT_WEIGHTS", "1") == "1":
            raise RuntimeError(msg)
        logger.error(msg)
    return True
