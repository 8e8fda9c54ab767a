"""Resolves a model id to a registry entry and builds the generator with its weights (reference:
python/cornserve/task_executors/geri/executor/loader.py:20-159).  Checkpoints keep their published layout: a
diffusers directory (``model_index.json``, ``transformer/``, ``vae/``) for Qwen-Image, a transformers checkpoint
with ``code2wav.*`` tensors for the Qwen3-Omni vocoder.  Without weights on disk the architecture is instantiated
with random weights (benchmarks and tests)."""

from __future__ import annotations

import json
import os
from pathlib import Path
from typing import Any

import torch

from ...logging import get_logger
from ...parallel.state import ParallelGroup
from ...utils.hub import BUILTIN_CONFIGS, has_weights, iter_safetensors, load_config, resolve_model_dir
from .registry import MODEL_REGISTRY, RegistryEntry

logger = get_logger(__name__)

# architecture-only entries for runs without checkpoints
BUILTIN_CONFIGS.setdefault("Qwen/Qwen-Image", {"_class_name": "QwenImagePipeline"})
BUILTIN_CONFIGS.setdefault("Qwen/Qwen3-Omni-30B-A3B-Instruct", {"model_type": "qwen3_omni_moe", "code2wav_config": {}})
BUILTIN_CONFIGS.setdefault("cornserve-b200/tiny-image-generator", {
    "_class_name": "QwenImagePipeline", "torch_dtype": "float32",
    "transformer": {"in_channels": 64, "out_channels": 16, "num_layers": 1, "attention_head_dim": 64,
                    "num_attention_heads": 2, "joint_attention_dim": 256, "axes_dims_rope": [8, 28, 28]},
    "vae": {"base_dim": 16, "z_dim": 16, "dim_mult": [1, 2, 4, 4], "num_res_blocks": 1}})
BUILTIN_CONFIGS.setdefault("cornserve-b200/tiny-vocoder", {
    "model_type": "qwen3_omni_moe", "torch_dtype": "float32",
    "code2wav_config": {"codebook_size": 32, "hidden_size": 64, "num_attention_heads": 2, "num_key_value_heads": 2,
                        "sliding_window": 6, "intermediate_size": 128, "num_hidden_layers": 2, "num_quantizers": 4,
                        "upsample_rates": [3, 2, 2, 2], "upsampling_ratios": [2, 2], "decoder_dim": 128}})


def model_descriptor(model_id: str) -> dict[str, Any]:
    """``model_index.json`` (diffusers) or ``config.json`` (transformers) of the model, else the built-in table."""
    d = resolve_model_dir(model_id)
    if d is not None:
        for name in ("model_index.json", "config.json"):
            if (d / name).is_file():
                return json.loads((d / name).read_text())
    return load_config(model_id)


def resolve_entry(model_id: str) -> tuple[RegistryEntry, dict[str, Any]]:
    desc = model_descriptor(model_id)
    key = desc.get("_class_name") or desc.get("model_type")
    if key not in MODEL_REGISTRY:
        raise ValueError(f"Model {model_id} ({key!r}) is not supported by the generator executor "
                         f"(supported: {sorted(MODEL_REGISTRY)})")
    return MODEL_REGISTRY[key], desc


def find_embedding_dim(model_id: str) -> int:
    """Row width of the conditioning tensors, without instantiating the model."""
    entry, desc = resolve_entry(model_id)
    if entry.builder == "build_qwen_image":
        d = resolve_model_dir(model_id)
        if d is not None and (d / "text_encoder" / "config.json").is_file():
            return int(json.loads((d / "text_encoder" / "config.json").read_text())["hidden_size"])
        return int((desc.get("transformer") or {}).get("joint_attention_dim", 3584))
    return int((desc.get("code2wav_config") or {}).get("num_quantizers", 16))


def _sub_config(model_id: str, desc: dict, sub: str) -> dict:
    d = resolve_model_dir(model_id)
    if d is not None and (d / sub / "config.json").is_file():
        return json.loads((d / sub / "config.json").read_text())
    return dict(desc.get(sub) or {})


def build_qwen_image(model_id: str, desc: dict, device: torch.device, group: ParallelGroup | None, seed: int = 0):
    from ...models.qwen_image import (FlowMatchConfig, QwenImageDiTConfig, QwenImageModel, QwenImagePipelineConfig)
    from ...models.qwen_image_vae import QwenImageVAEConfig

    sched = _sub_config(model_id, desc, "scheduler")
    if not sched:
        d = resolve_model_dir(model_id)
        if d is not None and (d / "scheduler" / "scheduler_config.json").is_file():
            sched = json.loads((d / "scheduler" / "scheduler_config.json").read_text())
    cfg = QwenImagePipelineConfig(
        dit=QwenImageDiTConfig.from_hf(_sub_config(model_id, desc, "transformer")),
        vae=QwenImageVAEConfig.from_hf(_sub_config(model_id, desc, "vae")),
        sched=FlowMatchConfig(**{k: sched[k] for k in FlowMatchConfig.__dataclass_fields__ if k in sched}))
    model = QwenImageModel(cfg, group=group, device=device, seed=seed)
    d = resolve_model_dir(model_id)
    if d is not None and has_weights(str(d / "transformer")) and has_weights(str(d / "vae")):
        lt, lv = model.load_weights(iter_safetensors(str(d / "transformer")), iter_safetensors(str(d / "vae")))
        logger.info("Loaded %d transformer and %d VAE tensors of %s", len(lt), len(lv), model_id)
    elif os.environ.get("CORNSERVE_ALLOW_RANDOM_INIT", "1") == "1":
        logger.warning("No checkpoint for %s on this machine: keeping randomly initialised weights", model_id)
    else:
        raise FileNotFoundError(f"No safetensors found for {model_id}")
    if device.type == "cpu":  # the CUDA kernels are bf16
        model.dit.float()
        model.vae.float()
    return model


def build_code2wav(model_id: str, desc: dict, device: torch.device, group: ParallelGroup | None, seed: int = 0):
    from ...models.code2wav import Code2Wav, Code2WavConfig

    model = Code2Wav(Code2WavConfig.from_hf(desc), device=device)
    if has_weights(model_id):
        loaded = model.load_weights(iter_safetensors(model_id, ["code2wav."]))
        logger.info("Loaded %d vocoder tensors of %s", len(loaded), model_id)
    elif os.environ.get("CORNSERVE_ALLOW_RANDOM_INIT", "1") != "1":
        raise FileNotFoundError(f"No safetensors found for {model_id}")
    else:
        logger.warning("No checkpoint for %s on this machine: keeping randomly initialised weights", model_id)
    return model


def load_model(model_id: str, device: torch.device, group: ParallelGroup | None = None, seed: int = 0):
    entry, desc = resolve_entry(model_id)
    torch.manual_seed(int(os.environ.get("CORNSERVE_SEED", "0")))
    model = globals()[entry.builder](model_id, desc, device, group, seed)
    return entry, model
