"""Apps written for the reference run here without edits: the unmodified sources of the reference's
``examples/mllm.py`` and ``examples/qwen_image.py`` (``from cornserve.app.base import AppConfig``,
``from cornserve_tasklib.task.composite.llm import MLLMTask``, ...) are registered with a live local cluster and
invoked.  The model ids they name resolve, through ``CORNSERVE_MODEL_DIR``, to directories that hold tiny
configurations, so the executors start on the CPU with random weights."""

import base64
import json
import os
from pathlib import Path

import pytest

from test_config1_e2e import _serve_app

_HERE = Path(__file__).resolve()


def _reference_examples() -> Path | None:
    for cand in (os.environ.get("CORNSERVE_REFERENCE_DIR"), _HERE.parents[2] / "reference"):
        if cand and (Path(cand) / "examples" / "mllm.py").is_file():
            return Path(cand) / "examples"
    return None


EXAMPLES = _reference_examples()
needs_reference = pytest.mark.skipif(EXAMPLES is None, reason="the reference checkout is not on this machine")


def _model_dir(tmp_path, entries: dict[str, tuple[str, dict]]) -> str:
    root = tmp_path / "models"
    for model_id, (fname, cfg) in entries.items():
        d = root / model_id
        d.mkdir(parents=True)
        (d / fname).write_text(json.dumps(cfg))
    return str(root)


@needs_reference
@pytest.mark.timeout(600)
def test_reference_mllm_example_runs_unmodified(tmp_path, monkeypatch):
    from cornserve.utils.hub import BUILTIN_CONFIGS

    models = _model_dir(tmp_path, {"Qwen/Qwen3-VL-8B-Instruct": ("config.json", BUILTIN_CONFIGS["cornserve-b200/tiny-vlm"])})

    def request(i):
        return {"model": "Qwen/Qwen3-VL-8B-Instruct", "max_completion_tokens": 8, "ignore_eos": True,
                "messages": [{"role": "user", "content": [
                    {"type": "text", "text": f"Write a poem about picture {i}."},
                    {"type": "image_url", "image_url": {"url": f"synthetic:224x224:{i}"}}]}]}

    def finish_reasons(chunks):
        assert all(ch["object"] == "chat.completion.chunk" for ch in chunks)
        return [ch["choices"][0]["finish_reason"] for ch in chunks if ch.get("choices")]

    streams = _serve_app(tmp_path, monkeypatch, (EXAMPLES / "mllm.py").read_text(), num_gpus=2, request_of=request,
                         collect=finish_reasons, extra_env={"CORNSERVE_MODEL_DIR": models})
    assert len(streams) == 4
    for reasons in streams:  # a stream of deltas that ends because the token budget ran out
        assert len(reasons) >= 2 and reasons[-1] == "length" and not any(reasons[:-1])


@needs_reference
@pytest.mark.timeout(600)
def test_reference_qwen_image_example_runs_unmodified(tmp_path, monkeypatch):
    import cornserve.task_executors.geri.loader  # noqa: F401  (adds the generator entries to the table)
    from cornserve.utils.hub import BUILTIN_CONFIGS

    models = _model_dir(tmp_path, {
        "Qwen/Qwen2.5-VL-7B-Instruct": ("config.json", BUILTIN_CONFIGS["cornserve-b200/tiny-vlm"]),
        "Qwen/Qwen-Image": ("model_index.json", BUILTIN_CONFIGS["cornserve-b200/tiny-image-generator"])})

    def request(i):
        return {"prompt": f"a watercolour of cornfield number {i} under a wide evening sky", "height": 64, "width": 64,
                "num_inference_steps": 2}

    def png_of(chunks):
        (out,) = chunks
        return base64.b64decode(out["image"])

    images = _serve_app(tmp_path, monkeypatch, (EXAMPLES / "qwen_image.py").read_text(), num_gpus=2, request_of=request,
                        collect=png_of, extra_env={"CORNSERVE_MODEL_DIR": models})
    assert all(img[:8] == b"\x89PNG\r\n\x1a\n" for img in images)


@needs_reference
@pytest.mark.parametrize("name", ["mllm", "encoder_sharing", "gemmarena", "qwen3_omni", "qwen_image", "stream_transform"])
def test_every_reference_example_is_a_valid_app_here(name):
    """Each example of the reference loads from its unmodified source, passes the gateway's validation of
    ``Config`` / ``serve`` and yields unit tasks that have an execution descriptor."""
    import cornserve_tasklib  # noqa: F401
    from cornserve.services.gateway.app_manager import load_module_from_source, validate_app_module
    from cornserve.task.base import discover_unit_tasks

    module = load_module_from_source((EXAMPLES / f"{name}.py").read_text(), f"reference_example_{name}")
    classes = validate_app_module(module)
    units = discover_unit_tasks(classes.config_cls.tasks.values())
    assert units
    for u in units:
        assert u.execution_descriptor is not None
