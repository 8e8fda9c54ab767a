"""Every shipped example is a valid app: it loads, its ``Config`` / ``serve`` pass the gateway's validation, and its
unit tasks are discoverable."""

from pathlib import Path

import pytest

EXAMPLES = sorted((Path(__file__).resolve().parents[1] / "examples").glob("*.py"))


@pytest.mark.parametrize("path", EXAMPLES, ids=lambda p: p.stem)
def test_example_is_a_valid_app(path):
    import cornserve_tasklib  # noqa: F401
    from cornserve.services.gateway.app_manager import load_module_from_source, validate_app_module
    from cornserve.task.base import discover_unit_tasks

    module = load_module_from_source(path.read_text(), f"example_{path.stem}")
    classes = validate_app_module(module)
    units = discover_unit_tasks(classes.config_cls.tasks.values())
    assert units, "an app must deploy at least one unit task"


def test_expected_examples_exist():
    assert {p.stem for p in EXAMPLES} >= {"mllm", "encoder_sharing", "gemmarena", "qwen3_omni", "qwen_image", "stream_transform"}
