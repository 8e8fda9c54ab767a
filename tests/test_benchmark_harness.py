"""Load generator: arrival processes and latency metric definitions."""

import numpy as np
import pytest

from benchmark.load_generator import RequestRecord, arrival_times, duty_cycle_times, percentiles, summarise


def test_arrival_processes():
    t = arrival_times(20000, rate=10.0, burstiness=1.0, seed=1)
    gaps = np.diff(t)
    assert t[0] == 0 and abs(gaps.mean() - 0.1) < 0.005 and abs(gaps.std() - 0.1) < 0.01   # exponential gaps
    regular = np.diff(arrival_times(20000, 10.0, burstiness=8.0, seed=1))
    assert abs(regular.mean() - 0.1) < 0.005 and regular.std() < 0.05                        # same rate, less variance
    assert (arrival_times(5, float("inf")) == 0).all()
    d = duty_cycle_times(2000, rate_on=50.0, on_s=1.0, off_s=3.0, seed=2)
    assert ((d % 4.0) < 1.0 + 1e-9).all()                                                      # traffic only in the "on" second


def test_latency_metrics():
    r = RequestRecord(send_time=10.0, chunk_times=[10.5, 10.6, 10.8, 11.1], output_tokens=4, ok=True)
    assert abs(r.ttft - 0.5) < 1e-9 and abs(r.e2el - 1.1) < 1e-9
    assert np.allclose(r.itl, [0.1, 0.2, 0.3]) and abs(r.tpot - 0.2) < 1e-9
    bad = RequestRecord(send_time=10.0, error="boom")
    s = summarise([r, bad], duration_s=2.0)
    assert s.completed == 1 and s.failed == 1 and s.request_throughput == 0.5 and s.output_token_throughput == 2.0
    assert abs(s.ttft_ms["median"] - 500.0) < 1e-6 and abs(s.itl_ms["p99"] - 298.0) < 1.0
    p = percentiles(list(range(1, 101)))
    assert p["median"] == 50.5 and abs(p["p99"] - 99.01) < 1e-6


def test_experiment_configurations_and_app_sources():
    """Backend shapes of the comparison harness: validation, result naming, and that every generated app is a valid
    app whose unit tasks are the parts the configuration names."""
    import json

    import pytest

    from benchmark.experiment import BACKENDS, PARTS, ExperimentConfig, Workload, app_source, part_of
    from cornserve.services.gateway.app_manager import load_module_from_source, validate_app_module

    with pytest.raises(ValueError):
        ExperimentConfig("EV", gpus={"llm": 2})
    with pytest.raises(ValueError):
        ExperimentConfig("XX")
    a = ExperimentConfig("EPD", gpus={"encoder": 2, "prefill": 2, "decode": 4}, workload=Workload(request_rate=5))
    b = ExperimentConfig("EPD", gpus={"encoder": 2, "prefill": 2, "decode": 4}, workload=Workload(request_rate=6))
    assert a.total_gpus == 8 and a.key() != b.key() and a.key() == ExperimentConfig(**{**a.__dict__}).key()
    assert a.result_path("x").name.endswith(".json") and "EPD" in a.key() and "d4-e2-p2" in a.key()
    for backend in BACKENDS:
        cfg = ExperimentConfig(backend, "cornserve-b200/tiny-vlm", {p: 1 for p in PARTS[backend]})
        module = load_module_from_source(app_source(cfg), f"bench_app_{backend}")
        classes = validate_app_module(module)
        from cornserve.task.base import discover_unit_tasks

        parts = {part_of(json.dumps({"class_name": type(t).__name__})) for t in discover_unit_tasks(classes.config_cls.tasks.values())}
        assert parts == set(PARTS[backend]), (backend, parts)


@pytest.mark.gpu
def test_encoder_compare_reports_both_arms():
    """The comparison tool runs this package's tower and, when the reference package is installed beside the repository,
    the reference's own encoder module, and prints one JSON line with both rates."""
    import json
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    r = subprocess.run([sys.executable, "-m", "benchmark.encoder_compare", "--images", "1", "--iters", "1", "--warmup", "1"],
                       cwd=root, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])
    assert out["metric"] == "encoder_images_per_second" and out["ours"]["images_per_second"] > 0
    ref = out["reference"]
    assert ("unavailable" in ref) or (ref["images_per_second"] > 0 and out["ours_over_reference"] > 0)
