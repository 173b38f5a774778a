"""The parts of the benchmark driver that need no GPU: the reference arm's one-line answer, the
clock summary made from nvidia-smi rows, and that every named workload points at an experiment
which composes with the overrides the driver adds."""

import importlib.util
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("vrl_bench_module", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_reference_arm_prints_one_json_line_and_exits_zero():
    done = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference",
                           "--gpus", "1", "--steps", "2", "--warmup", "3"],
                          capture_output=True, text=True, timeout=120)
    assert done.returncode == 0, done.stderr
    lines = [ln for ln in done.stdout.splitlines() if ln.strip()]
    assert len(lines) == 1
    answer = json.loads(lines[0])
    assert answer["impl"] == "reference" and isinstance(answer["unavailable"], str) and answer["unavailable"]
    assert "\n" not in answer["unavailable"]


def test_clock_summary_takes_the_median_and_collects_active_reasons():
    sampler = _bench().ClockSampler(0)
    idle = "Not Active"
    sampler.rows = [
        ["0", "1905", "1965", "712.1", "0x4", idle, idle, idle, "Active"],
        ["0", "1935", "1965", "640.0", "0x0", idle, idle, idle, idle],
        ["0", "1920", "1965", "655.3", "0x0", idle, idle, idle, idle],
        ["0", "[N/A]", "1965", "1.0", "0x0", idle, idle, idle, idle],      # unreadable sample: skipped
    ]
    summary = sampler.stop()
    assert summary == {"sm_mhz": 1920.0, "sm_max_mhz": 1965.0, "reasons": ["sw_power_cap"], "samples": 3}
    sampler.rows = [["0", "1100", "1965", "300", "0x8", "Active", "Active", idle, idle]]
    assert sampler.stop()["reasons"] == ["hw_slowdown", "hw_thermal_slowdown"]
    sampler.rows = []
    assert sampler.stop() == {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}


@pytest.mark.parametrize("name", ["sd3_5", "wan_1_3b", "wan_14b", "janus"])
def test_named_workloads_compose_with_the_driver_overrides(name):
    from visionrl_b200.config.loader import load_config

    bench = _bench()
    spec = bench.CONFIGS[name]
    overrides = ["distributed.collectives=fused", "distributed.param_sharding=full",
                 "distributed.rollout_replica=true", "distributed.destroy_on_exit=false",
                 "trainer.output_dir=/tmp/vrl_bench", f"rollout.rollout_batch_size={spec['prompts']}"]
    overrides += [f"rollout.n_samples_per_prompt={spec['group']}"] if name == "janus" else [f"rollout.n={spec['group']}"]
    if name == "wan_1_3b":
        overrides += ["distributed.mesh.sp=4"]
    if name == "wan_14b":
        overrides += ["distributed.mesh.sp=8"]
    cfg = load_config(spec["experiment"], overrides=overrides)
    assert cfg.distributed.collectives == "fused" and cfg.distributed.destroy_on_exit is False
    assert int(cfg.rollout.rollout_batch_size) == spec["prompts"]
    assert spec["seq_len"] > 0 and spec["model"]


def test_headline_line_names_the_metric_of_the_headline_workload():
    bench = _bench()
    assert bench.METRIC.startswith("GRPO samples/sec")
    assert bench.CONFIGS["sd3_5"]["prompts"] * bench.CONFIGS["sd3_5"]["group"] == 64
    assert bench.CONFIGS["sd3_5"]["seq_len"] == 1178
