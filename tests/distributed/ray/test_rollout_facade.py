"""The ``vrl.distributed.ray`` rollout facade on CPU workers with the real tiny DiT: chunks are
planned prompt-major and spread round-robin, results come back in order, stale policy versions
are refused, weight updates reach ``policy.load_trainable_state`` (reference expectations:
``tests/distributed/ray/test_large_rollout_execution.py:216-470``)."""

import asyncio

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.distributed.ray import (DistributedExecutionPlanner, RayRolloutLauncher,
                                           RayRolloutWorker, RayWorkerHandle)
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.microbatching import MicroBatchPlan
from visionrl_b200.rollouts.collector import build_rollout_collector
from visionrl_b200.rollouts.collector.configs import SD3_5CollectorConfig
from visionrl_b200.rollouts.runtime import build_rollout_runtime_inputs


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


@pytest.fixture(scope="module")
def tiny_cfg():
    return load_config("experiment/tiny_dit_grpo", overrides=[
        "distributed.backend=ray", "distributed.rollout.num_workers=2",
        "distributed.rollout.gpus_per_worker=0", "distributed.rollout.sync_trainable_state=lora_only",
        "sampling.num_steps=3", "rollout.sample_batch_size=2"])


@pytest.fixture(scope="module")
def runtime(tiny_cfg):
    inputs = build_rollout_runtime_inputs(tiny_cfg, "sd3_5", weight_dtype=torch.float32, policy_version=5)
    rt = RayRolloutLauncher().launch(tiny_cfg, inputs.runtime_spec, inputs.gatherer)
    yield rt
    _run(rt.shutdown())


def _collector_config(cfg):
    s = cfg.sampling
    return SD3_5CollectorConfig(num_steps=int(s.num_steps), guidance_scale=float(s.guidance_scale),
                                height=int(s.height), width=int(s.width), sample_batch_size=2,
                                max_sequence_length=int(s.max_sequence_length), noise_level=0.7)


def test_round_robin_planner_is_prompt_major():
    req = GenerationRequest(request_id="r", family="sd3_5", task="t2i", prompts=["a", "b"],
                            samples_per_prompt=5, sampling={"sample_batch_size": 2})
    workers = [RayWorkerHandle("w0", "n0"), RayWorkerHandle("w1", "n0")]
    plan = DistributedExecutionPlanner().plan(req, workers)
    assert [(a.worker_id, a.chunk.prompt_index, a.chunk.sample_start, a.chunk.sample_count) for a in plan] == [
        ("w0", 0, 0, 2), ("w1", 0, 2, 2), ("w0", 0, 4, 1), ("w1", 1, 0, 2), ("w0", 1, 2, 2), ("w1", 1, 4, 1)]
    with pytest.raises(ValueError):
        DistributedExecutionPlanner().plan(req, [])


def test_generate_spreads_chunks_and_returns_ordered_cpu_results(tiny_cfg, runtime):
    collector = build_rollout_collector("sd3_5", model=None, reward_fn=None,
                                        config=_collector_config(tiny_cfg), runtime=runtime)
    batch = _run(collector.collect(["p0", "p1"], group_size=4, seed=3))
    steps = 3
    assert batch.observations.shape[:2] == (8, steps) and batch.actions.shape == batch.observations.shape
    assert batch.extras["log_probs"].shape == (8, steps) and batch.extras["timesteps"].shape == (8, steps)
    assert batch.group_ids.tolist() == [0, 0, 0, 0, 1, 1, 1, 1]
    assert batch.observations.device.type == "cpu"
    again = _run(collector.collect(["p0", "p1"], group_size=4, seed=3))
    assert torch.equal(batch.actions, again.actions) and torch.equal(batch.extras["log_probs"],
                                                                      again.extras["log_probs"])
    other = _run(collector.collect(["p0", "p1"], group_size=4, seed=4))
    assert not torch.equal(batch.actions, other.actions)
    assert len({h.worker_id for h in runtime.workers}) == 2


def test_runtime_fills_current_policy_version_and_rejects_stale_ones(runtime):
    assert runtime.current_policy_version == 5
    worker = runtime.workers[0].actor
    assert isinstance(worker, RayRolloutWorker) and worker.current_policy_version() == 5
    req = GenerationRequest(request_id="stale", family="sd3_5", task="t2i", prompts=["a"],
                            samples_per_prompt=1, sampling={"num_steps": 2}, policy_version=4)
    result = worker.execute_chunk(req, MicroBatchPlan(prompt_index=0, prompt="a", sample_start=0,
                                                       sample_count=1))
    assert result.output is None and "policy_version" in (result.error or "")


def test_weight_update_reaches_the_policy_and_bumps_the_version(runtime):
    worker = runtime.workers[0].actor
    policy = worker.executor.model
    state = {k: torch.full_like(v, 0.125) for k, v in policy.trainable_modules["transformer"].state_dict().items()
             if "lora" in k}
    assert state, "the tiny recipe trains LoRA adapters"
    payload = {f"transformer.{k}": v for k, v in state.items()}
    _run(runtime.update_weights(payload, 6))
    assert runtime.current_policy_version == 6
    for h in runtime.workers:
        assert h.actor.current_policy_version() == 6
        sd = h.actor.executor.model.trainable_modules["transformer"].state_dict()
        assert all(torch.equal(sd[k], v) for k, v in state.items())
    with pytest.raises(Exception):
        _run(runtime.update_weights({"not_transformer.x": torch.zeros(1)}, 7))


def test_inflight_cap_is_validated(tiny_cfg):
    inputs = build_rollout_runtime_inputs(tiny_cfg, "sd3_5", weight_dtype=torch.float32)
    bad = {"backend": "ray", "num_workers": 1, "gpus_per_worker": 0, "max_inflight_chunks_per_worker": 0}
    with pytest.raises(ValueError):
        RayRolloutLauncher().launch(bad, inputs.runtime_spec, inputs.gatherer)
