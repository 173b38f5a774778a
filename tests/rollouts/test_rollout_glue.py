"""Rollout glue: batch stacking, family registry, request builder, collector routing, runtime
inputs and backend validation (reference expectations: ``tests/rollouts/test_*.py`` and
``tests/engine/generation/test_runtime_factory.py``)."""

import asyncio
import pickle
from types import SimpleNamespace

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.engine.core.types import GenerationMetrics, OutputBatch
from visionrl_b200.rollouts.batch import RolloutBatch, stack_batches
from visionrl_b200.rollouts.collector import build_rollout_collector
from visionrl_b200.rollouts.collector.configs import SD3_5CollectorConfig
from visionrl_b200.rollouts.collector.core import RolloutCollector
from visionrl_b200.rollouts.collector.requests import RolloutEngineRequestBuilder
from visionrl_b200.rollouts.collector.rewards import RewardScorer
from visionrl_b200.rollouts.families.specs import (FAMILY_REGISTRY, get_rollout_family_entry,
                                                   normalize_rollout_family)
from visionrl_b200.rollouts.runtime import (RolloutBackendConfig, build_rollout_backend_from_cfg,
                                            build_rollout_runtime_inputs)
from visionrl_b200.rollouts.runtime.backend import validate_rollout_backend_config


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


# ------------------------------------------------------------------------------------ batch
def test_stack_batches_concatenates_samples_and_keeps_first_context():
    def mk(n, tag):
        return RolloutBatch(observations=torch.zeros(n, 2, 3), actions=torch.ones(n, 2, 3),
                            rewards=torch.arange(n, dtype=torch.float32), dones=torch.ones(n),
                            group_ids=torch.full((n,), tag), extras={"log_probs": torch.zeros(n, 2), "tag": tag},
                            context={"guidance_scale": tag}, videos=torch.zeros(n, 3, 4, 4),
                            prompts=[f"p{tag}"] * n)

    a, b = mk(2, 1), mk(3, 2)
    s = stack_batches([a, b])
    assert s.observations.shape == (5, 2, 3) and s.extras["log_probs"].shape == (5, 2)
    assert s.group_ids.tolist() == [1, 1, 2, 2, 2] and s.context == {"guidance_scale": 1}
    assert s.extras["tag"] == 1 and s.prompts == ["p1"] * 2 + ["p2"] * 3 and s.videos.shape[0] == 5
    assert stack_batches([a]) is a


# --------------------------------------------------------------------------------- registry
def test_family_registry_covers_the_five_families_with_importable_paths():
    assert set(FAMILY_REGISTRY) == {"sd3_5", "wan_2_1", "cosmos", "janus_pro", "nextstep_1"}
    tasks = {f: e.task for f, e in FAMILY_REGISTRY.items()}
    assert tasks == {"sd3_5": "t2i", "wan_2_1": "t2v", "cosmos": "v2w", "janus_pro": "ar_t2i",
                     "nextstep_1": "ar_t2i"}
    import importlib

    for entry in FAMILY_REGISTRY.values():
        for path in (entry.executor_cls, entry.runtime_builder, entry.runtime_spec_extractor,
                     entry.gatherer.import_path, entry.collector.config_cls):
            module, _, attr = path.partition(":")
            assert hasattr(importlib.import_module(module), attr), path
    assert normalize_rollout_family("wan_2_1_14b") == "wan_2_1"
    assert get_rollout_family_entry("janus").family == "janus_pro"
    with pytest.raises(ValueError):
        get_rollout_family_entry("nope")
    assert FAMILY_REGISTRY["cosmos"].executor_kwargs.include_reference_image


# -------------------------------------------------------------------------- request builder
def test_request_builder_uses_declared_fields_only():
    cfg = SimpleNamespace(num_steps=10, size=(64, 64), hidden="x")
    rb = RolloutEngineRequestBuilder(family="sd3_5", task="t2i", request_prefix="sd3", config=cfg,
                                     sampling_fields=("num_steps", "size"), return_artifacts=("output",),
                                     default_task_type="text_to_image")
    plan = rb.build(["a", "b"], 4, {"seed": 11, "target_text": "HI", "policy_version": 3,
                                    "request_overrides": {"num_steps": 5}})
    req = plan.request
    assert req.request_id.startswith("sd3-") and req.samples_per_prompt == 4
    assert req.sampling == {"num_steps": 5, "size": [64, 64], "seed": 11}       # tuple -> list, no "hidden"
    assert req.metadata["target_text"] == "HI" and req.metadata["task_type"] == "text_to_image"
    assert req.policy_version == 3 and req.return_artifacts == {"output"}
    bad = RolloutEngineRequestBuilder(family="sd3_5", task="t2i", request_prefix="sd3", config=cfg,
                                      sampling_fields=("missing",), return_artifacts=("output",))
    with pytest.raises(ValueError):
        bad.build(["a"], 1, {})
    nested = RolloutEngineRequestBuilder(family="nextstep_1", task="ar_t2i", request_prefix="ns",
                                         config=cfg, sampling_fields=("num_steps",),
                                         return_artifacts=("output",), metadata_key="rollout_metadata")
    assert nested.build(["a"], 1, {"target_text": "T"}).request.metadata == {"rollout_metadata": {"target_text": "T"}}


# -------------------------------------------------------------------------------- collector
class _Runtime:
    def __init__(self, error=None):
        self.requests, self.error = [], error

    async def generate(self, request):
        self.requests.append(request)
        n = len(request.prompts) * request.samples_per_prompt
        return OutputBatch(request_id=request.request_id, family=request.family, task=request.task,
                           prompts=list(request.prompts), sample_specs=[], output=torch.zeros(n, 3, 2, 2),
                           rollout_trajectory_data=None, extra={}, metrics=GenerationMetrics(),
                           error=self.error)


class _Packer:
    def __init__(self):
        self.seen = {}

    def reward_outputs(self, output, ctx):
        return output.output

    def reward_prompts(self, output, ctx):
        return [p for p in output.prompts for _ in range(output.output.shape[0] // len(output.prompts))]

    async def pack(self, output, rewards, ctx):
        self.seen = {"rewards": rewards, "metadata": ctx.metadata}
        n = output.output.shape[0]
        return RolloutBatch(observations=torch.zeros(n, 1), actions=torch.zeros(n, 1), rewards=rewards,
                            dones=torch.ones(n), group_ids=torch.zeros(n, dtype=torch.long))


class _Reward:
    def __init__(self):
        self.calls = []

    async def score_batch(self, rollouts):
        self.calls.append(rollouts)
        return [float(len(r.trajectory.prompt)) for r in rollouts]


def _collector(runtime, reward):
    rb = RolloutEngineRequestBuilder(family="sd3_5", task="t2i", request_prefix="sd3",
                                     config=SimpleNamespace(num_steps=2), sampling_fields=("num_steps",),
                                     return_artifacts=("output",))
    return RolloutCollector(model=None, config=SimpleNamespace(), family="sd3_5", task="t2i",
                            executor_cls=object, request_builder=rb, packer=_Packer(),
                            reward_scorer=RewardScorer(reward), runtime=runtime)


def test_collector_routes_request_runtime_reward_packer():
    rt, reward = _Runtime(), _Reward()
    col = _collector(rt, reward)
    batch = _run(col.collect(["ab", "cde"], group_size=2, target_text="X"))
    assert len(rt.requests) == 1 and rt.requests[0].samples_per_prompt == 2
    assert batch.rewards.tolist() == [2.0, 2.0, 3.0, 3.0] and batch.rewards.dtype == torch.float32
    assert col.packer.seen["metadata"]["target_text"] == "X"
    assert len(reward.calls) == 1 and len(reward.calls[0]) == 4


def test_collector_requires_runtime_and_surfaces_generation_errors():
    col = _collector(None, None)
    with pytest.raises(RuntimeError):
        _run(col.collect(["a"], group_size=1))
    with pytest.raises(TypeError):
        col.set_runtime(object())
    failing = _collector(_Runtime(error="boom"), None)
    with pytest.raises(RuntimeError, match="boom"):
        _run(failing.collect(["a"], group_size=1))
    quiet = _collector(_Runtime(), None)                         # no reward function -> zeros
    assert _run(quiet.collect(["a"], group_size=3)).rewards.tolist() == [0.0, 0.0, 0.0]


def test_factory_builds_family_collectors():
    col = build_rollout_collector("sd3_5", model=None, reward_fn=None, config=SD3_5CollectorConfig(),
                                  runtime=_Runtime())
    assert col.family == "sd3_5" and col.task == "t2i"
    with pytest.raises(ValueError):
        build_rollout_collector("unknown", model=None, reward_fn=None, config=None, runtime=None)


# --------------------------------------------------------------------------- runtime inputs
def test_runtime_inputs_are_picklable_and_registry_backed():
    cfg = load_config("experiment/sd3_5_ocr_grpo", overrides=["distributed.rollout.gpus_per_worker=0"])
    inputs = build_rollout_runtime_inputs(cfg, "sd3_5", weight_dtype=torch.bfloat16, policy_version=4)
    spec = inputs.runtime_spec
    pickle.loads(pickle.dumps(spec))
    assert spec.family == "sd3_5" and spec.task == "t2i" and spec.policy_version == 4
    assert spec.build_spec["device"] == "cpu" and spec.build_spec["dtype"] == "bfloat16"
    assert spec.executor_cls == FAMILY_REGISTRY["sd3_5"].executor_cls
    assert spec.executor_kwargs["sample_batch_size"] == int(cfg.rollout.sample_batch_size)
    assert type(inputs.gatherer).__name__ == "DiffusionChunkGatherer"
    gpu = build_rollout_runtime_inputs(load_config("experiment/sd3_5_ocr_grpo"), "sd3_5",
                                       weight_dtype="float16", executor_kwargs={"sample_batch_size": 1})
    assert gpu.runtime_spec.build_spec["device"] == "cuda" and gpu.runtime_spec.executor_kwargs["sample_batch_size"] == 1


def test_cosmos_reference_image_is_threaded_into_executor_kwargs():
    cfg = load_config("experiment/cosmos_predict2_2b_grpo",
                      overrides=["distributed.rollout.gpus_per_worker=0", "model.reference_image=/x/ref.png"])
    inputs = build_rollout_runtime_inputs(cfg, "cosmos", weight_dtype=torch.bfloat16)
    assert inputs.runtime_spec.executor_kwargs["reference_image"] == "/x/ref.png"


# ------------------------------------------------------------------------ backend validation
class _FakeDevice:
    def __init__(self, kind):
        self.type = kind


class _FakeParam:
    def __init__(self, kind):
        self.device = _FakeDevice(kind)


class _FakeModule:
    def __init__(self, kind):
        self._p = _FakeParam(kind)

    def parameters(self):
        return iter([self._p])


def test_backend_config_validation_rules():
    with pytest.raises(ValueError):
        RolloutBackendConfig(backend="mpi")
    with pytest.raises(ValueError):
        RolloutBackendConfig(num_workers=0)
    with pytest.raises(ValueError):
        RolloutBackendConfig(max_inflight_chunks_per_worker=0)
    with pytest.raises(ValueError):
        RolloutBackendConfig(sync_trainable_state="everything")
    with pytest.raises(ValueError):
        RolloutBackendConfig.from_cfg({"rollout": {"num_workers": 2}})          # no backend key
    cfg = RolloutBackendConfig.from_cfg({"distributed": {"backend": "ray", "rollout": {"num_workers": 3}}})
    assert cfg.num_workers == 3 and cfg.backend == "ray"
    assert RolloutBackendConfig.from_cfg({"backend": "native"}).backend == "native"


def test_driver_policy_on_cuda_needs_explicit_overlap():
    base = {"distributed": {"backend": "ray", "rollout": {"gpus_per_worker": 1}}}
    with pytest.raises(ValueError):
        validate_rollout_backend_config(base, driver_policy=SimpleNamespace(device=_FakeDevice("cuda")))
    validate_rollout_backend_config(base, driver_policy=SimpleNamespace(device=_FakeDevice("cpu")))
    overlap = {"distributed": {"backend": "ray", "rollout": {"allow_driver_gpu_overlap": True}}}
    validate_rollout_backend_config(overlap, driver_policy=SimpleNamespace(device=_FakeDevice("cuda")))
    with pytest.raises(ValueError):
        validate_rollout_backend_config(base, driver_bundle=SimpleNamespace(
            policy=None, trainable_modules={"transformer": _FakeModule("cuda")}))
    with pytest.raises(ValueError):
        validate_rollout_backend_config(base, trainable_modules={"transformer": _FakeModule("cuda")})


def test_backend_requires_spec_and_gatherer():
    cfg = {"distributed": {"backend": "ray", "rollout": {"gpus_per_worker": 0}}}
    with pytest.raises(ValueError, match="runtime_spec"):
        build_rollout_backend_from_cfg(cfg)
    with pytest.raises(ValueError, match="gatherer"):
        build_rollout_backend_from_cfg(cfg, runtime_spec=object())
