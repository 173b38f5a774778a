"""What a rollout worker may be told and what it answers: the runtime spec has to be plain data
(workers build their executor from import paths, nothing live crosses the process boundary), a
worker answers with CPU tensors and reports errors instead of raising, weight updates need a model
that can take them, and the train actor builds its trainer from a factory inside the actor.
Reference expectations: ``tests/distributed/ray/test_large_rollout_execution.py:236-470``,
``test_rollout_launcher.py:239-279``."""

import asyncio
import pickle
from types import SimpleNamespace

import pytest
import torch
from torch import nn

from visionrl_b200.distributed.ray import RayRolloutWorker
from visionrl_b200.distributed.ray.rollout.worker import to_cpu
from visionrl_b200.distributed.ray.train.actor import RayTrainActor, run_awaitable
from visionrl_b200.distributed.ray.train.group import RayTrainGroup
from visionrl_b200.engine.core.runtime_spec import GenerationRuntimeSpec
from visionrl_b200.engine.core.types import GenerationRequest
from visionrl_b200.engine.microbatching import MicroBatchPlan

PATHS = {"runtime_builder": "pkg.mod:build", "executor_cls": "pkg.mod:Executor"}


# ------------------------------------------------------------------------------------- the spec
def test_spec_survives_pickling_and_round_trips_through_a_dict():
    spec = GenerationRuntimeSpec(family="sd3_5", task="t2i", model_config={"dtype": "bfloat16", "layers": [1, 2]},
                                 executor_kwargs={"sample_batch_size": 2}, policy_version="7", **PATHS)
    assert spec.policy_version == 7                                   # normalised to int
    again = pickle.loads(pickle.dumps(spec))
    assert again == spec and GenerationRuntimeSpec.from_value(spec.to_dict()) == spec
    assert GenerationRuntimeSpec.from_value(spec) is spec


@pytest.mark.parametrize("key", ["executor", "policy", "pipeline"])
def test_spec_refuses_keys_that_name_live_objects(key):
    with pytest.raises(ValueError, match="live object keys"):
        GenerationRuntimeSpec.from_dict({"family": "sd3_5", key: object(), **PATHS})


def test_spec_refuses_unknown_keys_tensors_modules_and_callables():
    with pytest.raises(ValueError, match="unsupported GenerationRuntimeSpec keys"):
        GenerationRuntimeSpec.from_dict({"family": "sd3_5", "weights": {}, **PATHS})
    with pytest.raises(TypeError, match="torch.Tensor"):
        GenerationRuntimeSpec(family="sd3_5", model_config={"w": torch.zeros(1)}, **PATHS)
    with pytest.raises(TypeError, match="torch.nn.Module"):
        GenerationRuntimeSpec(family="sd3_5", executor_kwargs={"net": nn.Linear(1, 1)}, **PATHS)
    with pytest.raises(TypeError, match="callable"):
        GenerationRuntimeSpec(family="sd3_5", model_config={"hook": len}, **PATHS)
    with pytest.raises(TypeError, match="keys must be strings"):
        GenerationRuntimeSpec(family="sd3_5", model_config={1: "x"}, **PATHS)


@pytest.mark.parametrize("missing", ["runtime_builder", "executor_cls"])
def test_spec_needs_both_import_paths_and_they_must_be_strings(missing):
    paths = dict(PATHS)
    del paths[missing]
    with pytest.raises(ValueError, match="runtime_builder and executor_cls"):
        GenerationRuntimeSpec(family="sd3_5", **paths)
    with pytest.raises(TypeError, match="import path string"):
        GenerationRuntimeSpec(family="sd3_5", **{**PATHS, missing: object})
    with pytest.raises(TypeError, match="GenerationRuntimeSpec or dict"):
        GenerationRuntimeSpec.from_value(["not", "a", "spec"])


# ----------------------------------------------------------------------------------- the worker
class _Executor:
    """Stands in for a family executor: returns what it is told to, or raises."""

    def __init__(self, model=None, fail=False):
        self.model = model
        self.fail = fail
        self.calls = []

    def forward_chunk(self, request, chunk):
        self.calls.append((request.request_id, chunk.prompt_index, chunk.sample_start))
        if self.fail:
            raise RuntimeError("executor exploded")
        return SimpleNamespace(latents=torch.ones(chunk.sample_count, 2), tag="kept",
                               nested={"t": torch.zeros(1), "n": [torch.ones(1), 3]})


def _worker(executor, version=3):
    spec = GenerationRuntimeSpec(family="sd3_5", task="t2i", policy_version=version, **PATHS)
    worker = RayRolloutWorker("w0", spec)
    worker.executor = executor                    # skip the import-path build: the contract under test is the worker's
    return worker


def _request(version=None):
    return GenerationRequest(request_id="r1", family="sd3_5", task="t2i", prompts=["p"], samples_per_prompt=2,
                             policy_version=version)


CHUNK = MicroBatchPlan(prompt_index=0, prompt="p", sample_start=0, sample_count=2)


def test_worker_needs_a_family_and_reports_itself():
    with pytest.raises(ValueError, match="family is required"):
        RayRolloutWorker("w", GenerationRuntimeSpec(**PATHS))
    meta = _worker(_Executor()).worker_metadata()
    assert meta["worker_id"] == "w0" and meta["policy_version"] == 3 and "gpu_ids" in meta


def test_worker_answers_with_cpu_data_and_its_policy_version():
    worker = _worker(_Executor())
    res = worker.execute_chunk(_request(version=3), CHUNK)
    assert res.error is None and res.worker_id == "w0" and res.policy_version == 3 and res.chunk is CHUNK
    assert res.output.latents.device.type == "cpu" and res.output.tag == "kept"
    assert res.output.nested["n"][1] == 3 and res.output.nested["t"].device.type == "cpu"
    assert to_cpu({"a": (torch.ones(1), "s")})["a"][1] == "s"


def test_worker_refuses_a_stale_version_and_turns_exceptions_into_results():
    worker = _worker(_Executor())
    stale = worker.execute_chunk(_request(version=4), CHUNK)
    assert stale.output is None and "policy_version mismatch: expected=4, actual=3" in stale.error
    assert worker.executor.calls == []                                # nothing ran at the wrong version
    unversioned = worker.execute_chunk(_request(version=None), CHUNK)
    assert unversioned.error is None
    broken = _worker(_Executor(fail=True)).execute_chunk(_request(version=3), CHUNK)
    assert broken.output is None and broken.error == "executor exploded"


def test_weight_update_needs_a_model_that_can_take_it():
    class _Policy:
        def __init__(self):
            self.seen = None

        def load_trainable_state(self, state):
            self.seen = state

    policy = _Policy()
    worker = _worker(_Executor(model=policy))
    worker.update_weights({"w": torch.ones(1)}, policy_version=9)
    assert policy.seen is not None and worker.current_policy_version() == 9
    worker.update_weights(None, policy_version=10)                    # a bare version bump is fine
    assert worker.current_policy_version() == 10
    with pytest.raises(RuntimeError, match="must expose model"):
        _worker(_Executor(model=None)).update_weights({"w": 1}, 1)
    with pytest.raises(RuntimeError, match="load_trainable_state"):
        _worker(_Executor(model=object())).update_weights({"w": 1}, 1)


# ------------------------------------------------------------------------------ the train actors
class _Trainer:
    def __init__(self, tag):
        self.tag = tag
        self.batches = []

    async def step(self, prompts):
        self.batches.append(list(prompts))
        return {"tag": self.tag, "n": len(prompts)}


def test_train_actor_builds_its_trainer_from_a_factory_inside_the_actor():
    built = []

    def factory(train_config):
        built.append(train_config)
        return _Trainer(train_config["tag"])

    actor = RayTrainActor({"trainer_factory": factory, "tag": "a"})
    assert actor.trainer is None and actor.metadata()["trainer_loaded"] is False
    assert actor.train_step(["p0", "p1"]) == {"tag": "a", "n": 2}      # first step sets the trainer up
    assert len(built) == 1 and actor.metadata()["trainer_loaded"] is True
    actor.train_step(["p2"])
    assert len(built) == 1 and actor.trainer.batches == [["p0", "p1"], ["p2"]]
    assert RayTrainActor({"trainer_factory": lambda: _Trainer("z")}).train_step([]) == {"tag": "z", "n": 0}


def test_train_actor_refuses_to_run_without_a_factory():
    with pytest.raises(ValueError, match="requires train_config"):
        RayTrainActor().setup()
    with pytest.raises(NotImplementedError, match="trainer_factory"):
        RayTrainActor({"other": 1}).setup()
    with pytest.raises(TypeError, match="callable or an import path"):
        RayTrainActor({"trainer_factory": 42}).setup()


def test_train_group_sets_every_actor_up_and_steps_through_the_first():
    group = RayTrainGroup.local({"trainer_factory": lambda train_config: _Trainer("g")}, world_size=3)
    group.setup()
    assert [m["trainer_loaded"] for m in group.metadata()] == [True, True, True]
    assert group.train_step(["p"]) == {"tag": "g", "n": 1}
    assert group.actors[0].trainer.batches == [["p"]] and group.actors[1].trainer.batches == []
    with pytest.raises(ValueError, match="at least one train actor"):
        RayTrainGroup([])


def test_run_awaitable_works_with_and_without_a_running_loop():
    async def value():
        return 5

    assert run_awaitable(7) == 7 and run_awaitable(value()) == 5

    async def inside():
        return run_awaitable(value())                                 # a loop is running here: resolved on a helper thread

    assert asyncio.new_event_loop().run_until_complete(inside()) == 5

    async def boom():
        raise KeyError("inner")

    async def inside_boom():
        return run_awaitable(boom())

    with pytest.raises(KeyError):
        asyncio.new_event_loop().run_until_complete(inside_boom())


def test_placement_record_and_call_shapes_of_the_reference():
    from visionrl_b200.distributed.ray.placement import RayPlacement, create_rollout_placement_group, sort_node_gpu_key
    from visionrl_b200.rollouts.runtime.config import RolloutBackendConfig

    cfg = RolloutBackendConfig.from_cfg({"backend": "ray", "num_workers": 3, "gpus_per_worker": 0, "cpus_per_worker": 2,
                                         "placement_strategy": "PACK"})
    placement = create_rollout_placement_group(cfg)
    assert isinstance(placement, RayPlacement) and placement.strategy == "PACK"
    assert placement.ordered_bundle_indices == [0, 1, 2] and placement.placement_group is not None
    assert all(b.resources == {"CPU": 2.0} for b in placement.bundles)
    assert create_rollout_placement_group(config=2, gpus_per_worker=0).ordered_bundle_indices == [0, 1]
    placement.remove()
    assert placement.placement_group is None and placement.ordered_bundle_indices == []
    # (index, node, gpu): by node address, then GPU, then index; names that are not addresses sort after
    items = [(0, "10.0.0.9", 1), (1, "10.0.0.10", 0), (2, "10.0.0.9", 0), (3, "nodeb", 0)]
    assert [i for i, _, _ in sorted(items, key=sort_node_gpu_key)] == [2, 0, 1, 3]


def test_runtime_launcher_and_train_group_take_the_reference_keywords():
    from visionrl_b200.distributed.ray import (
        RayDistributedRuntime, RayRolloutLauncher, RayTrainGroup, RayTrainRankSpec, RolloutWeightSync,
    )

    class _Executor:
        async def execute(self, request):
            return request

    runtime = RayDistributedRuntime(_Executor(), weight_sync=None, owned_workers=[], placement_group=None)
    assert runtime.workers == [] and runtime.current_policy_version is None
    launcher = RayRolloutLauncher(init_ray=False, ray_init_kwargs={"num_cpus": 2})
    assert launcher.init_ray is False and launcher.ray_init_kwargs == {"num_cpus": 2}
    spec = RayTrainRankSpec(rank=1, local_rank=1, world_size=2, node_id="n0", gpu_ids=(1,))
    assert (spec.rank, spec.local_rank, spec.world_size, spec.node_id) == (1, 1, 2, "n0")
    group = RayTrainGroup(["first", "second"])
    assert group.primary() == "first"
    assert hasattr(RolloutWeightSync, "push_to_rollout_workers")
