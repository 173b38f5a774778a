"""Request / sample-spec contracts, micro-batching, OOM bisection, request fusion, runtime spec."""

import pickle

import pytest
import torch

from vrl.engine import (
    FamilyPipelineRegistry, GenerationIdFactory, GenerationRequest, GenerationRuntime,
    GenerationRuntimeSpec, GenerationWorker, OutputBatch, WorkloadSignature,
    forward_batch_by_merging_prompts,
)
from vrl.engine.microbatching import (
    MicroBatchPlan, plan_prompt_group_microbatches, run_microbatches_with_oom_retry,
)


def _req(**kw):
    base = dict(request_id="req", family="f", task="t", prompts=["a", "b"], samples_per_prompt=2)
    base.update(kw)
    return GenerationRequest(**base)


def test_request_validation():
    for bad in (dict(prompts=[]), dict(samples_per_prompt=0), dict(policy_version=-1),
                dict(request_id=""), dict(family="")):
        with pytest.raises(ValueError):
            _req(**bad)


def test_sample_ids_and_seeds():
    specs = GenerationIdFactory().build_sample_specs(_req(sampling={"seed": 10}, policy_version=3))
    assert [s.sample_id for s in specs] == ["req:prompt:0:sample:0", "req:prompt:0:sample:1",
                                             "req:prompt:1:sample:0", "req:prompt:1:sample:1"]
    assert [s.seed for s in specs] == [10, 11, 12, 13]
    assert specs[2].group_id == "req:prompt:1" and specs[3].metadata["policy_version"] == 3
    assert GenerationIdFactory().build_sample_specs(_req())[0].seed is None


def test_workload_signature():
    sig = WorkloadSignature.from_request(_req(sampling={"height": 64, "width": "32", "num_steps": 4},
                                              return_artifacts={"b", "a"}))
    assert (sig.height, sig.width, sig.num_steps, sig.artifact_mode) == (64, 32, 4, ("a", "b"))


def test_microbatch_plan_is_prompt_major():
    plan = plan_prompt_group_microbatches(["a", "b"], 5, 2)
    got = [(m.prompt_index, m.prompt, m.sample_start, m.sample_count) for m in plan.micro_batches]
    assert got == [(0, "a", 0, 2), (0, "a", 2, 2), (0, "a", 4, 1), (1, "b", 0, 2), (1, "b", 2, 2),
                   (1, "b", 4, 1)]
    assert plan.total_samples == 10
    with pytest.raises(ValueError):
        plan_prompt_group_microbatches([], 1, 1)
    with pytest.raises(ValueError):
        MicroBatchPlan(0, "a", 0, 1).split()


def test_oom_bisection_order():
    seen = []

    def run(mb):
        seen.append(mb.sample_count)
        if mb.sample_count > 2:
            raise RuntimeError("CUDA out of memory. Tried to allocate")
        return mb.sample_count

    out = run_microbatches_with_oom_retry([MicroBatchPlan(0, "a", 0, 5)], run)
    assert seen == [5, 2, 3, 1, 2] and out == [2, 1, 2]
    with pytest.raises(RuntimeError, match="boom"):
        run_microbatches_with_oom_retry([MicroBatchPlan(0, "a", 0, 2)],
                                        lambda mb: (_ for _ in ()).throw(RuntimeError("boom")))
    with pytest.raises(RuntimeError, match="out of memory"):
        run_microbatches_with_oom_retry(
            [MicroBatchPlan(0, "a", 0, 1)],
            lambda mb: (_ for _ in ()).throw(RuntimeError("CUDA out of memory")))


class _Echo:
    family, task = "f", "t"

    def __init__(self):
        self.calls = 0

    def workload_signature(self, request):
        return WorkloadSignature.from_request(request)

    def forward(self, request, specs):
        self.calls += 1
        n = len(specs)
        return OutputBatch(request_id=request.request_id, family="f", task="t",
                           prompts=list(request.prompts), sample_specs=specs,
                           output=torch.arange(n).float(), extra={"x": torch.arange(n) * 10})

    def forward_batch(self, requests, specs_by_request):
        return forward_batch_by_merging_prompts(self, requests, specs_by_request)


def test_worker_fuses_identical_requests_and_reports_errors():
    reg = FamilyPipelineRegistry()
    ex = _Echo()
    reg.register(ex)
    with pytest.raises(ValueError, match="already registered"):
        reg.register(_Echo())
    with pytest.raises(NotImplementedError):
        reg.resolve("f", "other")
    worker = GenerationWorker(reg)
    r1, r2 = _req(request_id="r1"), _req(request_id="r2", prompts=["c"])
    out = worker.execute([r1, r2])
    assert ex.calls == 1
    assert out["r1"].output.tolist() == [0, 1, 2, 3] and out["r2"].output.tolist() == [4, 5]
    assert out["r2"].extra["x"].tolist() == [40, 50]
    ex.calls = 0
    worker.execute([_req(request_id="s1", sampling={"seed": 1}), _req(request_id="s2", sampling={"seed": 1})])
    assert ex.calls == 2        # seeded requests are never merged
    err = worker.execute([_req(request_id="bad", family="zzz")])["bad"]
    assert err.error and err.output is None


def test_generation_runtime_roundtrip():
    import asyncio

    reg = FamilyPipelineRegistry()
    reg.register(_Echo())
    runtime = GenerationRuntime(GenerationWorker(reg), execute_in_thread=True)
    out = asyncio.run(runtime.generate(_req()))
    assert out.request_id == "req" and out.output.numel() == 4


def test_runtime_spec_is_primitives_only_and_picklable():
    spec = GenerationRuntimeSpec(family="f", task="t", runtime_builder="m:b", executor_cls="m:E",
                                 build_spec={"a": [1, (2, 3)], "b": {"c": None}}, policy_version="4")
    assert spec.policy_version == 4 and pickle.loads(pickle.dumps(spec)) == spec
    assert GenerationRuntimeSpec.from_value(spec.to_dict()).build_spec_payload() == spec.build_spec
    with pytest.raises(ValueError, match="runtime_builder"):
        GenerationRuntimeSpec(family="f")
    with pytest.raises(TypeError, match="Tensor"):
        GenerationRuntimeSpec(runtime_builder="m:b", executor_cls="m:E", model_config={"t": torch.zeros(1)})
    with pytest.raises(TypeError, match="Module"):
        GenerationRuntimeSpec(runtime_builder="m:b", executor_cls="m:E",
                              executor_kwargs={"m": torch.nn.Linear(1, 1)})
    with pytest.raises(TypeError, match="callable"):
        GenerationRuntimeSpec(runtime_builder="m:b", executor_cls="m:E", model_config={"f": print})
    with pytest.raises(ValueError, match="live object keys"):
        GenerationRuntimeSpec.from_dict({"policy": object(), "runtime_builder": "m:b", "executor_cls": "m:E"})
    with pytest.raises(ValueError, match="unsupported"):
        GenerationRuntimeSpec.from_dict({"weird": 1})
