"""Engine core and small shared pieces with fixed inputs: prompt-major micro-batch plans, the
out-of-memory bisection (which chunks are retried, in which order, what is re-raised), chunk
splitting, sample specs, the worker's error capture, the averaged-parameter wrapper's warm-up and
update interval, the weighted reward mix with its per-component history, and batch stacking.
``compute()`` returns JSON strings; ``tests/golden/engine_core_outputs.json`` holds what the
reference's own code gives."""

import asyncio
import json

import torch
from torch import nn
from vrl.engine.core.types import GenerationRequest, OutputBatch, GenerationMetrics
from vrl.engine.core.worker import GenerationIdFactory, GenerationWorker
from vrl.engine.core.registry import FamilyPipelineRegistry
from vrl.engine.microbatching import MicroBatchPlan, plan_prompt_group_microbatches, run_microbatches_with_oom_retry
from vrl.trainers.ema import EMAModuleWrapper
from vrl.rewards.multi import MultiReward
from vrl.rewards.base import RewardFunction
from vrl.algorithms.types import Rollout, Trajectory
from vrl.rollouts.batch import RolloutBatch, stack_batches


def compute() -> dict:
    res = {}

    def rec(k, v):
        res[k] = json.dumps(v, sort_keys=True, default=str)

    # --- micro-batch plans and OOM bisection
    for prompts, n, bs in ((["a", "b"], 5, 2), (["a"], 8, 8), (["a", "b", "c"], 1, 4)):
        plan = plan_prompt_group_microbatches(prompts, n, bs)
        chunks = plan.micro_batches
        rec(f"plan/{len(prompts)}x{n}/{bs}/total", plan.total_samples() if callable(plan.total_samples) else plan.total_samples)
        rec(f"plan/{len(prompts)}x{n}/{bs}", [(c.prompt_index, c.prompt, c.sample_start, c.sample_count) for c in chunks])
    calls = []
    def run(chunk):
        calls.append((chunk.prompt_index, chunk.sample_start, chunk.sample_count))
        if chunk.sample_count > 2: raise RuntimeError("CUDA out of memory. Tried to allocate 2.00 GiB")
        return (chunk.prompt_index, chunk.sample_start, chunk.sample_count)
    chunks = [MicroBatchPlan(prompt_index=0, prompt="a", sample_start=0, sample_count=7), MicroBatchPlan(prompt_index=1, prompt="b", sample_start=0, sample_count=2)]
    rec("oom/results", run_microbatches_with_oom_retry(chunks, run))
    rec("oom/calls", calls)
    try:
        run_microbatches_with_oom_retry([MicroBatchPlan(prompt_index=0, prompt="a", sample_start=0, sample_count=1)], lambda c: (_ for _ in ()).throw(RuntimeError("CUDA out of memory")))
        rec("oom/single", "no error")
    except Exception as e: rec("oom/single", type(e).__name__)
    try:
        run_microbatches_with_oom_retry(chunks, lambda c: (_ for _ in ()).throw(RuntimeError("shape mismatch")))
    except Exception as e: rec("oom/other", [type(e).__name__, str(e)])
    a, b = chunks[0].split()
    rec("split", [(a.sample_start, a.sample_count), (b.sample_start, b.sample_count)])
    # --- sample specs
    r = GenerationRequest(request_id="req-1", family="f", task="t", prompts=["x", "y"], samples_per_prompt=3, sampling={"seed": 9})
    specs = GenerationIdFactory().build_sample_specs(r)
    rec("specs", [{k: getattr(s, k) for k in s.__dataclass_fields__} for s in specs])
    # --- worker: errors become OutputBatch.error; batching of requests
    class Ex:
        family, task = "f", "t"
        def __init__(self): self.seen = []
        def workload_signature(self, request):
            from vrl.engine.core.types import WorkloadSignature
            return WorkloadSignature.from_request(request)
        def forward(self, request, sample_specs):
            self.seen.append((request.request_id, len(sample_specs)))
            if request.metadata.get("boom"): raise ValueError("executor failed: boom")
            return OutputBatch(request_id=request.request_id, family="f", task="t", prompts=list(request.prompts), sample_specs=list(sample_specs),
                               output=torch.zeros(len(sample_specs), 1), rollout_trajectory_data=None, extra={}, metrics=GenerationMetrics())
    reg = FamilyPipelineRegistry()
    ex = Ex()
    reg.register(ex)
    w = GenerationWorker(reg)
    ok = w.execute([r])[r.request_id]
    rec("worker/ok", {"error": ok.error, "n": len(ok.sample_specs), "rid": ok.request_id})
    bad_req = GenerationRequest(request_id="req-2", family="f", task="t", prompts=["x"], samples_per_prompt=1, sampling={}, metadata={"boom": True})
    bad = w.execute([bad_req])[bad_req.request_id]
    rec("worker/bad", {"error": bad.error, "rid": bad.request_id, "has_output": bad.output is not None})
    unk = GenerationRequest(request_id="req-3", family="nope", task="t", prompts=["x"], samples_per_prompt=1, sampling={})
    u = w.execute([unk])[unk.request_id]
    rec("worker/unknown", {"error": u.error})
    # --- EMA
    for kw in (dict(decay=0.9, update_step_interval=2), dict(decay=0.999, update_step_interval=1)):
        torch.manual_seed(0)
        lin = nn.Linear(3, 2)
        ema = EMAModuleWrapper(list(lin.parameters()), **kw)
        decays, snaps = [], []
        for step in range(1, 7):
            with torch.no_grad():
                for p in lin.parameters(): p.add_(0.1)
            ema.step(list(lin.parameters()), step)
            decays.append(ema.get_current_decay(step))
            snaps.append([float(t.sum()) for t in ema.ema_parameters])
        rec(f"ema/{kw['decay']}/decays", decays)
        rec(f"ema/{kw['decay']}/sums", snaps)
        ema.copy_ema_to(list(lin.parameters()), store_temp=False)
        rec(f"ema/{kw['decay']}/swapped_in", [float(p.detach().sum()) for p in lin.parameters()])
        rec(f"ema/{kw['decay']}/state_keys", sorted(ema.state_dict()))
    # --- MultiReward
    class R1(RewardFunction):
        async def score(self, rollout): return float(len(rollout.trajectory.prompt))
    class R2(RewardFunction):
        async def score(self, rollout): return 0.5
        async def score_batch(self, rollouts): return [0.25 * i for i in range(len(rollouts))]
    def ro(p): return Rollout(request=None, trajectory=Trajectory(prompt=p, seed=0, steps=[], output=torch.zeros(1)), reward=0.0, metadata={}) if "request" in Rollout.__dataclass_fields__ else Rollout(trajectory=Trajectory(prompt=p, seed=0, steps=[], output=torch.zeros(1)))
    loop = asyncio.new_event_loop()
    try:
        mr = MultiReward([("len", R1(), 2.0), ("half", R2(), -1.0)])
        rec("multi/score", loop.run_until_complete(mr.score(ro("abc"))))
        rec("multi/batch", loop.run_until_complete(mr.score_batch([ro("a"), ro("bb"), ro("ccc")])))
        rec("multi/components", {k: list(v) for k, v in mr.last_components.items()} if hasattr(mr, "last_components") else None)
        mr.reset_components()
        rec("multi/after_reset", {k: list(v) for k, v in mr.last_components.items()} if hasattr(mr, "last_components") else None)
    except Exception as e:
        rec("multi/error", [type(e).__name__, str(e)[:200]])
    # --- stack_batches
    def rb(n, off): return RolloutBatch(observations=torch.arange(n * 2.0).view(n, 2) + off, actions=torch.ones(n, 2), rewards=torch.arange(float(n)), dones=torch.ones(n), group_ids=torch.full((n,), off),
                                        extras={"lp": torch.zeros(n, 2) + off, "note": "x"}, context={"c": off}, prompts=[f"p{off}"] * n)
    s = stack_batches([rb(2, 0), rb(3, 1)])
    rec("stack", {"obs": s.observations.tolist(), "gid": s.group_ids.tolist(), "extras": sorted(s.extras), "lp": s.extras["lp"].tolist(), "ctx": s.context, "prompts": s.prompts})
    return res
