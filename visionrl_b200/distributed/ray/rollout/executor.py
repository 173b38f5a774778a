"""Runs one request across rollout workers and gathers the chunks
(reference: ``vrl/distributed/ray/rollout/executor.py:18-141``).

Worker methods are called directly unless they expose ``.remote`` (a Ray actor
method); remote jobs respect a per-worker in-flight cap.  Results are restored to
plan order, then checked for errors, stale policy versions and missing outputs.
"""

from __future__ import annotations

import asyncio
from collections import deque
from typing import Any

from visionrl_b200.distributed.ray.dependencies import require_ray
from visionrl_b200.distributed.ray.rollout.planner import DistributedExecutionPlanner
from visionrl_b200.distributed.ray.rollout.types import RayChunkResult, RayWorkerHandle
from visionrl_b200.engine.core.types import GenerationRequest, OutputBatch
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.engine.gather import ChunkGatherer, gather_pipeline_chunks


class DistributedRolloutExecutor:
    def __init__(self, planner: DistributedExecutionPlanner, workers: list[RayWorkerHandle],
                 gatherer: ChunkGatherer, *, id_factory: GenerationIdFactory | None = None,
                 max_inflight_chunks_per_worker: int = 1) -> None:
        if not workers:
            raise ValueError("DistributedRolloutExecutor requires at least one worker")
        if max_inflight_chunks_per_worker < 1:
            raise ValueError("max_inflight_chunks_per_worker must be >= 1")
        self.planner, self.workers, self.gatherer = planner, list(workers), gatherer
        self.id_factory = id_factory or GenerationIdFactory()
        self.max_inflight_chunks_per_worker = int(max_inflight_chunks_per_worker)

    async def execute(self, request: GenerationRequest) -> OutputBatch:
        assignments = self.planner.plan(request, self.workers)
        by_id = {w.worker_id: w for w in self.workers}
        done: dict[int, RayChunkResult] = {}
        remote_jobs = []
        for idx, a in enumerate(assignments):
            worker = by_id[a.worker_id]
            if worker.actor is None:
                raise RuntimeError(f"worker {worker.worker_id!r} has no actor")
            fn = worker.actor.execute_chunk
            remote = getattr(fn, "remote", None)
            if callable(remote):
                remote_jobs.append((idx, remote, worker, a.chunk))
            else:
                done[idx] = fn(request, a.chunk)
        if remote_jobs:
            done.update(await self._run_remote(request, remote_jobs))
        if len(done) != len(assignments):
            raise RuntimeError("distributed rollout returned wrong number of chunks: "
                               f"{len(done)} != {len(assignments)}")
        outputs = []
        for idx in range(len(assignments)):
            r = done[idx]
            if r.error:
                raise RuntimeError(f"distributed rollout chunk failed (worker_id={r.worker_id}, "
                                   f"chunk={r.chunk}): {r.error}")
            if request.policy_version is not None and r.policy_version != request.policy_version:
                raise RuntimeError(
                    f"distributed rollout policy_version mismatch (worker_id={r.worker_id}, "
                    f"expected={request.policy_version}, actual={r.policy_version})")
            if r.output is None:
                raise RuntimeError(f"distributed rollout chunk returned no output: {r}")
            outputs.append(r.output)
        specs = self.id_factory.build_sample_specs(request)
        return gather_pipeline_chunks(self.gatherer, request, specs, outputs)

    async def _run_remote(self, request, jobs) -> dict[int, RayChunkResult]:
        ray = require_ray()
        pending = deque(jobs)
        inflight = {w.worker_id: 0 for _, _, w, _ in jobs}
        refs: dict[Any, tuple[int, str]] = {}
        out: dict[int, RayChunkResult] = {}

        def submit() -> None:
            for _ in range(len(pending)):
                idx, remote, worker, chunk = pending.popleft()
                if inflight[worker.worker_id] >= self.max_inflight_chunks_per_worker:
                    pending.append((idx, remote, worker, chunk))
                    continue
                refs[remote(request, chunk)] = (idx, worker.worker_id)
                inflight[worker.worker_id] += 1

        submit()
        while refs:
            ready, _ = await asyncio.to_thread(ray.wait, list(refs), num_returns=1)
            idx, wid = refs.pop(ready[0])
            inflight[wid] -= 1
            out[idx] = await asyncio.to_thread(ray.get, ready[0])
            submit()
        return out


__all__ = ["DistributedRolloutExecutor"]
