"""One request over a pool of rollout workers.

Each assignment of the planner becomes one job.  A worker whose ``execute_chunk`` is a plain
method (workers living in this process: tests, the in-process facade) is called directly; one that
exposes ``.remote`` (a Ray actor method) is awaited on a helper thread, with a per-worker
semaphore keeping at most ``max_inflight_chunks_per_worker`` of its chunks in flight.  Jobs are
independent coroutines collected with ``asyncio.gather``, so results come back in plan order by
construction.  Before gathering, every result is vetted: a chunk that reported an error, ran with
another policy version than the request names, or carries no output ends the request with a
``RuntimeError`` that says which worker and which chunk.  Behavioural reference:
``vrl/distributed/ray/rollout/executor.py:18-141``.
"""

from __future__ import annotations

import asyncio
from typing import Any

from visionrl_b200.distributed.ray.dependencies import require_ray
from visionrl_b200.distributed.ray.rollout.planner import DeviceAssignment, DistributedExecutionPlanner
from visionrl_b200.distributed.ray.rollout.types import RayChunkResult, RayWorkerHandle
from visionrl_b200.engine.core.types import GenerationRequest, OutputBatch
from visionrl_b200.engine.core.worker import GenerationIdFactory
from visionrl_b200.engine.gather import ChunkGatherer, gather_pipeline_chunks


def vet_chunk_result(result: RayChunkResult, request: GenerationRequest) -> Any:
    """The chunk's output, or a ``RuntimeError`` describing why it cannot be used."""
    where = f"worker_id={result.worker_id}"
    if result.error:
        raise RuntimeError(f"distributed rollout chunk failed ({where}, chunk={result.chunk}): "
                           f"{result.error}")
    if request.policy_version is not None and result.policy_version != request.policy_version:
        raise RuntimeError(f"distributed rollout policy_version mismatch ({where}, "
                           f"expected={request.policy_version}, actual={result.policy_version})")
    if result.output is None:
        raise RuntimeError(f"distributed rollout chunk returned no output: {result}")
    return result.output


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

    async def _run_job(self, request: GenerationRequest, job: DeviceAssignment,
                       worker: RayWorkerHandle, gate: asyncio.Semaphore) -> RayChunkResult:
        if worker.actor is None:
            raise RuntimeError(f"worker {worker.worker_id!r} has no actor")
        call = worker.actor.execute_chunk
        remote = getattr(call, "remote", None)
        if not callable(remote):
            return call(request, job.chunk)
        ray = require_ray()
        async with gate:
            return await asyncio.to_thread(ray.get, remote(request, job.chunk))

    async def execute(self, request: GenerationRequest) -> OutputBatch:
        jobs = self.planner.plan(request, self.workers)
        workers = {w.worker_id: w for w in self.workers}
        gates = {wid: asyncio.Semaphore(self.max_inflight_chunks_per_worker) for wid in workers}
        results = await asyncio.gather(*(
            self._run_job(request, job, workers[job.worker_id], gates[job.worker_id])
            for job in jobs))
        if len(results) != len(jobs):
            raise RuntimeError("distributed rollout returned wrong number of chunks: "
                               f"{len(results)} != {len(jobs)}")
        outputs = [vet_chunk_result(r, request) for r in results]
        return gather_pipeline_chunks(self.gatherer, request,
                                      self.id_factory.build_sample_specs(request), outputs)


__all__ = ["DistributedRolloutExecutor", "vet_chunk_result"]
