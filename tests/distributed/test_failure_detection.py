"""Failure detection without a device fault: host-side injection on gloo ranks, stale versions,
and (on GPUs) a bounded flag wait that runs out because a rank skips its arrival."""

import asyncio

import pytest
import torch

from tests.distributed import _workers
from tests.distributed.test_multiprocess import _run


def test_rank_that_raises_is_reported_to_its_peer():
    res = _run(_workers.rank_raises_between_steps, 2)
    assert res["detected"] and res["failed_rank"] == 1
    assert "injected collector failure" in res["reason"]
    assert res["seconds"] < 4.0


def test_withheld_heartbeat_is_detected_after_the_deadline():
    res = _run(_workers.heartbeat_withheld, 2)
    assert res["detected"] and res["failed_rank"] == 1
    assert "last heartbeat" in res["reason"]
    assert 0.5 < res["seconds"] < 2.3


def test_collective_after_a_rank_left_fails_instead_of_blocking():
    res = _run(_workers.rank_leaves_between_steps, 2)
    assert res["failed"] and res["seconds"] < 10.0


def test_liveness_with_a_fake_store_and_clock():
    from visionrl_b200.parallel.liveness import RankFailure, RankLiveness

    class Store(dict):
        def set(self, k, v):
            self[k] = v.encode() if isinstance(v, str) else v

        def check(self, keys):
            return all(k in self for k in keys)

        def get(self, k):
            return self[k]

    now = [100.0]
    store = Store()
    a = RankLiveness(store, 0, 2, interval_s=1.0, deadline_s=5.0, clock=lambda: now[0])
    b = RankLiveness(store, 1, 2, interval_s=1.0, deadline_s=5.0, clock=lambda: now[0])
    a.beat(0)
    a.check()                       # peer not heard yet, still inside the start-up window
    b.beat(3)
    now[0] += 4.0
    a.check()
    assert abs(a.peer_age_s(1) - 4.0) < 1e-6
    now[0] += 2.0
    with pytest.raises(RankFailure, match="last heartbeat"):
        a.check()
    b.beat(4)
    a.check()
    b.announce_failure("CUDA out of memory")
    with pytest.raises(RankFailure, match="CUDA out of memory") as info:
        a.check()
    assert info.value.rank == 1
    with pytest.raises(ValueError):
        RankLiveness(store, 0, 2, interval_s=2.0, deadline_s=1.0)


def test_peer_that_never_starts_is_reported_after_the_startup_window():
    from visionrl_b200.parallel.liveness import RankFailure, RankLiveness

    class Store(dict):
        def set(self, k, v):
            self[k] = v

        def check(self, keys):
            return all(k in self for k in keys)

        def get(self, k):
            return self[k]

    now = [0.0]
    live = RankLiveness(Store(), 0, 3, interval_s=0.5, deadline_s=2.0, clock=lambda: now[0])
    live.check()
    now[0] = 2.5
    with pytest.raises(RankFailure, match="start-up"):
        live.check()


def test_stale_policy_version_is_refused_by_the_rollout_runtime():
    from visionrl_b200.distributed.native.runtime import NativeRolloutRuntime
    from visionrl_b200.engine.core.types import GenerationRequest
    from visionrl_b200.parallel.mesh import ProcessMesh

    class Executor:
        family, task = "sd3_5", "t2i"

        def workload_signature(self, request):
            return None

        def forward(self, request, specs):
            raise AssertionError("must not run")

        def forward_chunk(self, request, chunk):
            raise AssertionError("a stale request must be refused before any chunk runs")

        def gather_chunks(self, request, specs, chunks):
            raise AssertionError("must not run")

    class Gatherer:
        def gather_chunks(self, request, specs, chunks):
            raise AssertionError("must not run")

    runtime = NativeRolloutRuntime(Executor(), Gatherer(), ProcessMesh(), policy_version=4)
    stale = GenerationRequest(request_id="r", family="sd3_5", task="t2i", prompts=["p"],
                              samples_per_prompt=1, sampling={}, policy_version=3)
    with pytest.raises(RuntimeError, match="policy_version mismatch"):
        asyncio.new_event_loop().run_until_complete(runtime.generate(stale))
    # an update moves the runtime forward; the old version stays refused
    asyncio.new_event_loop().run_until_complete(runtime.update_weights(None, 5))
    with pytest.raises(RuntimeError, match="policy_version mismatch"):
        asyncio.new_event_loop().run_until_complete(runtime.generate(stale))


def test_trainer_announces_its_own_failure():
    class Live:
        def __init__(self):
            self.failures, self.beats, self.checks = [], [], 0

        def check(self):
            self.checks += 1

        def beat(self, step):
            self.beats.append(step)

        def announce_failure(self, reason):
            self.failures.append(reason)

    live = Live()
    trainer = _workers._fake_trainer(0, 1, fail_on_step=1, liveness=live)
    loop = asyncio.new_event_loop()
    loop.run_until_complete(trainer.step())
    with pytest.raises(RuntimeError, match="injected"):
        loop.run_until_complete(trainer.step())
    assert live.checks == 2 and live.beats == [0, 1]
    assert live.failures and "injected collector failure" in live.failures[0]


@pytest.mark.gpu
@pytest.mark.multigpu
def test_flag_barrier_gives_up_when_a_rank_never_arrives():
    res = _run(_workers.barrier_times_out_when_a_rank_skips, 2)
    assert res["timed_out"] and res["stream_ok"]
    assert res["seconds"] < 5.0
    assert "did not arrive" in res["message"]
