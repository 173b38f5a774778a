"""Placement of rollout workers: one ``{CPU, GPU?}`` bundle per worker, ordered by
(node ip, GPU id, bundle index) (reference: ``vrl/distributed/ray/placement/group.py:16-84``).
Without Ray the bundles describe local devices of this process's node."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from visionrl_b200.distributed.ray.dependencies import current_gpu_ids, current_node_ip
from visionrl_b200.distributed.ray.placement.network import bundle_sort_key


@dataclass(frozen=True, slots=True)
class PlacementBundle:
    index: int
    node_ip: str
    gpu_id: int | None
    resources: dict


@dataclass(slots=True)
class RolloutPlacementGroup:
    strategy: str
    bundles: list[PlacementBundle]
    handle: Any | None = None

    def remove(self) -> None:
        self.handle = None
        self.bundles = []


# the name the reference's launcher and tests use for the placement record
RayPlacement = RolloutPlacementGroup


def create_rollout_placement_group(num_workers: int, *, gpus_per_worker: float = 1.0,
                                   cpus_per_worker: float = 1.0,
                                   strategy: str = "SPREAD") -> RolloutPlacementGroup:
    if num_workers < 1:
        raise ValueError("num_workers must be >= 1")
    ip = current_node_ip()
    gpus = current_gpu_ids() if gpus_per_worker > 0 else []
    bundles = []
    for i in range(num_workers):
        gpu = gpus[i % len(gpus)] if gpus else None
        res = {"CPU": float(cpus_per_worker)}
        if gpus_per_worker > 0:
            res["GPU"] = float(gpus_per_worker)
        bundles.append(PlacementBundle(i, ip, gpu, res))
    bundles.sort(key=lambda b: bundle_sort_key(b.node_ip, b.gpu_id, b.index))
    return RolloutPlacementGroup(strategy=strategy, bundles=bundles, handle=object())
