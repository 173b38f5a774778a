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

    # the two fields of the reference's ``RayPlacement`` record, as views of this one
    @property
    def placement_group(self) -> Any:
        return self.handle

    @property
    def ordered_bundle_indices(self) -> list[int]:
        return [b.index for b in self.bundles]


# the name the reference's launcher and tests use for the placement record
RayPlacement = RolloutPlacementGroup


def create_rollout_placement_group(config: Any, *, gpus_per_worker: float | None = None,
                                   cpus_per_worker: float | None = None,
                                   strategy: str | None = None) -> RolloutPlacementGroup:
    """One bundle per worker, in stable (node, GPU, index) order.  ``config`` is a rollout backend
    config carrying ``num_workers``, ``gpus_per_worker``, ``cpus_per_worker`` and
    ``placement_strategy`` (the reference's call shape), or just the worker count."""
    num_workers = config
    if not isinstance(config, int):
        pick = (lambda k, d: config.get(k, d)) if isinstance(config, dict) else (lambda k, d: getattr(config, k, d))
        num_workers = int(pick("num_workers", 1))
        gpus_per_worker = float(pick("gpus_per_worker", 1.0)) if gpus_per_worker is None else gpus_per_worker
        cpus_per_worker = float(pick("cpus_per_worker", 1.0)) if cpus_per_worker is None else cpus_per_worker
        strategy = str(pick("placement_strategy", "SPREAD")) if strategy is None else strategy
    gpus_per_worker = 1.0 if gpus_per_worker is None else gpus_per_worker
    cpus_per_worker = 1.0 if cpus_per_worker is None else cpus_per_worker
    strategy = "SPREAD" if strategy is None else strategy
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
