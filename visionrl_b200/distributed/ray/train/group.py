"""Group of train actors addressed as one trainer; calls go to actor 0
(reference: ``vrl/distributed/ray/train/group.py:9-41``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any

from visionrl_b200.distributed.ray.train.actor import RayTrainActor


@dataclass(frozen=True, slots=True)
class RayTrainRankSpec:
    """Where one rank of a train group runs."""

    rank: int
    local_rank: int = 0
    world_size: int = 1
    node_id: str = ""
    gpu_ids: tuple[int, ...] = ()
    env: dict[str, str] = field(default_factory=dict)


class RayTrainGroup:
    def __init__(self, actors: list[Any]) -> None:
        if not actors:
            raise ValueError("RayTrainGroup requires at least one train actor")
        self.actors = list(actors)

    @classmethod
    def local(cls, train_config: Any, world_size: int = 1) -> "RayTrainGroup":
        return cls([RayTrainActor(train_config) for _ in range(world_size)])

    def setup(self, train_config: Any | None = None) -> None:
        for a in self.actors:
            a.setup(train_config)

    def primary(self) -> Any:
        return self.actors[0]

    def train_step(self, prompt_batch: list[Any]) -> Any:
        return self.primary().train_step(prompt_batch)

    def metadata(self) -> list[dict[str, Any]]:
        return [a.metadata() for a in self.actors]


__all__ = ["RayTrainGroup", "RayTrainRankSpec"]
