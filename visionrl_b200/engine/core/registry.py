"""``(family, task)`` → executor lookup (reference: ``vrl/engine/core/registry.py:10-42``)."""

from __future__ import annotations

from dataclasses import dataclass

from visionrl_b200.engine.core.protocols import FamilyPipelineExecutor


@dataclass(frozen=True, slots=True)
class ExecutorKey:
    family: str
    task: str


class FamilyPipelineRegistry:
    def __init__(self) -> None:
        self._executors: dict[ExecutorKey, FamilyPipelineExecutor] = {}

    def register(self, executor: FamilyPipelineExecutor) -> None:
        key = ExecutorKey(executor.family, executor.task)
        if key in self._executors:
            raise ValueError(
                f"Generation executor already registered for family={key.family!r}, task={key.task!r}"
            )
        self._executors[key] = executor

    def resolve(self, family: str, task: str) -> FamilyPipelineExecutor:
        found = self._executors.get(ExecutorKey(family, task))
        if found is None:
            known = sorted((k.family, k.task) for k in self._executors)
            raise NotImplementedError(
                f"No generation executor registered for family={family!r}, task={task!r}; "
                f"registered={known}"
            )
        return found
