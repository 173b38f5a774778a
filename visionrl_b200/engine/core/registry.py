"""Which executor serves which ``(family, task)``.

A plain mapping with two guarantees the engine relies on: a pair is claimed once (a second
registration is a configuration error, not an override), and a miss says what *is* available.
Same contract as the reference's registry (``vrl/engine/core/registry.py:10-42``).
"""

from __future__ import annotations

from typing import Iterator, NamedTuple

from visionrl_b200.engine.core.protocols import FamilyPipelineExecutor


class ExecutorKey(NamedTuple):
    family: str
    task: str


class FamilyPipelineRegistry:
    def __init__(self, executors: tuple[FamilyPipelineExecutor, ...] = ()) -> None:
        self._by_key: dict[ExecutorKey, FamilyPipelineExecutor] = {}
        for executor in executors:
            self.register(executor)

    def register(self, executor: FamilyPipelineExecutor) -> None:
        key = ExecutorKey(executor.family, executor.task)
        if self._by_key.setdefault(key, executor) is not executor:
            raise ValueError(
                f"Generation executor already registered for family={key.family!r}, task={key.task!r}")

    def resolve(self, family: str, task: str) -> FamilyPipelineExecutor:
        try:
            return self._by_key[ExecutorKey(family, task)]
        except KeyError:
            raise NotImplementedError(
                f"No generation executor registered for family={family!r}, task={task!r}; "
                f"registered={sorted(tuple(k) for k in self._by_key)}") from None

    def __contains__(self, key: object) -> bool:
        return key in self._by_key

    def __iter__(self) -> Iterator[ExecutorKey]:
        return iter(sorted(self._by_key))

    def __len__(self) -> int:
        return len(self._by_key)
