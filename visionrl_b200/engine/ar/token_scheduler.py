"""Token-level batching of active sequences inside an AR executor.

``pop_batch`` takes the first pending ``(key, position)`` group in arrival order
and returns at most ``max_batch_size`` of its sequences; unfinished sequences
return through ``push_back_unfinished`` (reference:
``vrl/engine/ar/token_scheduler.py:10-90``).
"""

from __future__ import annotations

from dataclasses import dataclass

from visionrl_b200.engine.ar.sequence import ActiveSequence, ARSequenceKey


@dataclass(slots=True)
class ARTokenBatch:
    key: ARSequenceKey
    sequences: list[ActiveSequence]

    def __post_init__(self) -> None:
        if not self.sequences:
            raise ValueError("ARTokenBatch.sequences must be non-empty")
        if any(seq.key != self.key for seq in self.sequences):
            raise ValueError("ARTokenBatch sequences must share the same key")

    @property
    def request_ids(self) -> list[str]:
        return [s.request_id for s in self.sequences]

    @property
    def sample_ids(self) -> list[str]:
        return [s.sample_id for s in self.sequences]


class ARTokenScheduler:
    def __init__(self, max_batch_size: int) -> None:
        if max_batch_size < 1:
            raise ValueError("max_batch_size must be >= 1")
        self.max_batch_size = max_batch_size
        self._pending: list[ActiveSequence] = []

    def __len__(self) -> int:
        return sum(1 for s in self._pending if not s.finished)

    def add(self, sequence: ActiveSequence) -> None:
        if not sequence.finished:
            self._pending.append(sequence)

    def add_many(self, sequences: list[ActiveSequence]) -> None:
        for s in sequences:
            self.add(s)

    def pop_batch(self) -> ARTokenBatch | None:
        live = [s for s in self._pending if not s.finished]
        if not live:
            self._pending = []
            return None
        lead = (live[0].key, live[0].position)
        picked: list[ActiveSequence] = []
        rest: list[ActiveSequence] = []
        for s in live:
            if len(picked) < self.max_batch_size and (s.key, s.position) == lead:
                picked.append(s)
            else:
                rest.append(s)
        self._pending = rest
        return ARTokenBatch(key=lead[0], sequences=picked)

    def push_back_unfinished(self, batch: ARTokenBatch) -> None:
        self._pending.extend(s for s in batch.sequences if not s.finished)


__all__ = ["ARTokenBatch", "ARTokenScheduler"]
