"""Bookkeeping of one autoregressive sample while it is being decoded.

The decode loop of this package advances whole batches on the device (one CUDA-graph replay per
position), so the host-side record of a sequence is deliberately small: an immutable *batching key*
(what must agree for two sequences to share a token-forward batch) plus a position counter that
saturates at ``max_new_tokens``.  ``finished`` is derived from the counter unless the sequence was
closed early.  Field names and constructor keywords follow the reference's record
(``vrl/engine/ar/sequence.py:9-73``), which callers and schedulers rely on.
"""

from __future__ import annotations

from typing import Any, NamedTuple


class ARSequenceKey(NamedTuple):
    """Sequences may share a token-forward batch only if their keys are equal."""

    family: str
    task: str
    tokenizer_key: str
    dtype: str
    max_new_tokens: int


class ActiveSequence:
    __slots__ = ("request_id", "sample_id", "key", "position", "metadata", "_closed")

    def __init__(self, request_id: str, sample_id: str, family: str, task: str, tokenizer_key: str,
                 dtype: str, max_new_tokens: int, position: int = 0, finished: bool = False,
                 metadata: dict[str, Any] | None = None) -> None:
        for label, value in (("request_id", request_id), ("sample_id", sample_id)):
            if not value:
                raise ValueError(f"ActiveSequence.{label} must be non-empty")
        if max_new_tokens < 1:
            raise ValueError("ActiveSequence.max_new_tokens must be >= 1")
        if position < 0:
            raise ValueError("ActiveSequence.position must be >= 0")
        self.request_id = request_id
        self.sample_id = sample_id
        self.key = ARSequenceKey(family, task, tokenizer_key, dtype, int(max_new_tokens))
        self.position = int(position)
        self.metadata: dict[str, Any] = {} if metadata is None else metadata
        self._closed = bool(finished)

    # the key's fields read through, so a sequence still looks like a flat record
    family = property(lambda self: self.key.family)
    task = property(lambda self: self.key.task)
    tokenizer_key = property(lambda self: self.key.tokenizer_key)
    dtype = property(lambda self: self.key.dtype)
    max_new_tokens = property(lambda self: self.key.max_new_tokens)

    @property
    def finished(self) -> bool:
        return self._closed or self.position >= self.key.max_new_tokens

    @finished.setter
    def finished(self, value: bool) -> None:
        self._closed = bool(value)

    @property
    def remaining_tokens(self) -> int:
        return max(0, self.key.max_new_tokens - self.position)

    def advance(self, steps: int = 1) -> None:
        if steps < 1:
            raise ValueError("steps must be >= 1")
        if not self.finished:
            self.position = min(self.position + steps, self.key.max_new_tokens)

    def mark_finished(self) -> None:
        self.position = min(self.position, self.key.max_new_tokens)
        self._closed = True

    def __repr__(self) -> str:
        return (f"ActiveSequence({self.request_id}/{self.sample_id}, {self.position}/"
                f"{self.key.max_new_tokens}{', finished' if self.finished else ''})")


__all__ = ["ARSequenceKey", "ActiveSequence"]
