"""Autoregressive policy protocol and per-row cache helpers
(reference: ``vrl/models/ar.py:25-150``).

``ar_split_rows`` / ``ar_concat_rows`` walk nested tuples / lists / mappings whose
tensors carry the batch on dim 0, so rows that reached different lengths under
partial scheduling can be regrouped.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
from contextlib import AbstractContextManager
from dataclasses import dataclass, field
from typing import Any, Protocol, runtime_checkable

import torch


@dataclass(slots=True)
class ARStepResult:
    """One scheduled token step; all values follow the order of ``sequence_ids``."""

    sequence_ids: list[str]
    positions: list[int]
    token: Any
    log_prob: Any
    replay_extras: dict[str, Any] = field(default_factory=dict)


def _legacy(value: Any) -> Any:
    to_legacy = getattr(value, "to_legacy_cache", None)
    return to_legacy() if callable(to_legacy) else value


def ar_split_rows(value: Any, batch_size: int) -> list[Any]:
    if batch_size < 1:
        raise ValueError("batch_size must be >= 1")
    value = _legacy(value)
    if isinstance(value, torch.Tensor):
        if value.shape[0] != batch_size:
            raise ValueError(
                f"cannot split tensor with batch={value.shape[0]} into {batch_size} rows")
        return [value[i:i + 1] for i in range(batch_size)]
    if isinstance(value, Mapping):
        parts = {k: ar_split_rows(v, batch_size) for k, v in value.items()}
        return [type(value)((k, p[i]) for k, p in parts.items()) for i in range(batch_size)]
    if isinstance(value, (tuple, list)):
        parts = [ar_split_rows(v, batch_size) for v in value]
        return [type(value)(p[i] for p in parts) for i in range(batch_size)]
    return [value] * batch_size


def ar_concat_rows(values: Sequence[Any]) -> Any:
    if not values:
        raise ValueError("values must be non-empty")
    values = [_legacy(v) for v in values]
    head = values[0]
    if isinstance(head, torch.Tensor):
        return torch.cat(list(values), dim=0)
    if isinstance(head, Mapping):
        return type(head)((k, ar_concat_rows([v[k] for v in values])) for k in head)
    if isinstance(head, (tuple, list)):
        return type(head)(ar_concat_rows([v[i] for v in values]) for i in range(len(head)))
    if any(v != head for v in values[1:]):
        raise ValueError("cannot concatenate non-tensor AR values that differ")
    return head


@runtime_checkable
class AutoregressivePolicy(Protocol):
    @property
    def device(self) -> torch.device: ...

    def disable_adapter(self) -> AbstractContextManager[None]: ...

    def replay_forward(self, batch: Any, timestep_idx: int = 0) -> dict[str, Any]:
        """Discrete families return ``{"logits", "image_token_ids"}``; continuous
        families return ``{"log_probs", ...}``.  Evaluators dispatch on the keys."""
        ...


__all__ = ["ARStepResult", "AutoregressivePolicy", "ar_concat_rows", "ar_split_rows"]
