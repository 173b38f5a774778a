"""Trainer-side batch assembled from one or more generation outputs
(reference: ``vrl/rollouts/batch.py:9-80``)."""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass
class RolloutBatch:
    observations: Any            # [B, T, ...]  state before each step
    actions: Any                 # [B, T, ...]  state after each step / sampled tokens
    rewards: Any                 # [B]
    dones: Any                   # [B]
    group_ids: Any               # [B] prompt group of every sample
    extras: dict[str, Any] = field(default_factory=dict)    # per-sample tensors
    context: dict[str, Any] = field(default_factory=dict)   # shared scalars, never stacked
    videos: Any | None = None
    prompts: list[str] | None = None


def stack_batches(batches: list[RolloutBatch]) -> RolloutBatch:
    """Concatenate along the sample axis; ``context`` and non-tensor extras come from the first."""
    import torch

    if len(batches) == 1:
        return batches[0]
    cat = lambda name: torch.cat([getattr(b, name) for b in batches], dim=0)  # noqa: E731
    head = batches[0]
    extras = {
        k: torch.cat([b.extras[k] for b in batches], dim=0) if isinstance(v, torch.Tensor) else v
        for k, v in head.extras.items()
    }
    videos = cat("videos") if all(b.videos is not None for b in batches) else None
    prompts = [p for b in batches if b.prompts is not None for p in b.prompts]
    return RolloutBatch(
        observations=cat("observations"), actions=cat("actions"), rewards=cat("rewards"),
        dones=cat("dones"), group_ids=cat("group_ids"), extras=extras,
        context=dict(head.context), videos=videos, prompts=prompts or None,
    )
