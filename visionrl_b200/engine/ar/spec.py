"""Family-neutral fields of an autoregressive image request
(reference: ``vrl/engine/ar/spec.py:8-21``)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True, slots=True)
class ARGenerationSpec:
    image_token_num: int
    image_size: int
    max_text_length: int
    seed: int | None
    use_ar_scheduler: bool


__all__ = ["ARGenerationSpec"]
