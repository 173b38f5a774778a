"""Parsed sampling fields of a diffusion request (reference: ``vrl/engine/diffusion/spec.py:8-41``)."""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True, slots=True)
class BaseDiffusionGenerationSpec:
    num_steps: int
    guidance_scale: float
    height: int
    width: int
    num_frames: int = 1
    fps: int | None = None
    sample_batch_size: int = 1
    max_sequence_length: int = 512
    seed: int | None = None
    negative_prompt: str | None = None


@dataclass(frozen=True, slots=True)
class SDEDiffusionSpec:
    noise_level: float = 1.0
    sde_type: str = "sde"
    sde_window_size: int = 0
    sde_window_range: tuple[int, int] = (0, 0)
    same_latent: bool = False
    return_kl: bool = False


@dataclass(frozen=True, slots=True)
class DiffusionGenerationSpec:
    base: BaseDiffusionGenerationSpec
    sde: SDEDiffusionSpec | None = None


__all__ = ["BaseDiffusionGenerationSpec", "DiffusionGenerationSpec", "SDEDiffusionSpec"]
