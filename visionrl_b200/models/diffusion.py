"""``DiffusionPolicy`` — the one contract every diffusion family implements.

The engine drives sampling through ``encode_prompt`` → ``prepare_sampling`` →
``forward_step`` (one CFG-batched transformer forward, no scheduler step) →
``decode_latents``; the trainer replays a recorded step through
``replay_forward``.  ``SamplingState`` objects are private to a family: callers
use ``export_batch_context`` / ``export_training_extras`` / ``restore_eval_state``
(reference: ``vrl/models/diffusion.py:46-284``).
"""

from __future__ import annotations

import contextlib
from abc import ABC, abstractmethod
from collections.abc import Mapping
from dataclasses import dataclass, field
from typing import Any

import torch.nn as nn


@dataclass(slots=True)
class VideoGenerationRequest:
    """Per-request inference parameters; family-specific knobs go in ``extra``."""

    prompt: str = ""
    negative_prompt: str = ""
    references: list[str] = field(default_factory=list)
    task_type: str = "text_to_video"
    width: int = 1024
    height: int = 640
    frame_count: int = 16
    num_steps: int = 35
    guidance_scale: float = 5.0
    high_noise_guidance_scale: float | None = None
    seed: int | None = None
    model_name: str = ""
    model_size: str = "A14B"
    ckpt_dir: str | None = None
    fps: int = 16
    sample_solver: str = "dpmpp"
    shift: float = 1.0
    t5_cpu: bool = True
    convert_model_dtype: bool = True
    offload_model: bool = False
    action_sequence: list[list[float]] | None = None
    action_dim: int | None = None
    action_conditioning_mode: str = "none"
    extra: dict[str, Any] = field(default_factory=dict)


class DiffusionPolicy(nn.Module, ABC):
    family: str = "diffusion"

    async def load(self) -> None:
        return None

    def describe(self) -> dict[str, Any]:
        return {"family": self.family}

    # -- inference primitives ------------------------------------------------------
    @abstractmethod
    def encode_prompt(self, prompt, negative_prompt=None, **kwargs: Any) -> dict[str, Any]: ...

    @abstractmethod
    def prepare_sampling(self, request: VideoGenerationRequest, encoded: dict[str, Any],
                         **kwargs: Any) -> Any: ...

    @abstractmethod
    def forward_step(self, state: Any, step_idx: int) -> dict[str, Any]:
        """One transformer forward; returns at least ``{"noise_pred": Tensor}``."""

    def forward(self, state: Any, step_idx: int) -> dict[str, Any]:
        return self.forward_step(state, step_idx)

    @abstractmethod
    def decode_latents(self, latents: Any) -> Any:
        """Latents → frames (image ``[B,C,H,W]``, video ``[B,C,T,H,W]``)."""

    # -- collector boundary -------------------------------------------------------
    def export_batch_context(self, state: Any) -> dict[str, Any]:
        raise NotImplementedError

    def export_training_extras(self, state: Any) -> dict[str, Any]:
        raise NotImplementedError

    def restore_eval_state(self, batch_extras, batch_context, latents, step_idx) -> Any:
        raise NotImplementedError

    def replay_forward(self, batch: Any, timestep_idx: int) -> dict[str, Any]:
        """Rebuild the sampling state of step ``timestep_idx`` and run one forward.

        Eval states pack their timesteps as ``[1, B]`` so index 0 is right for
        families that read ``state.timesteps[step_idx]``; families that index a
        schedule by the true step override this method.
        """
        state = self.restore_eval_state(batch.extras, batch.context,
                                        batch.observations[:, timestep_idx], timestep_idx)
        return self.forward(state, 0)

    # -- trainer-facing helpers -----------------------------------------------------
    def _require_transformer(self) -> Any:
        transformer = getattr(self, "transformer", None)
        if transformer is None:
            raise RuntimeError(f"{type(self).__name__} has no registered trainable transformer")
        return transformer

    def disable_adapter(self) -> contextlib.AbstractContextManager[None]:
        transformer = self._require_transformer()
        disable = getattr(transformer, "disable_adapter", None)
        if not callable(disable):
            raise RuntimeError(f"{type(transformer).__name__} does not expose disable_adapter()")
        return disable()

    def load_trainable_state(self, state_dict: Mapping[str, Any]) -> Any:
        transformer = self._require_transformer()
        state = dict(state_dict)
        if not state:
            raise ValueError("load_trainable_state received an empty state dict")
        prefix = "transformer."
        bad = [k for k in state if not k.startswith(prefix)]
        if bad:
            raise ValueError(
                f"load_trainable_state only accepts policy keys prefixed with {prefix!r}; got {bad}"
            )
        sub = {k[len(prefix):]: v for k, v in state.items()}
        own = transformer.state_dict()
        unexpected = sorted(k for k in sub if k not in own)
        if unexpected:
            raise ValueError(f"load_trainable_state got keys the transformer does not have: {unexpected}")
        if len(sub) == len(own):
            return transformer.load_state_dict(sub, strict=True)
        # a partial payload must at least cover everything that trains (adapters or full weights)
        trainable = {n for n, p in transformer.named_parameters() if p.requires_grad}
        missing = sorted(trainable - sub.keys())
        if missing:
            raise ValueError(f"load_trainable_state payload misses trainable keys: {missing[:8]}"
                             f"{' ...' if len(missing) > 8 else ''}")
        return transformer.load_state_dict(sub, strict=False)

    def trainable_state_dict(self) -> dict[str, Any]:
        """``transformer.``-prefixed tensors of exactly the parameters that train, in name order —
        the payload of a trainer-to-rollout weight push."""
        transformer = self._require_transformer()
        return {f"transformer.{n}": p.detach() for n, p in sorted(transformer.named_parameters())
                if p.requires_grad}

    # -- backend ownership ------------------------------------------------------------
    @classmethod
    def from_spec(cls, spec: Any) -> "DiffusionPolicy":  # pragma: no cover
        raise NotImplementedError

    def apply_lora(self, spec: Any) -> None:  # pragma: no cover
        raise NotImplementedError

    def enable_full_finetune(self) -> None:  # pragma: no cover
        raise NotImplementedError

    def torch_compile_transformer(self, mode: str) -> None:  # pragma: no cover
        raise NotImplementedError

    def set_num_steps(self, n: int) -> None:  # pragma: no cover
        raise NotImplementedError

    @property
    def trainable_modules(self) -> dict[str, Any]:  # pragma: no cover
        raise NotImplementedError

    @property
    def scheduler(self) -> Any:  # pragma: no cover
        raise NotImplementedError

    @property
    def backend_handle(self) -> Any:  # pragma: no cover
        raise NotImplementedError


__all__ = ["DiffusionPolicy", "VideoGenerationRequest"]
