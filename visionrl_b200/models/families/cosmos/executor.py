"""Cosmos video-to-world executor: threads the reference image (constructor default, or
``request.metadata["reference_image"]`` when present) into ``encode_prompt`` and ``prepare_sampling``
(reference: ``vrl/models/families/cosmos/executor.py:17-116``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.engine.diffusion import DiffusionPipelineExecutorBase, repeat_tensor_batch


class CosmosPipelineExecutor(DiffusionPipelineExecutorBase):
    family = "cosmos"
    task = "v2w"
    default_num_frames = 93
    default_fps = 16
    default_max_sequence_length = 512
    respect_cfg_flag = False

    def __init__(self, model: Any, *, sample_batch_size: int = 8, reference_image: Any = None) -> None:
        self.model = model
        self.default_sample_batch_size = max(1, int(sample_batch_size))
        self.reference_image = reference_image

    def _reference_image(self, generation_request: Any) -> Any:
        override = (generation_request.metadata or {}).get("reference_image")
        return override if override is not None else self.reference_image

    def encode_prompt_for_chunk(self, *, generation_request, video_request, spec, chunk):
        # the reference image reaches the encoder as well as the sampler preparation
        return self.model.encode_prompt(
            chunk.prompt, video_request.negative_prompt or None,
            max_sequence_length=spec.base.max_sequence_length,
            guidance_scale=spec.base.guidance_scale, request=video_request,
            reference_image=self._reference_image(generation_request))

    def build_chunk_encoded(self, *, encoded, generation_request, video_request, spec, chunk):
        del generation_request, video_request, spec
        return {k: repeat_tensor_batch(encoded[k], chunk.sample_count)
                for k in ("prompt_embeds", "negative_prompt_embeds") if encoded.get(k) is not None}

    def build_prepare_kwargs(self, *, encoded, generation_request, video_request, spec, chunk):
        del encoded, video_request, spec, chunk
        return {"reference_image": self._reference_image(generation_request)}


__all__ = ["CosmosPipelineExecutor"]
