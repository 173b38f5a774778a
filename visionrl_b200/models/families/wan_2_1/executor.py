"""Wan-2.1 text-to-video executor (reference: ``vrl/models/families/wan_2_1/executor.py:17-59``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.engine.diffusion import DiffusionPipelineExecutorBase, repeat_tensor_batch


class Wan_2_1PipelineExecutor(DiffusionPipelineExecutorBase):
    family = "wan_2_1"
    task = "t2v"
    default_num_frames = 33
    default_max_sequence_length = 512

    def __init__(self, model: Any, *, sample_batch_size: int = 1) -> None:
        self.model = model
        self.default_sample_batch_size = max(1, int(sample_batch_size))

    def build_chunk_encoded(self, *, encoded, generation_request, video_request, spec, chunk):
        del generation_request, video_request, spec
        return {k: repeat_tensor_batch(encoded[k], chunk.sample_count)
                for k in ("prompt_embeds", "negative_prompt_embeds") if encoded.get(k) is not None}


__all__ = ["Wan_2_1PipelineExecutor"]
