"""SD3.5 text-to-image executor (reference: ``vrl/models/families/sd3_5/executor.py:17-69``)."""

from __future__ import annotations

from typing import Any

from visionrl_b200.engine.diffusion import DiffusionPipelineExecutorBase, repeat_tensor_batch


class SD3_5PipelineExecutor(DiffusionPipelineExecutorBase):
    family = "sd3_5"
    task = "t2i"
    default_num_frames = 1
    default_max_sequence_length = 128

    def __init__(self, model: Any, *, sample_batch_size: int = 8) -> None:
        self.model = model
        self.default_sample_batch_size = max(1, int(sample_batch_size))

    def build_chunk_encoded(self, *, encoded, generation_request, video_request, spec, chunk):
        del generation_request, video_request, spec
        keys = ("prompt_embeds", "pooled_prompt_embeds", "negative_prompt_embeds",
                "negative_pooled_prompt_embeds")
        return {k: repeat_tensor_batch(encoded[k], chunk.sample_count)
                for k in keys if encoded.get(k) is not None}


__all__ = ["SD3_5PipelineExecutor"]
