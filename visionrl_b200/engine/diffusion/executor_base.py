"""Shared ``GenerationRequest`` → diffusion ``OutputBatch`` path.

``forward`` plans prompt-major micro-batches of at most ``sample_batch_size``
samples, runs them with out-of-memory bisection and gathers; ``forward_chunk`` /
``gather_chunks`` expose the same work to a distributed backend.  Families
override the three hooks at the bottom (reference:
``vrl/engine/diffusion/executor_base.py:40-317``).
"""

from __future__ import annotations

from collections.abc import Sequence
from typing import Any

from visionrl_b200.engine.batching import forward_batch_by_merging_prompts
from visionrl_b200.engine.core.types import (
    GenerationRequest, GenerationSampleSpec, OutputBatch, WorkloadSignature,
)
from visionrl_b200.engine.diffusion.denoise import (
    DiffusionChunkResult, DiffusionDenoiseConfig, repeat_tensor_batch,
    run_diffusion_denoise_chunk, select_sde_window,
)
from visionrl_b200.engine.diffusion.spec import (
    BaseDiffusionGenerationSpec, DiffusionGenerationSpec, SDEDiffusionSpec,
)
from visionrl_b200.engine.gather import gather_diffusion_chunks
from visionrl_b200.engine.microbatching import (
    MicroBatchPlan, plan_prompt_group_microbatches, run_microbatches_with_oom_retry,
)
from visionrl_b200.models.diffusion import VideoGenerationRequest


def _window_range(value: Any) -> tuple[int, int]:
    try:
        return int(value[0]), int(value[1])
    except (TypeError, IndexError, ValueError) as exc:
        raise ValueError("sampling.sde_window_range must contain two integer values") from exc


def _sde_type(value: Any) -> str:
    if str(value) not in ("sde", "cps"):
        raise ValueError("sampling.sde_type must be 'sde' or 'cps'")
    return str(value)


class DiffusionPipelineExecutorBase:
    family: str
    task: str
    model: Any
    default_sample_batch_size: int = 1
    default_num_frames: int = 1
    default_fps: int | None = None
    default_max_sequence_length: int = 512
    respect_cfg_flag: bool = True
    sde_type: str = "sde"
    include_max_sequence_length_extra: bool = True

    def workload_signature(self, request: GenerationRequest) -> WorkloadSignature:
        return WorkloadSignature.from_request(request)

    def parse_spec(self, request: GenerationRequest) -> DiffusionGenerationSpec:
        s = request.sampling
        steps = int(s["num_steps"])
        fps = s.get("fps", self.default_fps)
        seed = s.get("seed")
        base = BaseDiffusionGenerationSpec(
            num_steps=steps, guidance_scale=float(s["guidance_scale"]), height=int(s["height"]),
            width=int(s["width"]),
            num_frames=int(s.get("num_frames", s.get("frame_count", self.default_num_frames))),
            fps=None if fps is None else int(fps),
            sample_batch_size=max(1, int(s.get("sample_batch_size", self.default_sample_batch_size))),
            max_sequence_length=int(s.get("max_sequence_length", self.default_max_sequence_length)),
            seed=None if seed is None else int(seed), negative_prompt=s.get("negative_prompt"),
        )
        sde = SDEDiffusionSpec(
            noise_level=float(s.get("noise_level", 1.0)),
            sde_type=_sde_type(s.get("sde_type", self.sde_type)),
            sde_window_size=int(s.get("sde_window_size", 0)),
            sde_window_range=_window_range(s.get("sde_window_range", (0, steps))),
            same_latent=bool(s.get("same_latent", False)), return_kl=bool(s.get("return_kl", False)),
        )
        return DiffusionGenerationSpec(base=base, sde=sde)

    def build_video_request(self, prompt: str, spec: DiffusionGenerationSpec) -> VideoGenerationRequest:
        b = spec.base
        kwargs: dict[str, Any] = dict(prompt=prompt, num_steps=b.num_steps,
                                      guidance_scale=b.guidance_scale, height=b.height,
                                      width=b.width, frame_count=b.num_frames)
        if b.fps is not None:
            kwargs["fps"] = b.fps
        if b.negative_prompt is not None:
            kwargs["negative_prompt"] = b.negative_prompt
        if b.seed is not None:
            kwargs["seed"] = b.seed
        extra = self.build_video_request_extra(spec)
        if extra:
            kwargs["extra"] = extra
        return VideoGenerationRequest(**kwargs)

    def build_video_request_extra(self, spec: DiffusionGenerationSpec) -> dict[str, Any]:
        if not self.include_max_sequence_length_extra:
            return {}
        return {"max_sequence_length": spec.base.max_sequence_length}

    def build_denoise_config(self, spec: DiffusionGenerationSpec,
                             chunk: MicroBatchPlan) -> DiffusionDenoiseConfig:
        if spec.sde is None:
            raise NotImplementedError(
                f"{type(self).__name__} must override denoise for non-SDE diffusion")
        return DiffusionDenoiseConfig(
            sample_start=chunk.sample_start, seed=spec.base.seed, same_latent=spec.sde.same_latent,
            sde_window=select_sde_window(spec.sde.sde_window_size, spec.sde.sde_window_range),
            return_kl=spec.sde.return_kl, noise_level=spec.sde.noise_level,
            sde_type=spec.sde.sde_type,
        )

    def forward(self, request: GenerationRequest,
                sample_specs: list[GenerationSampleSpec]) -> OutputBatch:
        spec = self.parse_spec(request)
        plan = plan_prompt_group_microbatches(
            list(request.prompts), int(request.samples_per_prompt), spec.base.sample_batch_size)
        # every prompt is encoded once, however many micro-batches its group is split into
        encoded_by_prompt: dict[int, Any] = {}
        chunks = run_microbatches_with_oom_retry(
            plan.micro_batches,
            lambda mb: self.forward_chunk(request, mb, encoded_cache=encoded_by_prompt))
        return self.gather_chunks(request, sample_specs, chunks)

    def forward_chunk(self, request: GenerationRequest, chunk: MicroBatchPlan,
                      encoded_cache: dict[int, Any] | None = None) -> DiffusionChunkResult:
        spec = self.parse_spec(request)
        video_request = self.build_video_request(chunk.prompt, spec)
        hook = dict(generation_request=request, video_request=video_request, spec=spec, chunk=chunk)
        if encoded_cache is not None and chunk.prompt_index in encoded_cache:
            encoded = encoded_cache[chunk.prompt_index]
        else:
            encoded = self.encode_prompt_for_chunk(**hook)
            if encoded_cache is not None:
                encoded_cache[chunk.prompt_index] = encoded
        return run_diffusion_denoise_chunk(
            policy=self.model, request=video_request,
            encoded=self.build_chunk_encoded(encoded=encoded, **hook),
            config=self.build_denoise_config(spec, chunk),
            prepare_kwargs=self.build_prepare_kwargs(encoded=encoded, **hook),
        )

    def gather_chunks(self, request: GenerationRequest, sample_specs: Sequence[GenerationSampleSpec],
                      chunks: Sequence[DiffusionChunkResult]) -> OutputBatch:
        return gather_diffusion_chunks(request, sample_specs, chunks, model_family=self.family,
                                       respect_cfg_flag=self.respect_cfg_flag)

    def forward_batch(self, requests, sample_specs_by_request):
        return forward_batch_by_merging_prompts(self, requests, sample_specs_by_request)

    # -- family hooks ----------------------------------------------------------------
    def encode_prompt_for_chunk(self, *, generation_request, video_request, spec, chunk):
        del generation_request
        return self.model.encode_prompt(
            chunk.prompt, video_request.negative_prompt or None,
            max_sequence_length=spec.base.max_sequence_length,
            guidance_scale=spec.base.guidance_scale, request=video_request,
        )

    def build_chunk_encoded(self, *, encoded, generation_request, video_request, spec, chunk):
        del generation_request, video_request, spec
        return {k: repeat_tensor_batch(v, chunk.sample_count) for k, v in encoded.items()}

    def build_prepare_kwargs(self, *, encoded, generation_request, video_request, spec, chunk):
        del encoded, generation_request, video_request, spec, chunk
        return None


__all__ = ["DiffusionPipelineExecutorBase"]
