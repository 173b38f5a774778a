"""``GenerationRequest`` → ``OutputBatch`` for every diffusion family.

The executor is what a rollout backend drives: ``forward`` runs a whole request on this device,
``forward_chunk`` one chunk of it (the unit the SPMD runtime deals over ranks) and
``gather_chunks`` assembles chunk results.  A chunk is processed in four moves:

1. the request's ``sampling`` mapping is read ONCE into a typed ``DiffusionGenerationSpec``
   (:class:`_Sampling` does the reading: defaults of the family, type coercion, validation);
2. the chunk's prompt is encoded — once per prompt and request, however many chunks its group
   was cut into (``_EncodedPrompts``) — and the encoding is expanded to the chunk's samples;
3. the denoise loop runs (``run_diffusion_denoise_chunk``);
4. nothing is copied off the device.

Families customise steps 2 and 3 through the three hooks at the bottom and the class attributes
at the top.  Behavioural reference: ``vrl/engine/diffusion/executor_base.py:40-317``.
"""

from __future__ import annotations

from collections.abc import Mapping, Sequence
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
    BisectingRunner, MicroBatchPlan, plan_prompt_group_microbatches,
)
from visionrl_b200.models.diffusion import VideoGenerationRequest

_SDE_TYPES = ("sde", "cps")


class _Sampling:
    """Typed reads of a request's ``sampling`` mapping."""

    def __init__(self, values: Mapping[str, Any]) -> None:
        self._values = values

    def need(self, key: str, kind: type) -> Any:
        return kind(self._values[key])

    def take(self, key: str, kind: type, default: Any) -> Any:
        value = self._values.get(key, default)
        return None if value is None else kind(value)

    def first(self, keys: tuple[str, ...], kind: type, default: Any) -> Any:
        for key in keys:
            if key in self._values:
                return kind(self._values[key])
        return kind(default)

    def window(self, key: str, default: tuple[int, int]) -> tuple[int, int]:
        raw = self._values.get(key, default)
        try:
            lo, hi = raw[0], raw[1]
            return int(lo), int(hi)
        except (TypeError, IndexError, ValueError) as exc:
            raise ValueError(f"sampling.{key} must contain two integer values") from exc

    def choice(self, key: str, allowed: tuple[str, ...], default: str) -> str:
        value = str(self._values.get(key, default))
        if value not in allowed:
            raise ValueError(f"sampling.{key} must be " + " or ".join(repr(a) for a in allowed))
        return value


class _EncodedPrompts:
    """Prompt encodings of one request, keyed by prompt index."""

    def __init__(self, store: dict[int, Any] | None) -> None:
        self._store = store

    def get(self, index: int, encode) -> Any:
        if self._store is None:
            return encode()
        if index not in self._store:
            self._store[index] = encode()
        return self._store[index]


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

    # -- request → typed spec ---------------------------------------------------------------
    def parse_spec(self, request: GenerationRequest) -> DiffusionGenerationSpec:
        s = _Sampling(request.sampling)
        steps = s.need("num_steps", int)
        base = BaseDiffusionGenerationSpec(
            num_steps=steps, guidance_scale=s.need("guidance_scale", float),
            height=s.need("height", int), width=s.need("width", int),
            num_frames=s.first(("num_frames", "frame_count"), int, self.default_num_frames),
            fps=s.take("fps", int, self.default_fps),
            sample_batch_size=max(1, s.take("sample_batch_size", int, self.default_sample_batch_size)),
            max_sequence_length=s.take("max_sequence_length", int, self.default_max_sequence_length),
            seed=s.take("seed", int, None), negative_prompt=s.take("negative_prompt", str, None))
        sde = SDEDiffusionSpec(
            noise_level=s.take("noise_level", float, 1.0),
            sde_type=s.choice("sde_type", _SDE_TYPES, self.sde_type),
            sde_window_size=s.take("sde_window_size", int, 0),
            sde_window_range=s.window("sde_window_range", (0, steps)),
            same_latent=s.take("same_latent", bool, False), return_kl=s.take("return_kl", bool, False))
        return DiffusionGenerationSpec(base=base, sde=sde)

    def build_video_request_extra(self, spec: DiffusionGenerationSpec) -> dict[str, Any]:
        if not self.include_max_sequence_length_extra:
            return {}
        return {"max_sequence_length": spec.base.max_sequence_length}

    def build_video_request(self, prompt: str, spec: DiffusionGenerationSpec) -> VideoGenerationRequest:
        base = spec.base
        fields: dict[str, Any] = {
            "prompt": prompt, "num_steps": base.num_steps, "guidance_scale": base.guidance_scale,
            "height": base.height, "width": base.width, "frame_count": base.num_frames,
            # optional fields are passed only when set, so the request's own defaults apply
            "fps": base.fps, "negative_prompt": base.negative_prompt, "seed": base.seed,
            "extra": self.build_video_request_extra(spec) or None,
        }
        return VideoGenerationRequest(**{k: v for k, v in fields.items() if v is not None})

    def build_denoise_config(self, spec: DiffusionGenerationSpec,
                             chunk: MicroBatchPlan) -> DiffusionDenoiseConfig:
        sde = spec.sde
        if sde is None:
            raise NotImplementedError(
                f"{type(self).__name__} must override denoise for non-SDE diffusion")
        return DiffusionDenoiseConfig(
            sample_start=chunk.sample_start, seed=spec.base.seed, same_latent=sde.same_latent,
            sde_window=select_sde_window(sde.sde_window_size, sde.sde_window_range),
            return_kl=sde.return_kl, noise_level=sde.noise_level, sde_type=sde.sde_type)

    # -- execution -------------------------------------------------------------------------------
    def forward(self, request: GenerationRequest,
                sample_specs: list[GenerationSampleSpec]) -> OutputBatch:
        spec = self.parse_spec(request)
        plan = plan_prompt_group_microbatches(list(request.prompts), int(request.samples_per_prompt),
                                              spec.base.sample_batch_size)
        encodings: dict[int, Any] = {}
        runner = BisectingRunner(lambda c: self.forward_chunk(request, c, encoded_cache=encodings))
        return self.gather_chunks(request, sample_specs, runner.run(plan.micro_batches))

    def forward_chunk(self, request: GenerationRequest, chunk: MicroBatchPlan,
                      encoded_cache: dict[int, Any] | None = None) -> DiffusionChunkResult:
        spec = self.parse_spec(request)
        video_request = self.build_video_request(chunk.prompt, spec)
        hook = {"generation_request": request, "video_request": video_request, "spec": spec,
                "chunk": chunk}
        encoded = _EncodedPrompts(encoded_cache).get(
            chunk.prompt_index, lambda: self.encode_prompt_for_chunk(**hook))
        return run_diffusion_denoise_chunk(
            policy=self.model, request=video_request,
            encoded=self.build_chunk_encoded(encoded=encoded, **hook),
            config=self.build_denoise_config(spec, chunk),
            prepare_kwargs=self.build_prepare_kwargs(encoded=encoded, **hook))

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
            guidance_scale=spec.base.guidance_scale, request=video_request)

    def build_chunk_encoded(self, *, encoded, generation_request, video_request, spec, chunk):
        del generation_request, video_request, spec
        return {name: repeat_tensor_batch(value, chunk.sample_count)
                for name, value in encoded.items()}

    def build_prepare_kwargs(self, *, encoded, generation_request, video_request, spec, chunk):
        del encoded, generation_request, video_request, spec, chunk
        return None


__all__ = ["DiffusionPipelineExecutorBase"]
