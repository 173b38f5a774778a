"""NextStep-1 continuous-token executor (reference:
``vrl/models/families/nextstep_1/executor.py:64-570``).  Same structure as the discrete
executor; chunks carry the continuous tokens, their log-probs and the saved prior noise."""

from __future__ import annotations

from collections.abc import Sequence
from dataclasses import dataclass
from typing import Any

import torch

from visionrl_b200.engine.ar import (
    ActiveSequence, ARPipelineExecutorBase, ARTokenScheduler, ordered_chunks,
)
from visionrl_b200.engine.core.protocols import PipelineChunkResult
from visionrl_b200.engine.core.types import (
    GenerationMetrics, GenerationRequest, GenerationSampleSpec, OutputBatch, RolloutTrajectoryData,
    WorkloadSignature,
)
from visionrl_b200.engine.microbatching import MicroBatchPlan

_ROW_FIELDS = ("output", "tokens", "log_probs", "saved_noise", "prompt_input_ids",
               "prompt_attention_mask", "uncond_input_ids", "uncond_attention_mask")


@dataclass(slots=True)
class NextStep1ARChunkResult(PipelineChunkResult):
    prompt_index: int
    sample_start: int
    sample_count: int
    output: torch.Tensor
    tokens: torch.Tensor
    log_probs: torch.Tensor
    saved_noise: torch.Tensor
    prompt_input_ids: torch.Tensor
    prompt_attention_mask: torch.Tensor
    uncond_input_ids: torch.Tensor
    uncond_attention_mask: torch.Tensor
    context: dict[str, Any]
    peak_memory_mb: float | None = None

    @property
    def images_for_reward(self) -> torch.Tensor:
        """What reward models see of this chunk: ``[0, 1]`` pixels when the request asked for the
        rescale (``context["rescale_to_unit"]``, the default), else the decoder's own range."""
        if self.context.get("rescale_to_unit", True):
            return ((self.output + 1.0) * 0.5).clamp(0.0, 1.0)
        return self.output


def _pack(request, sample_specs, fields, context, steps, micro_batches, peak) -> OutputBatch:
    extra = {k: fields[k] for k in _ROW_FIELDS if k != "output"}
    extra["context"] = dict(context)
    # what reward models see: [0, 1] pixels when asked for, otherwise the decoder's own range
    images = fields["output"]
    extra["images_for_reward"] = ((images + 1.0) * 0.5).clamp(0.0, 1.0) if context.get("rescale_to_unit", True) \
        else images
    return OutputBatch(
        request_id=request.request_id, family=request.family, task=request.task,
        prompts=list(request.prompts), sample_specs=list(sample_specs), output=fields["output"],
        # continuous tokens have no denoising trajectory; the log-probabilities are carried here too
        rollout_trajectory_data=RolloutTrajectoryData(rollout_log_probs=fields["log_probs"]), extra=extra,
        metrics=GenerationMetrics(num_prompts=len(request.prompts), num_samples=len(sample_specs),
                                  num_steps=steps, micro_batches=micro_batches, peak_memory_mb=peak),
        peak_memory_mb=peak or 0.0)


class NextStep1ChunkGatherer:
    def gather_chunks(self, request: GenerationRequest, sample_specs: Sequence[GenerationSampleSpec],
                      chunks: Sequence[NextStep1ARChunkResult]) -> OutputBatch:
        ordered = ordered_chunks(request, sample_specs, chunks, row_fields=_ROW_FIELDS)
        fields = {k: torch.cat([getattr(c, k) for c in ordered], dim=0) for k in _ROW_FIELDS}
        peaks = [c.peak_memory_mb for c in ordered if c.peak_memory_mb is not None]
        return _pack(request, sample_specs, fields, ordered[0].context,
                     int(fields["tokens"].shape[1]), len(ordered), max(peaks) if peaks else None)


class NextStep1PipelineExecutor(ARPipelineExecutorBase):
    family = "nextstep_1"
    task = "ar_t2i"
    default_image_token_num = 1024
    default_image_size = 256
    default_max_text_length = 256

    def __init__(self, model: Any) -> None:
        self.model = model
        self._gatherer = NextStep1ChunkGatherer()

    def workload_signature(self, request: GenerationRequest) -> WorkloadSignature:
        return WorkloadSignature.from_request(request)

    def _encode_texts(self, texts: list[str], max_length: int):
        """Token ids and mask from the policy's own tokenizer, or — for a policy that carries a
        Hugging Face style ``processor`` instead (the reference's policy contract) — from that."""
        device = self.model.device
        tok = getattr(self.model, "tokenizer", None)
        if tok is not None and hasattr(tok, "batch_encode"):
            return (*tok.batch_encode(list(texts), max_length, device), getattr(tok, "pad_id", 0))
        enc = self.model.processor(list(texts), return_tensors="pt", padding="max_length", truncation=True,
                                   max_length=max_length)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device), 0

    def _tokenize_prompts(self, prompts: list[str], max_length: int):
        c_ids, c_mask, pad = self._encode_texts(list(prompts), max_length)
        u_ids, u_mask, _ = self._encode_texts([""] * len(prompts), max_length)
        return self.align_pair(c_ids, c_mask, u_ids, u_mask, pad_id=pad)

    def _embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        embed = getattr(self.model, "embed_text", None)
        if callable(embed):
            return embed(token_ids)
        return self.model.language_model.get_input_embeddings()(token_ids)

    def _sample_with_ar_scheduler(self, *, request, sample_ids, cond_embeds, uncond_embeds,
                                  prompt_mask, uncond_mask, sample_kwargs, batch_size: int):
        state = self.model.init_ar_state(cond_embeds, uncond_embeds, prompt_mask, uncond_mask,
                                         **sample_kwargs)
        scheduler = ARTokenScheduler(max_batch_size=max(1, int(batch_size)))
        scheduler.add_many([
            ActiveSequence(request_id=request.request_id, sample_id=sid, family=self.family,
                           task=self.task, tokenizer_key="nextstep", dtype=str(getattr(self.model, "dtype", "float32")),
                           max_new_tokens=int(sample_kwargs["image_token_num"]), metadata={"row_index": row})
            for row, sid in enumerate(sample_ids)])
        while len(scheduler):
            batch = scheduler.pop_batch()
            if batch is None:
                break
            self.model.step_ar(state, batch.sequences)
            for seq in batch.sequences:
                seq.advance()
            scheduler.push_back_unfinished(batch)
        return self.model.finalize_ar_state(state)

    def _run_rows(self, request: GenerationRequest, prompts: list[str], sample_ids: list[str],
                  seed_offset: int):
        spec = self.parse_spec(request)
        # request values win; a policy without a config object gets the published defaults
        s, cfg = request.sampling, getattr(self.model, "config", None)
        kwargs = dict(cfg_scale=float(s.get("cfg_scale", getattr(cfg, "cfg_scale", 4.5))),
                      num_flow_steps=int(s.get("num_flow_steps", getattr(cfg, "num_flow_steps", 20))),
                      noise_level=float(s.get("noise_level", getattr(cfg, "noise_level", 1.0))),
                      image_token_num=spec.image_token_num)
        if spec.seed is not None:
            kwargs["generator"] = torch.Generator(device="cpu").manual_seed(int(spec.seed) + seed_offset)
        c_ids, c_mask, u_ids, u_mask = self._tokenize_prompts(prompts, spec.max_text_length)
        if spec.use_ar_scheduler:
            tokens, noise, log_probs = self._sample_with_ar_scheduler(
                request=request, sample_ids=sample_ids, cond_embeds=self._embed(c_ids),
                uncond_embeds=self._embed(u_ids), prompt_mask=c_mask, uncond_mask=u_mask,
                sample_kwargs=kwargs, batch_size=int(s.get("ar_scheduler_batch_size", len(prompts))))
        else:
            tokens, noise, log_probs = self.model.sample_image_tokens(
                self._embed(c_ids), self._embed(u_ids), c_mask, u_mask, **kwargs)
        images = self.model.decode_image_tokens(tokens, image_size=spec.image_size)
        fields = {"output": images, "tokens": tokens, "log_probs": log_probs, "saved_noise": noise,
                  "prompt_input_ids": c_ids, "prompt_attention_mask": c_mask,
                  "uncond_input_ids": u_ids, "uncond_attention_mask": u_mask}
        context = {"cfg_scale": kwargs["cfg_scale"], "num_flow_steps": kwargs["num_flow_steps"],
                   "noise_level": kwargs["noise_level"], "image_token_num": spec.image_token_num,
                   "image_size": spec.image_size,
                   "rescale_to_unit": bool(s.get("rescale_to_unit", True)),
                   "model_family": "nextstep_1"}
        return fields, context, spec.image_token_num

    def forward(self, request: GenerationRequest,
                sample_specs: list[GenerationSampleSpec]) -> OutputBatch:
        fields, context, steps = self._run_rows(request, self.expand_prompts(request),
                                                [s.sample_id for s in sample_specs], 0)
        return _pack(request, sample_specs, fields, context, steps, 1, self.peak_memory_mb())

    def forward_chunk(self, request: GenerationRequest, chunk: MicroBatchPlan) -> NextStep1ARChunkResult:
        self.validate_chunk(request, chunk)
        ids = [f"{request.request_id}:prompt:{chunk.prompt_index}:sample:{j}"
               for j in range(chunk.sample_start, chunk.sample_end)]
        fields, context, _ = self._run_rows(request, [chunk.prompt] * chunk.sample_count, ids,
                                            self.chunk_seed_offset(request, chunk))
        return NextStep1ARChunkResult(prompt_index=chunk.prompt_index,
                                      sample_start=chunk.sample_start,
                                      sample_count=chunk.sample_count, context=context,
                                      peak_memory_mb=self.peak_memory_mb(), **fields)

    def gather_chunks(self, request, sample_specs, chunks) -> OutputBatch:
        return self._gatherer.gather_chunks(request, sample_specs, chunks)


__all__ = ["NextStep1ARChunkResult", "NextStep1ChunkGatherer", "NextStep1PipelineExecutor"]
