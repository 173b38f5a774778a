"""Janus-Pro autoregressive text-to-image executor.

Prompts are wrapped in the chat template, tokenised and right-padded to ``max_text_length``;
the unconditional branch uses the empty prompt; both are embedded, sampled with CFG (either
in one call or through the token scheduler in partial batches), and decoded by the VQ decoder
to images in ``[-1, 1]``.  Chunks carry ``(prompt_index, sample_start, sample_count)`` so a
model-free gatherer can reassemble them in prompt-major order
(reference: ``vrl/models/families/janus_pro/executor.py:64-560``).
"""

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
    GenerationMetrics, GenerationRequest, GenerationSampleSpec, OutputBatch, WorkloadSignature,
)
from visionrl_b200.engine.microbatching import MicroBatchPlan

_ROW_FIELDS = ("output", "token_ids", "token_log_probs", "token_mask", "prompt_input_ids",
               "prompt_attention_mask", "uncond_input_ids", "uncond_attention_mask")


@dataclass(slots=True)
class JanusProARChunkResult(PipelineChunkResult):
    prompt_index: int
    sample_start: int
    sample_count: int
    output: torch.Tensor
    token_ids: torch.Tensor
    token_log_probs: torch.Tensor
    token_mask: torch.Tensor
    prompt_input_ids: torch.Tensor
    prompt_attention_mask: torch.Tensor
    uncond_input_ids: torch.Tensor
    uncond_attention_mask: torch.Tensor
    context: dict[str, Any]
    peak_memory_mb: float | None = None


def _pack_output(request: GenerationRequest, sample_specs: Sequence[GenerationSampleSpec],
                 fields: dict[str, torch.Tensor], context: dict[str, Any], num_steps: int,
                 micro_batches: int, peak: float | None) -> OutputBatch:
    extra = {k: fields[k] for k in _ROW_FIELDS if k != "output"}
    extra["context"] = dict(context)
    return OutputBatch(
        request_id=request.request_id, family=request.family, task=request.task,
        prompts=list(request.prompts), sample_specs=list(sample_specs), output=fields["output"],
        rollout_trajectory_data=None, extra=extra,
        metrics=GenerationMetrics(num_prompts=len(request.prompts), num_samples=len(sample_specs),
                                  num_steps=num_steps, micro_batches=micro_batches,
                                  peak_memory_mb=peak),
        peak_memory_mb=peak or 0.0)


class JanusProChunkGatherer:
    """Pure (model-free) gatherer of Janus chunks."""

    def gather_chunks(self, request: GenerationRequest, sample_specs: Sequence[GenerationSampleSpec],
                      chunks: Sequence[JanusProARChunkResult]) -> OutputBatch:
        ordered = ordered_chunks(request, sample_specs, chunks, row_fields=_ROW_FIELDS)
        fields = {k: torch.cat([getattr(c, k) for c in ordered], dim=0) for k in _ROW_FIELDS}
        peaks = [c.peak_memory_mb for c in ordered if c.peak_memory_mb is not None]
        steps = int(fields["token_ids"].shape[1])
        return _pack_output(request, sample_specs, fields, ordered[0].context, steps, len(ordered),
                            max(peaks) if peaks else None)


class JanusProPipelineExecutor(ARPipelineExecutorBase):
    family = "janus_pro"
    task = "ar_t2i"
    default_image_token_num = 576
    default_image_size = 384
    default_max_text_length = 256

    def __init__(self, model: Any) -> None:
        self.model = model
        self._gatherer = JanusProChunkGatherer()

    def workload_signature(self, request: GenerationRequest) -> WorkloadSignature:
        return WorkloadSignature.from_request(request)

    # -- prompt handling ----------------------------------------------------------------
    @staticmethod
    def _format_t2i_prompt(prompt: str) -> str:
        return f"<｜User｜>: {prompt}\n\n<｜Assistant｜>:<begin_of_image>"

    def _encode_texts(self, texts: list[str], max_length: int):
        """Token ids and mask from the policy's own tokenizer, or — for a policy that carries a
        chat processor with a Hugging Face tokenizer instead (the reference's policy contract) —
        from that."""
        device = self.model.device
        tok = getattr(self.model, "tokenizer", None)
        if tok is not None and hasattr(tok, "batch_encode"):
            return (*tok.batch_encode(list(texts), max_length, device), getattr(tok, "pad_id", 0))
        processor = self.model.processor
        hf = getattr(processor, "tokenizer", processor)
        enc = hf(list(texts), return_tensors="pt", padding="max_length", truncation=True, max_length=max_length)
        return enc["input_ids"].to(device), enc["attention_mask"].to(device), int(getattr(hf, "pad_token_id", 0) or 0)

    def _tokenize_prompts(self, prompts: list[str], max_length: int):
        cond_ids, cond_mask, pad = self._encode_texts([self._format_t2i_prompt(p) for p in prompts], max_length)
        unc_ids, unc_mask, _ = self._encode_texts([self._format_t2i_prompt("")] * len(prompts), max_length)
        return self.align_pair(cond_ids, cond_mask, unc_ids, unc_mask, pad_id=pad)

    def _embed(self, token_ids: torch.Tensor) -> torch.Tensor:
        embed = getattr(self.model, "embed_text", None)
        if callable(embed):
            return embed(token_ids)
        return self.model.language_model.get_input_embeddings()(token_ids)

    def _takes_generator(self) -> bool:
        import inspect

        try:
            params = inspect.signature(self.model.sample_image_tokens).parameters
        except (TypeError, ValueError):
            return True
        return "generator" in params or any(p.kind == p.VAR_KEYWORD for p in params.values())

    # -- sampling -----------------------------------------------------------------------
    def _sample_with_ar_scheduler(self, *, request: GenerationRequest, sample_ids: list[str],
                                  cond_embeds, uncond_embeds, prompt_mask, uncond_mask,
                                  sample_kwargs: dict[str, Any], batch_size: int):
        state = self.model.init_ar_state(cond_embeds, uncond_embeds, prompt_mask, uncond_mask,
                                         **sample_kwargs)
        scheduler = ARTokenScheduler(max_batch_size=max(1, int(batch_size)))
        scheduler.add_many([
            ActiveSequence(request_id=request.request_id, sample_id=sid, family=self.family,
                           task=self.task, tokenizer_key="janus", dtype=str(getattr(self.model, "dtype", "float32")),
                           max_new_tokens=int(sample_kwargs["image_token_num"]), metadata={"row_index": row})
            for row, sid in enumerate(sample_ids)
        ])
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
                  seed_offset: int) -> tuple[dict[str, torch.Tensor], dict[str, Any], int]:
        spec = self.parse_spec(request)
        s = request.sampling
        # request values win; a policy without a config object gets the published defaults
        config = getattr(self.model, "config", None)
        cfg_weight = float(s.get("cfg_weight", getattr(config, "cfg_weight", 5.0)))
        temperature = float(s.get("temperature", getattr(config, "temperature", 1.0)))
        generator = None
        if spec.seed is not None:
            generator = torch.Generator(device="cpu").manual_seed(int(spec.seed) + seed_offset)
        cond_ids, cond_mask, unc_ids, unc_mask = self._tokenize_prompts(prompts, spec.max_text_length)
        kwargs = dict(cfg_weight=cfg_weight, temperature=temperature, image_token_num=spec.image_token_num)
        if generator is not None and self._takes_generator():
            kwargs["generator"] = generator
        elif generator is not None:
            # a policy that draws from the default generator (the reference's contract): seed that
            torch.manual_seed(int(spec.seed) + seed_offset)
        if spec.use_ar_scheduler:
            tokens, log_probs = self._sample_with_ar_scheduler(
                request=request, sample_ids=sample_ids, cond_embeds=self._embed(cond_ids),
                uncond_embeds=self._embed(unc_ids), prompt_mask=cond_mask, uncond_mask=unc_mask,
                sample_kwargs=kwargs,
                batch_size=int(s.get("ar_scheduler_batch_size", len(prompts))))
        else:
            tokens, log_probs = self.model.sample_image_tokens(
                self._embed(cond_ids), self._embed(unc_ids), cond_mask, unc_mask, **kwargs)
        images = self.model.decode_image_tokens(tokens, image_size=spec.image_size)
        fields = {"output": images, "token_ids": tokens, "token_log_probs": log_probs,
                  "token_mask": torch.ones_like(log_probs), "prompt_input_ids": cond_ids,
                  "prompt_attention_mask": cond_mask, "uncond_input_ids": unc_ids,
                  "uncond_attention_mask": unc_mask}
        context = {"cfg_weight": cfg_weight, "temperature": temperature,
                   "image_token_num": spec.image_token_num,
                   "model_family": getattr(self.model, "model_family", "janus_pro")}
        return fields, context, spec.image_token_num

    # -- executor protocol ----------------------------------------------------------------
    def forward(self, request: GenerationRequest,
                sample_specs: list[GenerationSampleSpec]) -> OutputBatch:
        prompts = self.expand_prompts(request)
        fields, context, steps = self._run_rows(request, prompts,
                                                [s.sample_id for s in sample_specs], 0)
        return _pack_output(request, sample_specs, fields, context, steps, 1, self.peak_memory_mb())

    def forward_chunk(self, request: GenerationRequest, chunk: MicroBatchPlan) -> JanusProARChunkResult:
        self.validate_chunk(request, chunk)
        ids = [f"{request.request_id}:prompt:{chunk.prompt_index}:sample:{j}"
               for j in range(chunk.sample_start, chunk.sample_end)]
        fields, context, _ = self._run_rows(request, [chunk.prompt] * chunk.sample_count, ids,
                                            self.chunk_seed_offset(request, chunk))
        return JanusProARChunkResult(prompt_index=chunk.prompt_index,
                                     sample_start=chunk.sample_start,
                                     sample_count=chunk.sample_count, context=context,
                                     peak_memory_mb=self.peak_memory_mb(), **fields)

    def gather_chunks(self, request, sample_specs, chunks) -> OutputBatch:
        return self._gatherer.gather_chunks(request, sample_specs, chunks)


__all__ = ["JanusProARChunkResult", "JanusProChunkGatherer", "JanusProPipelineExecutor"]
