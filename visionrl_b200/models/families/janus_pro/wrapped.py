"""Janus-Pro policy around an externally loaded multi-modality model.

``JanusProPolicy(config, mmgpt=model, processor=processor)`` is the reference's way to hand the
policy an already loaded Hugging Face ``MultiModalityCausalLM`` and its chat processor
(reference: ``vrl/models/families/janus_pro/policy.py:177-224``).  The native policy of this
package owns its trunk; this class serves code that owns one already.  It expects of ``mmgpt``

* ``language_model`` whose trunk (``.model`` when there is one) maps ``inputs_embeds`` /
  ``attention_mask`` / ``past_key_values`` to an object with ``last_hidden_state`` and
  ``past_key_values``, and which has ``get_input_embeddings()``;
* ``gen_head`` (hidden → image-codebook logits), ``prepare_gen_img_embeds(ids)`` (token ids →
  trunk inputs) and ``gen_vision_model.decode_code(ids, shape)``.

What differs from the reference's wrapper: adapters are this package's own (``nn.Linear`` targets
are re-hosted as :class:`LoRALinear` over the same parameters, so no PEFT install is needed and
the reference forward is the same module with adapters switched off); sampling draws one uniform
per token up front and inverts the CDF, so black-box and token-scheduled sampling return the same
tokens; rows that step together share one batched cache and are only split per row when the
scheduler asks for a subset.
"""

from __future__ import annotations

from collections.abc import Mapping
from dataclasses import dataclass
from typing import Any, Iterator

import torch
from torch import nn

from visionrl_b200.models.ar import ARStepResult, ar_concat_rows, ar_split_rows
from visionrl_b200.models.families.janus_pro.policy import JanusProConfig, JanusProPolicy
from visionrl_b200.models.nn.layers import LoRALinear, adapters_disabled, apply_lora, iter_lora_layers
from visionrl_b200.ops import sampling as sampling_ops

_REQUIRED = ("gen_head", "gen_vision_model", "language_model")


def host_linear_layers(module: nn.Module, target_modules) -> list[str]:
    """Replace every ``nn.Linear`` under ``module`` whose name ends with a target by a
    :class:`LoRALinear` over the SAME weight and bias parameters; returns the names replaced."""
    targets = tuple(target_modules)
    swapped: list[str] = []
    for parent_name, parent in list(module.named_modules()):
        for child_name, child in list(parent.named_children()):
            if type(child) is not nn.Linear or child_name not in targets:
                continue
            hosted = LoRALinear(child.in_features, child.out_features, bias=child.bias is not None)
            hosted.weight = child.weight
            hosted.bias = child.bias
            setattr(parent, child_name, hosted)
            swapped.append(f"{parent_name}.{child_name}" if parent_name else child_name)
    return swapped


@dataclass
class WrappedJanusARState:
    """Sampling state over an external trunk.  Rows ``[0, b)`` are conditional, ``[b, 2b)``
    unconditional; ``past`` is one batched cache while all rows step together and a per-row list
    (``past_rows``) once a subset stepped."""

    inputs: list[torch.Tensor]            # 2b entries [1, L, H]: what each row feeds next
    masks: list[torch.Tensor]             # 2b entries [1, L_total]
    past: Any
    past_rows: list[Any] | None
    token_ids: torch.Tensor               # [b, L_img] long
    log_probs: torch.Tensor               # [b, L_img] fp32
    uniforms: torch.Tensor                # [b, L_img] fp32
    positions: torch.Tensor               # [b] long
    cfg_weight: float
    temperature: float
    image_token_num: int
    cache_type: type | None = None        # class of the trunk's cache object, when it is one

    @property
    def logprobs(self) -> torch.Tensor:   # the reference's field name
        return self.log_probs


def _layer_pairs(cache: Any) -> tuple | None:
    """``((keys, values), ...)`` of a cache object that keeps one entry per layer under ``layers``
    (the ``DynamicCache`` of current ``transformers``); ``None`` for anything else."""
    layers = getattr(cache, "layers", None)
    if not layers:
        return None
    pairs = []
    for layer in layers:
        keys, values = getattr(layer, "keys", None), getattr(layer, "values", None)
        if not isinstance(keys, torch.Tensor) or not isinstance(values, torch.Tensor):
            return None
        pairs.append((keys, values))
    return tuple(pairs)


def _split_cache(cache: Any, rows: int) -> list[Any]:
    legacy = getattr(cache, "to_legacy_cache", None)
    value = legacy() if callable(legacy) else cache
    if not isinstance(value, (torch.Tensor, tuple, list, Mapping)):
        value = _layer_pairs(value) or value
    if not isinstance(value, (torch.Tensor, tuple, list, Mapping)):
        raise TypeError(
            f"cannot split a {type(cache).__name__} cache per row: step all rows of a request "
            "together, or use a trunk that returns nested tuples of tensors")
    return ar_split_rows(value, rows)


class WrappedJanusProPolicy(JanusProPolicy):
    """See the module docstring.  Constructed through ``JanusProPolicy(..., mmgpt=...)``."""

    def __init__(self, config: JanusProConfig | None = None, *, mmgpt: Any = None,
                 processor: Any | None = None, **unused: Any) -> None:
        nn.Module.__init__(self)
        del unused
        if mmgpt is None:
            raise ValueError("WrappedJanusProPolicy needs `mmgpt`")
        if processor is None:
            raise ValueError("Must pass `processor` when `mmgpt` is provided")
        self.config = config or JanusProConfig()
        for attr in _REQUIRED:
            if not hasattr(mmgpt, attr):
                raise RuntimeError(f"the model passed as `mmgpt` has no `{attr}`: it does not look "
                                   "like a Janus MultiModalityCausalLM")
        self._processor = processor
        for p in mmgpt.parameters():
            p.requires_grad_(False)
        self.mmgpt = mmgpt
        if self.config.use_lora:
            c = self.config
            hosted = host_linear_layers(mmgpt.language_model, c.lora_target_modules)
            if not hosted:
                raise ValueError(f"no nn.Linear under language_model matches {list(c.lora_target_modules)}")
            apply_lora(mmgpt.language_model, c.lora_rank, c.lora_alpha, list(c.lora_target_modules),
                       c.lora_init, freeze_base=True)
        if not self.config.freeze_aligner and hasattr(mmgpt, "gen_aligner"):
            mmgpt.gen_aligner.requires_grad_(True)
        self.fused_logprob = False
        self.decode_graph = False
        self._int4_layers = 0

    # -- module access -------------------------------------------------------------------
    @property
    def policy(self) -> nn.Module:
        return self.mmgpt

    @property
    def processor(self) -> Any:
        return self._processor

    @property
    def language_model(self) -> nn.Module:
        return self.mmgpt.language_model

    def _trunk(self) -> nn.Module:
        """The module that returns hidden states (a causal-LM wrapper's ``.model``), never the
        text-vocabulary head."""
        lm = self.mmgpt.language_model
        return lm.model if hasattr(lm, "model") else lm

    @property
    def vq_model(self) -> nn.Module:
        return self.mmgpt.gen_vision_model

    def _first_parameter(self) -> torch.Tensor:
        return next(self.mmgpt.parameters())

    @property
    def device(self) -> torch.device:
        return self._first_parameter().device

    @property
    def dtype(self) -> torch.dtype:
        return self._first_parameter().dtype

    @property
    def trainable_modules(self) -> dict[str, Any]:
        return {"policy": self.mmgpt}

    def trainable_parameters(self) -> Iterator[nn.Parameter]:
        return (p for p in self.mmgpt.parameters() if p.requires_grad)

    # -- adapters ------------------------------------------------------------------------
    @property
    def has_adapters(self) -> bool:
        return any(True for _ in iter_lora_layers(self.mmgpt.language_model))

    def disable_adapter(self):
        if not self.has_adapters:
            raise RuntimeError(
                "JanusProPolicy.disable_adapter(): no PEFT adapter or LoRA layer is attached "
                "(use_lora=False); a no-op here would make the reference forward equal the policy "
                "forward and the KL term zero.  Build with use_lora=True or pass a separate "
                "frozen reference model")
        return adapters_disabled(self.mmgpt.language_model)

    def _int4_context(self):
        import contextlib

        return contextlib.nullcontext()

    # -- teacher-forced replay -----------------------------------------------------------
    def embed_text(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.mmgpt.language_model.get_input_embeddings()(token_ids)

    def _image_embeds(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.mmgpt.prepare_gen_img_embeds(token_ids)

    def _head(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.mmgpt.gen_head(hidden)

    def forward_image_logits(self, prompt_inputs_embeds, prompt_attention_mask, image_token_ids):
        """``[B, L_img, V_img]``: position ``L_text - 1 + i`` of the teacher-forced sequence
        ``[text | image[:-1]]`` predicts image token ``i``."""
        b, l_img = image_token_ids.shape
        l_text = prompt_inputs_embeds.shape[1]
        image_embeds = self._image_embeds(image_token_ids)[:, : l_img - 1]
        seq = torch.cat([prompt_inputs_embeds.to(image_embeds.dtype), image_embeds], dim=1)
        mask = torch.cat([prompt_attention_mask,
                          prompt_attention_mask.new_ones(b, l_img - 1)], dim=1)
        hidden = self._trunk()(inputs_embeds=seq, attention_mask=mask, use_cache=False,
                               output_hidden_states=False).last_hidden_state
        return self._head(hidden[:, l_text - 1: l_text - 1 + l_img])

    def replay_forward(self, batch: Any, timestep_idx: int = 0) -> dict[str, Any]:
        del timestep_idx
        obs = batch.observations
        prompt_ids = obs[:, 0] if obs.ndim == 3 else obs
        dev = self.device
        tokens = batch.actions.to(dev)
        logits = self.forward_image_logits(
            self.embed_text(prompt_ids.to(dev)), batch.extras["prompt_attention_mask"].to(dev), tokens)
        return {"logits": logits, "image_token_ids": tokens}

    # -- sampling ------------------------------------------------------------------------
    @torch.no_grad()
    def init_ar_state(self, cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                      uncond_attention_mask, *, cfg_weight=None, temperature=None,
                      image_token_num=None, generator: torch.Generator | None = None):
        c = self.config
        n_img = int(image_token_num or c.image_token_num)
        b = cond_attention_mask.shape[0]
        dev = cond_inputs_embeds.device
        if generator is not None and generator.device.type != dev.type:
            uniforms = torch.rand(b, n_img, generator=generator).to(dev)
        else:
            uniforms = torch.rand(b, n_img, generator=generator, device=dev)
        embeds = torch.cat([cond_inputs_embeds, uncond_inputs_embeds], dim=0)
        masks = torch.cat([cond_attention_mask, uncond_attention_mask], dim=0)
        return WrappedJanusARState(
            inputs=[embeds[i:i + 1] for i in range(2 * b)], masks=[masks[i:i + 1] for i in range(2 * b)],
            past=None, past_rows=None,
            token_ids=torch.zeros(b, n_img, dtype=torch.long, device=dev),
            log_probs=torch.zeros(b, n_img, dtype=torch.float32, device=dev), uniforms=uniforms,
            positions=torch.zeros(b, dtype=torch.long, device=dev),
            cfg_weight=c.cfg_weight if cfg_weight is None else float(cfg_weight),
            temperature=c.temperature if temperature is None else float(temperature),
            image_token_num=n_img)

    def _past_for(self, state: WrappedJanusARState, both: list[int], everyone: bool) -> Any:
        if state.past_rows is None:
            if state.past is None or everyone:
                return state.past
            state.past_rows = _split_cache(state.past, len(state.inputs))
            state.past = None
        rows = [state.past_rows[i] for i in both]
        if all(r is None for r in rows):
            return None
        if any(r is None for r in rows):
            raise ValueError("the cache rows of this request are only partly initialised")
        joined = ar_concat_rows(rows)
        # a trunk that handed out a layered cache object gets one back
        return joined if state.cache_type is None else state.cache_type(ddp_cache_data=joined)

    def _keep_past(self, state: WrappedJanusARState, both: list[int], everyone: bool, past: Any) -> None:
        if past is not None and state.cache_type is None and _layer_pairs(past) is not None:
            state.cache_type = type(past)
        if state.past_rows is None and everyone:
            state.past = past
            return
        if state.past_rows is None:
            state.past_rows = [None] * len(state.inputs)
        parts = [None] * len(both) if past is None else _split_cache(past, len(both))
        for slot, part in zip(both, parts):
            state.past_rows[slot] = part

    def _sample_rows(self, state: WrappedJanusARState, rows: torch.Tensor | None, position: int):
        b = state.token_ids.shape[0]
        row_list = list(range(b)) if rows is None else [int(r) for r in rows.tolist()]
        if not row_list:
            raise ValueError("row_indices must be non-empty")
        if position >= state.image_token_num:
            raise ValueError("the sampling state has already produced every image token")
        at = {int(p) for p in state.positions[row_list].tolist()}
        if at != {int(position)}:
            raise ValueError(f"rows {row_list} stand at positions {sorted(at)}, not at {position}")
        everyone = len(row_list) == b
        both = row_list + [b + r for r in row_list]
        out = self._trunk()(inputs_embeds=torch.cat([state.inputs[i] for i in both], dim=0),
                            attention_mask=torch.cat([state.masks[i] for i in both], dim=0),
                            use_cache=True, past_key_values=self._past_for(state, both, everyone))
        self._keep_past(state, both, everyone, getattr(out, "past_key_values", None))
        logits = self._head(out.last_hidden_state[:, -1]).float()
        n = len(row_list)
        idx = torch.tensor(row_list, dtype=torch.long, device=state.token_ids.device)
        tokens, log_probs = sampling_ops.sample_cfg_tokens(
            logits[:n], logits[n:], state.uniforms[idx, position], state.cfg_weight, state.temperature)
        state.token_ids[idx, position] = tokens
        state.log_probs[idx, position] = log_probs
        nxt = self._image_embeds(tokens.unsqueeze(-1))
        nxt = nxt.reshape(n, 1, nxt.shape[-1])
        for k, slot in enumerate(both):
            state.inputs[slot] = nxt[k % n: k % n + 1]
            state.masks[slot] = torch.cat([state.masks[slot], state.masks[slot].new_ones(1, 1)], dim=1)
        state.positions[idx] += 1
        return tokens, log_probs

    @torch.no_grad()
    def sample_image_tokens(self, cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                            uncond_attention_mask, *, cfg_weight=None, temperature=None,
                            image_token_num=None, generator: torch.Generator | None = None):
        state = self.init_ar_state(cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                                   uncond_attention_mask, cfg_weight=cfg_weight, temperature=temperature,
                                   image_token_num=image_token_num, generator=generator)
        for position in range(state.image_token_num):
            self._sample_rows(state, None, position)
        return self.finalize_ar_state(state)

    @torch.no_grad()
    def step_ar(self, state: WrappedJanusARState, sequences: list[Any], *,
                generator: torch.Generator | None = None) -> ARStepResult:
        del generator
        if not sequences:
            raise ValueError("step_ar requires at least one ActiveSequence")
        rows = [int(seq.metadata.get("row_index", -1)) for seq in sequences]
        if any(r < 0 or r >= state.token_ids.shape[0] for r in rows):
            raise ValueError(f"invalid Janus row indices: {rows}")
        positions = {int(seq.position) for seq in sequences}
        if len(positions) != 1:
            raise ValueError("step_ar requires sequences at one common position")
        position = positions.pop()
        idx = torch.tensor(rows, dtype=torch.long, device=state.token_ids.device)
        tokens, log_probs = self._sample_rows(state, idx, position)
        return ARStepResult(sequence_ids=[seq.sample_id for seq in sequences],
                            positions=[position] * len(sequences), token=tokens, log_prob=log_probs)

    # -- decoding ------------------------------------------------------------------------
    def _resolve_vq_latent_channels(self) -> int:
        """Width of a codebook entry: the configured override, else the live embedding table of
        the quantiser.  Config fields of the VQ model (``z_channels``, ``embed_dim``) are not
        consulted — on the published 1B model ``z_channels`` is the encoder width, not this."""
        override = self.config.vq_latent_channels
        if override is not None:
            if not isinstance(override, int) or isinstance(override, bool) or override <= 0:
                raise RuntimeError(f"vq_latent_channels must be a positive int; got {override!r}")
            return override
        weight = getattr(getattr(getattr(self.vq_model, "quantize", None), "embedding", None), "weight", None)
        if isinstance(weight, torch.Tensor) and weight.ndim == 2 and weight.shape[-1] > 0:
            return int(weight.shape[-1])
        raise RuntimeError("cannot tell the VQ codebook width: set JanusProConfig.vq_latent_channels "
                           "or pass a VQ model that has quantize.embedding.weight")

    @torch.no_grad()
    def decode_image_tokens(self, image_token_ids: torch.Tensor, image_size: int | None = None):
        b, n = image_token_ids.shape
        side = int(round(n ** 0.5))
        if side * side != n:
            raise ValueError(f"image token count {n} is not a square grid")
        shape = [b, self._resolve_vq_latent_channels(), side, side]
        images = self.vq_model.decode_code(image_token_ids.to(torch.int32), shape=shape)
        images = images.float().clamp(-1.0, 1.0)
        if image_size is not None and images.shape[-1] != image_size and images.shape[-1] > 0:
            images = torch.nn.functional.interpolate(images, size=(image_size, image_size),
                                                     mode="bilinear", align_corners=False)
        return images


__all__ = ["WrappedJanusARState", "WrappedJanusProPolicy", "host_linear_layers"]
