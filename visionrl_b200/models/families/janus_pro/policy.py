"""Janus-Pro-style autoregressive image-token policy.

A LLaMA trunk predicts 16 384-way image-codebook tokens through a dedicated generation head
(``gen_head`` — never the text ``lm_head``); sampled tokens are fed back through
``gen_aligner(gen_embed(token))``.  Rollout uses classifier-free guidance on logits,
``guided = uncond + w (cond - uncond)``, samples from ``softmax(guided / T)`` and records
``log_softmax(cond / T)[token]`` — the log-probability under the *conditional* distribution,
which is what the teacher-forced replay recomputes (reference:
``vrl/models/families/janus_pro/policy.py:168-842``).

B200-oriented differences from the reference implementation: conditional and unconditional
rows share one static KV cache (rows ``[0, b)`` and ``[b, 2b)``) instead of per-row nested
tuples that are concatenated and split every step; the uniform variates that drive sampling
are drawn once per sequence, so black-box sampling and token-scheduled sampling give the same
tokens regardless of how rows are batched; the replay can return per-token log-probs directly
from the fused head kernel instead of ``[B, L, V]`` logits.
"""

from __future__ import annotations

import contextlib
from dataclasses import dataclass, field
from typing import Any, Iterator

import torch
from torch import nn

from visionrl_b200.models.ar import ARStepResult, AutoregressivePolicy
from visionrl_b200.models.families.flow_policy import resolve_dtype, seeded_construction, seeded_init
from visionrl_b200.models.nn.layers import Linear, adapters_disabled, apply_lora, iter_lora_layers
from visionrl_b200.models.nn.llama import KVCache, LlamaConfig, LlamaDecoder
from visionrl_b200.models.nn.vision import HashTokenizer, VQDecoder
from visionrl_b200.ops import logprob as logprob_ops
from visionrl_b200.ops import sampling as sampling_ops


# the published model's image-token geometry (defaults of the config below)
JANUS_IMAGE_TOKEN_NUM = 576
JANUS_IMAGE_VOCAB_SIZE = 16384
JANUS_IMAGE_PATCH_SIZE = 16
JANUS_IMAGE_PIXEL_SIZE = 384


@dataclass
class JanusProConfig:
    model_path: str = "deepseek-community/Janus-Pro-1B"
    dtype: str = "bfloat16"
    use_lora: bool = True
    lora_rank: int = 128
    lora_alpha: int = 256
    lora_dropout: float = 0.0
    lora_init: str = "gaussian"
    lora_target_modules: tuple = ("q_proj", "k_proj", "v_proj", "o_proj")
    cfg_weight: float = 5.0
    temperature: float = 1.0
    image_token_num: int = 576
    image_size: int = 384
    patch_size: int = 16
    freeze_vq: bool = True
    random_init: bool = True
    init_seed: int = 0
    int4_decode: bool = False
    arch: dict = field(default_factory=dict)
    # fields of the reference's config, accepted so that code and YAML written for it construct
    # this one: the native model has no remote code and no understanding-side vision encoder
    trust_remote_code: bool = True
    device: str | None = None
    freeze_vision_encoder: bool = True
    freeze_aligner: bool = True                 # False: the generation aligner trains with the trunk
    vq_latent_channels: int | None = None       # overrides arch["codebook_dim"] when set


@dataclass
class JanusProARState:
    """Per-request sampling state shared by black-box and scheduled sampling."""

    cache: KVCache
    token_ids: torch.Tensor          # [B, L_img] long
    log_probs: torch.Tensor          # [B, L_img] fp32
    uniforms: torch.Tensor           # [B, L_img] fp32, drives the inverse-CDF sampler
    last_hidden: torch.Tensor        # [2B, D] hidden state that predicts the next token
    positions: torch.Tensor          # [B] next image position per row
    text_len: int
    cfg_weight: float
    temperature: float
    image_token_num: int


class JanusNetwork(nn.Module):
    """Trainable trunk plus the frozen generation-side modules."""

    def __init__(self, arch: dict[str, Any]):
        super().__init__()
        cfg = LlamaConfig.from_dict(arch)
        d = cfg.hidden_size
        codebook = int(arch.get("image_vocab_size", 16384))
        code_dim = int(arch.get("codebook_dim", 8))
        self.language_model = LlamaDecoder(cfg)
        self.gen_embed = nn.Embedding(codebook, code_dim)
        self.gen_aligner = nn.Sequential()
        self.gen_aligner.fc1 = Linear(code_dim, d)
        self.gen_aligner.fc2 = Linear(d, d)
        self.gen_head = nn.Sequential()
        self.gen_head.fc1 = Linear(d, d)
        self.gen_head.fc2 = Linear(d, codebook)

    def align(self, token_ids: torch.Tensor) -> torch.Tensor:
        e = self.gen_embed(token_ids).to(self.gen_aligner.fc1.weight.dtype)
        return self.gen_aligner.fc2(self.gen_aligner.fc1(e, act="gelu_tanh"))

    def head_hidden(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.gen_head.fc1(hidden, act="gelu_tanh")

    def image_logits(self, hidden: torch.Tensor) -> torch.Tensor:
        return self.gen_head.fc2(self.head_hidden(hidden))

    def image_logits_fp32(self, hidden: torch.Tensor) -> torch.Tensor:
        """Logits kept in the GEMM's fp32 accumulator precision.

        Sampling records ``log_softmax`` of these values; the training replay forms the same
        quantity from fp32 head outputs tile by tile, so both sides must skip the bf16 rounding
        of the logits to agree.
        """
        from visionrl_b200.ops import linear as linear_ops

        hh = self.head_hidden(hidden)
        head = self.gen_head.fc2
        h2 = hh.reshape(-1, hh.shape[-1])
        if linear_ops._use_kernel(h2, head.weight):
            out = linear_ops.gemm_nt(h2.contiguous(), head.weight, head.bias, out_dtype=torch.float32)
            return out.view(*hh.shape[:-1], -1)
        return head(hh).float()


def image_token_logits_from_hidden(network: Any, hidden: torch.Tensor) -> torch.Tensor:
    """Image-vocabulary logits from trunk hidden states (always through ``gen_head``).
    ``network`` is a :class:`JanusNetwork` or an external multi-modality model with ``gen_head``."""
    if hasattr(network, "image_logits"):
        return network.image_logits(hidden)
    return network.gen_head(hidden)


class JanusProPolicy(nn.Module, AutoregressivePolicy):
    family = "janus_pro"
    model_family = "janus_pro"

    def __new__(cls, config: JanusProConfig | None = None, *args: Any, mmgpt: Any | None = None,
                **kwargs: Any):
        # an already loaded external model is served by the wrapper class of ``wrapped.py``
        if mmgpt is not None and cls is JanusProPolicy:
            from visionrl_b200.models.families.janus_pro.wrapped import WrappedJanusProPolicy

            return super().__new__(WrappedJanusProPolicy)
        return super().__new__(cls)

    def __init__(self, config: JanusProConfig | None = None, *, network: JanusNetwork | None = None,
                 vq_model: nn.Module | None = None, device: Any = "cpu", mmgpt: Any | None = None,
                 processor: Any | None = None) -> None:
        super().__init__()
        if mmgpt is not None:
            raise TypeError("an external `mmgpt` is served by WrappedJanusProPolicy")
        if processor is not None:
            self.processor = processor
        self.config = config or JanusProConfig()
        arch = dict(self.config.arch)
        if self.config.vq_latent_channels is not None:
            if int(self.config.vq_latent_channels) <= 0:
                raise ValueError("vq_latent_channels must be positive")
            arch["codebook_dim"] = int(self.config.vq_latent_channels)
        dtype = resolve_dtype(self.config.dtype)
        if self.config.device is not None and str(device) == "cpu":
            device = self.config.device          # the reference names the device in the config
        dev = torch.device(device)
        if network is None:
            with seeded_construction(self.config.init_seed, dev):
                network = JanusNetwork(arch)
                if self.config.random_init:
                    seeded_init(network, self.config.init_seed)
            if not self.config.random_init:
                self._load_checkpoint(network, self.config.model_path)
        self.policy = network.to(device=dev, dtype=dtype)
        if vq_model is None:
            grid = max(1, self.config.image_size // self.config.patch_size)
            del grid
            with seeded_construction(self.config.init_seed + 1, dev):
                vq_model = VQDecoder(int(arch.get("image_vocab_size", 16384)),
                                     int(arch.get("codebook_dim", 8)),
                                     int(arch.get("vq_base", 128)),
                                     tuple(arch.get("vq_mults", (1, 1, 2, 2, 4))),
                                     int(arch.get("vq_blocks", 2)))
                seeded_init(vq_model, self.config.init_seed + 1)
        vq_dtype = dtype if dev.type == "cuda" else torch.float32
        object.__setattr__(self, "_vq", vq_model.to(device=dev, dtype=vq_dtype).eval()
                           .requires_grad_(False))
        self.tokenizer = HashTokenizer(self.policy.language_model.cfg.vocab_size)
        # the codebook fed back into the trunk is the VQ codebook; it and the aligner / head
        # stay frozen, only the trunk (or its adapters) trains
        frozen = [self.policy.gen_embed, self.policy.gen_head]
        if self.config.freeze_aligner:
            frozen.append(self.policy.gen_aligner)
        for module in frozen:
            module.requires_grad_(False)
        self.policy.language_model.embed_tokens.requires_grad_(False)
        if self.config.use_lora:
            self._apply_lora()
        self.fused_logprob = True
        self._int4_layers = -1          # -1: int4 copies not built yet
        self.decode_graph = True        # replay the decode step from a CUDA graph on GPU

    def _int4_context(self):
        """Context under which the trunk's decode-sized linears read int4 weights.

        Active only when ``int4_decode`` is configured, the model sits on a CUDA device and the
        trunk's base weights are frozen (LoRA training); the copies are built on first use.
        """
        from visionrl_b200.models.nn.layers import attach_int4_shadows, int4_decode

        enabled = bool(self.config.int4_decode) and self.device.type == "cuda"
        if enabled and self._int4_layers < 0:
            self._int4_layers = attach_int4_shadows(self.policy.language_model)
        return int4_decode(enabled and self._int4_layers > 0)

    @staticmethod
    def _load_checkpoint(network: nn.Module, path: str) -> None:
        import os

        file = os.path.join(path, "janus.safetensors")
        if not os.path.exists(file):
            raise FileNotFoundError(
                f"{file} not found: set model.random_init=true for seeded random weights or "
                "point model.path at a directory in the native key layout")
        from safetensors.torch import load_file

        network.load_state_dict(load_file(file), strict=True)

    # -- module access -----------------------------------------------------------------
    @property
    def language_model(self) -> LlamaDecoder:
        return self.policy.language_model

    @property
    def vq_model(self) -> nn.Module:
        return self._vq

    @property
    def device(self) -> torch.device:
        return self.policy.gen_head.fc2.weight.device

    @property
    def dtype(self) -> torch.dtype:
        return self.policy.gen_head.fc2.weight.dtype

    @property
    def trainable_modules(self) -> dict[str, Any]:
        return {"policy": self.policy}

    def trainable_parameters(self) -> Iterator[nn.Parameter]:
        return (p for p in self.parameters() if p.requires_grad)

    def trainable_param_count(self) -> int:
        return sum(p.numel() for p in self.trainable_parameters())

    # -- adapters ----------------------------------------------------------------------
    def _apply_lora(self) -> None:
        c = self.config
        apply_lora(self.policy.language_model, c.lora_rank, c.lora_alpha,
                   list(c.lora_target_modules), c.lora_init, freeze_base=True)

    @property
    def has_adapters(self) -> bool:
        return any(True for _ in iter_lora_layers(self.policy.language_model))

    @property
    def has_lora_adapter(self) -> bool:
        return self.has_adapters

    def disable_adapter(self):
        if not self.has_adapters:
            raise RuntimeError("JanusProPolicy.disable_adapter(): the trunk carries no LoRA "
                               "adapter; pass a separate reference model instead")
        return adapters_disabled(self.policy.language_model)

    def load_trainable_state(self, state_dict: dict[str, Any]) -> Any:
        """Accepts ``policy.*`` keys (full or trainable-only)."""
        state = dict(state_dict)
        if not state:
            raise ValueError("load_trainable_state received an empty state dict")
        bad = [k for k in state if not k.startswith("policy.")]
        if bad:
            raise ValueError(f"load_trainable_state only accepts 'policy.'-prefixed keys; got {bad[:4]}")
        result = self.policy.load_state_dict({k[7:]: v for k, v in state.items()}, strict=False)
        if result.unexpected_keys:
            raise ValueError(f"unexpected keys: {result.unexpected_keys[:4]}")
        return result

    # -- teacher-forced replay ------------------------------------------------------------
    def embed_text(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.policy.language_model.embed_tokens(token_ids)

    def _replay_hidden(self, prompt_embeds, prompt_mask, image_token_ids):
        b, l_text = prompt_mask.shape
        l_img = image_token_ids.shape[1]
        img_embeds = self.policy.align(image_token_ids[:, :-1]) if l_img > 1 else \
            prompt_embeds.new_zeros(b, 0, prompt_embeds.shape[-1])
        seq = torch.cat([prompt_embeds.to(img_embeds.dtype), img_embeds], dim=1)
        mask = torch.cat([prompt_mask, prompt_mask.new_ones(b, l_img - 1)], dim=1)
        hidden = self.policy.language_model(seq, mask)
        return hidden[:, l_text - 1: l_text - 1 + l_img]

    def forward_image_logits(self, prompt_inputs_embeds, prompt_attention_mask, image_token_ids):
        """``[B, L_img, V_img]`` logits; position ``L_text-1+i`` predicts image token ``i``."""
        return self.policy.image_logits(
            self._replay_hidden(prompt_inputs_embeds, prompt_attention_mask, image_token_ids))

    def replay_forward(self, batch: Any, timestep_idx: int = 0) -> dict[str, Any]:
        obs = batch.observations
        prompt_ids = obs[:, 0] if obs.ndim == 3 else obs
        prompt_ids = prompt_ids.to(self.device)
        mask = batch.extras["prompt_attention_mask"].to(self.device)
        tokens = batch.actions.to(self.device)
        hidden = self._replay_hidden(self.embed_text(prompt_ids), mask, tokens)
        out: dict[str, Any] = {"image_token_ids": tokens}
        temperature = float((getattr(batch, "context", None) or {}).get("temperature", 1.0) or 1.0)
        if self.fused_logprob and hidden.is_cuda:
            head = self.policy.gen_head.fc2
            out["token_log_probs"] = logprob_ops.fused_head_log_probs(
                self.policy.head_hidden(hidden), head.weight, head.bias, tokens, temperature)
        else:
            out["logits"] = self.policy.gen_head.fc2(self.policy.head_hidden(hidden))
        return out

    # -- sampling --------------------------------------------------------------------------
    @torch.no_grad()
    def init_ar_state(self, cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                      uncond_attention_mask, *, cfg_weight=None, temperature=None,
                      image_token_num=None, generator: torch.Generator | None = None) -> JanusProARState:
        c = self.config
        w = c.cfg_weight if cfg_weight is None else float(cfg_weight)
        t = c.temperature if temperature is None else float(temperature)
        n_img = int(image_token_num or c.image_token_num)
        b, l_text = cond_attention_mask.shape
        lm = self.policy.language_model
        cache = lm.new_cache(2 * b, l_text + n_img, device=self.device, dtype=self.dtype)
        embeds = torch.cat([cond_inputs_embeds, uncond_inputs_embeds], dim=0).to(self.dtype)
        mask = torch.cat([cond_attention_mask, uncond_attention_mask], dim=0)
        hidden = lm(embeds, mask, cache=cache)
        if generator is not None and generator.device.type != self.device.type:
            uniforms = torch.rand(b, n_img, generator=generator).to(self.device)
        else:
            uniforms = torch.rand(b, n_img, generator=generator, device=self.device)
        return JanusProARState(
            cache=cache, token_ids=torch.zeros(b, n_img, dtype=torch.long, device=self.device),
            log_probs=torch.zeros(b, n_img, dtype=torch.float32, device=self.device),
            uniforms=uniforms, last_hidden=hidden[:, -1].contiguous(),
            positions=torch.zeros(b, dtype=torch.long, device=self.device), text_len=l_text,
            cfg_weight=w, temperature=t, image_token_num=n_img)

    def _sample_rows(self, state: JanusProARState, rows: torch.Tensor | None, position: int):
        """Sample the token at ``position`` for ``rows`` (all rows when ``None``) and advance."""
        b = state.token_ids.shape[0]
        if rows is None:
            hidden = state.last_hidden
            u = state.uniforms[:, position]
        else:
            hidden = state.last_hidden[torch.cat([rows, rows + b])]
            u = state.uniforms[rows, position]
        logits = self.policy.image_logits_fp32(hidden)
        n = logits.shape[0] // 2
        tokens, log_probs = sampling_ops.sample_cfg_tokens(
            logits[:n], logits[n:], u, state.cfg_weight, state.temperature)
        if rows is None:
            state.token_ids[:, position] = tokens
            state.log_probs[:, position] = log_probs
        else:
            state.token_ids[rows, position] = tokens
            state.log_probs[rows, position] = log_probs
        if position + 1 < state.image_token_num:
            nxt = self.policy.align(tokens)
            lm = self.policy.language_model
            if rows is None and self.config.int4_decode:
                with self._int4_context():
                    state.last_hidden = lm.decode_step(torch.cat([nxt, nxt], dim=0), state.cache)
            elif rows is None:
                state.last_hidden = lm.decode_step(torch.cat([nxt, nxt], dim=0), state.cache)
            else:
                both = torch.cat([rows, rows + b])
                state.last_hidden[both] = lm.decode_step(
                    torch.cat([nxt, nxt], dim=0), state.cache, rows=both,
                    position=state.text_len + position)
        if rows is None:
            state.positions += 1
        else:
            state.positions[rows] += 1
        return tokens, log_probs

    # -- whole-batch decode with device-side positions (CUDA-graph replay) ------------------
    def _step_all(self, state: JanusProARState, pos_img: torch.Tensor, pos_cache: torch.Tensor) -> None:
        """Sample the token at image position ``pos_img`` for every row, feed it back at cache
        position ``pos_cache`` and advance both counters — all indices live on the device."""
        u = state.uniforms.index_select(1, pos_img)[:, 0]
        logits = self.policy.image_logits_fp32(state.last_hidden)
        n = logits.shape[0] // 2
        tokens, log_probs = sampling_ops.sample_cfg_tokens(
            logits[:n], logits[n:], u, state.cfg_weight, state.temperature)
        state.token_ids.index_copy_(1, pos_img, tokens.unsqueeze(1))
        state.log_probs.index_copy_(1, pos_img, log_probs.unsqueeze(1))
        nxt = self.policy.align(tokens)
        with self._int4_context():
            hidden = self.policy.language_model.decode_step_at(
                torch.cat([nxt, nxt], dim=0), state.cache, pos_cache)
        state.last_hidden.copy_(hidden)
        pos_img.add_(1)
        pos_cache.add_(1)

    def _decode_all_positions(self, state: JanusProARState) -> None:
        """The 576-step (or so) decode loop is launch-bound: each step is a few hundred small
        kernels.  Two steps run eagerly (they also finish every lazy set-up), the third is
        captured in a CUDA graph and the graph is replayed for the remaining positions."""
        n = state.image_token_num
        dev = state.token_ids.device
        pos_img = torch.zeros(1, dtype=torch.long, device=dev)
        pos_cache = torch.full((1,), state.text_len, dtype=torch.long, device=dev)
        eager = min(n, 2)
        for _ in range(eager):
            self._step_all(state, pos_img, pos_cache)
        if n > eager:
            if self.decode_graph:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    self._step_all(state, pos_img, pos_cache)
                for _ in range(n - eager):
                    graph.replay()
                torch.cuda.current_stream().synchronize()
                del graph
            else:
                for _ in range(n - eager):
                    self._step_all(state, pos_img, pos_cache)
        state.cache.length = state.text_len + n
        state.positions += n

    @torch.no_grad()
    def sample_image_tokens(self, cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                            uncond_attention_mask, *, cfg_weight=None, temperature=None,
                            image_token_num=None, generator: torch.Generator | None = None):
        from visionrl_b200.ops import _ext

        state = self.init_ar_state(cond_inputs_embeds, uncond_inputs_embeds, cond_attention_mask,
                                   uncond_attention_mask, cfg_weight=cfg_weight,
                                   temperature=temperature, image_token_num=image_token_num,
                                   generator=generator)
        if self.device.type == "cuda" and _ext.kernels_enabled() and _ext.has("decode_attention") \
                and self.dtype == torch.bfloat16:
            self._decode_all_positions(state)
        else:
            for position in range(state.image_token_num):
                self._sample_rows(state, None, position)
        return self.finalize_ar_state(state)

    @torch.no_grad()
    def step_ar(self, state: JanusProARState, sequences: list[Any], *,
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
        idx = torch.tensor(rows, dtype=torch.long, device=self.device)
        tokens, log_probs = self._sample_rows(state, idx, position)
        return ARStepResult(sequence_ids=[seq.sample_id for seq in sequences],
                            positions=[position] * len(sequences), token=tokens, log_prob=log_probs)

    def finalize_ar_state(self, state: JanusProARState):
        return state.token_ids, state.log_probs

    # -- decoding ----------------------------------------------------------------------------
    def _resolve_vq_latent_channels(self) -> int:
        """Codebook width read from the live embedding table (not from a config field)."""
        return int(self._vq.quantize.embedding.weight.shape[-1])

    @torch.no_grad()
    def decode_image_tokens(self, image_token_ids: torch.Tensor, image_size: int | None = None):
        token_ids = image_token_ids
        b, n = token_ids.shape
        side = int(round(n ** 0.5))
        if side * side != n:
            raise ValueError(f"image token count {n} is not a square grid")
        shape = (b, self._resolve_vq_latent_channels(), side, side)
        images = self._vq.decode_code(token_ids.to(torch.long), shape).float().clamp(-1.0, 1.0)
        if image_size is not None and images.shape[-1] != image_size:
            images = torch.nn.functional.interpolate(images, size=(image_size, image_size),
                                                     mode="bilinear", align_corners=False)
        return images


__all__ = ["JanusNetwork", "JanusProARState", "JanusProConfig", "JanusProPolicy",
           "image_token_logits_from_hidden"]
