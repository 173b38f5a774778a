"""Checkpoints in the Hugging Face LLaMA layout → the native key layout.

The native decoder (``visionrl_b200/models/nn/llama.py``) differs from the Hugging Face one in
three ways a converter has to undo:

* q, k and v are one fused projection whose output is ``[q | k | v]``, and gate and up are one
  fused projection ``[gate | up]``;
* rotary embedding rotates ADJACENT pairs ``(2i, 2i+1)`` of a head, the Hugging Face code
  rotates the pair ``(i, i + Dh/2)``; the rows of the q and k projections are therefore
  permuted per head so that HF row ``i`` becomes native row ``2i`` and HF row ``i + Dh/2`` becomes
  native row ``2i + 1`` (q·k products are unchanged because both get the same permutation);
* names: ``input_layernorm`` → ``attn_norm``, ``post_attention_layernorm`` → ``mlp_norm``,
  ``self_attn.o_proj`` → ``attn.out``, ``mlp.down_proj`` → ``down``.

``llama_from_hf`` is checked against the ``transformers`` implementation in the tests (same
hidden states from the same weights).  ``janus_from_hf`` wraps it with the generation-side
modules of a Janus-Pro checkpoint under the key names of the public Janus code
(``gen_embed``, ``gen_aligner.layers.{0,2}``, ``gen_head.output_mlp_projector``,
``gen_head.vision_head``); no such checkpoint can be fetched here, so that part is exercised on
the key mapping only.

``clip_vision_from_hf`` does the same for the image tower of a CLIP checkpoint (the reward
towers), checked against ``transformers.CLIPVisionModelWithProjection`` in the tests.

    python -m visionrl_b200.models.convert janus <hf_dir> <out_dir> --num-heads 16
    python -m visionrl_b200.models.convert clip_vision <hf_dir> <out_dir>
"""

from __future__ import annotations

import argparse
import os
from typing import Mapping

import torch

_TRUNK_PREFIXES = ("language_model.model.", "model.", "")


def _interleave_rotary_rows(weight: torch.Tensor, num_heads: int) -> torch.Tensor:
    """Rows of a ``[H*Dh, K]`` q or k projection from half-split to adjacent-pair rotary order."""
    out_features, k = weight.shape
    dh = out_features // num_heads
    if dh * num_heads != out_features or dh % 2:
        raise ValueError(f"projection with {out_features} rows does not split into {num_heads} even heads")
    w = weight.view(num_heads, 2, dh // 2, k)              # [head, half, i, K]
    return w.transpose(1, 2).reshape(out_features, k).contiguous()   # [head, i, half, K]


def _strip_trunk_prefix(state: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    for prefix in _TRUNK_PREFIXES:
        probe = prefix + "layers.0.self_attn.q_proj.weight"
        if probe in state:
            return {k[len(prefix):]: v for k, v in state.items() if k.startswith(prefix)}
    raise KeyError("no LLaMA trunk found (looked for layers.0.self_attn.q_proj.weight under "
                   "'language_model.model.', 'model.' and no prefix)")


def llama_from_hf(state: Mapping[str, torch.Tensor], num_heads: int) -> dict[str, torch.Tensor]:
    """State dict of ``LlamaDecoder`` from a Hugging Face ``LlamaModel`` / ``LlamaForCausalLM`` /
    ``Qwen2Model`` state dict: multi-head or grouped-query attention (build the decoder with
    ``num_kv_heads``), with or without the q/k/v bias (``qkv_bias``)."""
    hf = _strip_trunk_prefix(state)
    out: dict[str, torch.Tensor] = {"embed_tokens.weight": hf["embed_tokens.weight"], "norm.weight": hf["norm.weight"]}
    layer = 0
    while f"layers.{layer}.self_attn.q_proj.weight" in hf:
        p = f"layers.{layer}."
        q, k, v = (hf[p + f"self_attn.{n}_proj.weight"] for n in "qkv")
        head_dim = q.shape[0] // num_heads
        kv_heads = k.shape[0] // head_dim          # fewer than num_heads: grouped-query attention
        if k.shape != v.shape or kv_heads * head_dim != k.shape[0] or num_heads % max(kv_heads, 1):
            raise ValueError(f"layer {layer}: key/value projections of {tuple(k.shape)} / {tuple(v.shape)} rows "
                             f"do not form whole heads of {head_dim}")
        for bias in ("self_attn.o_proj.bias", "mlp.gate_proj.bias", "mlp.down_proj.bias"):
            if p + bias in hf:
                raise ValueError(f"layer {layer}: a bias on {bias.rsplit('.', 1)[0]} has no native counterpart")
        out[p + "attn.qkv.weight"] = torch.cat([_interleave_rotary_rows(q, num_heads),
                                                _interleave_rotary_rows(k, kv_heads), v], dim=0)
        if p + "self_attn.q_proj.bias" in hf:      # Qwen2-style trunks: bias on q, k and v only
            qb, kb, vb = (hf[p + f"self_attn.{n}_proj.bias"] for n in "qkv")
            out[p + "attn.qkv.bias"] = torch.cat([_interleave_rotary_rows(qb.unsqueeze(1), num_heads).squeeze(1),
                                                  _interleave_rotary_rows(kb.unsqueeze(1), kv_heads).squeeze(1), vb])
        out[p + "attn.out.weight"] = hf[p + "self_attn.o_proj.weight"]
        out[p + "gate_up.weight"] = torch.cat([hf[p + "mlp.gate_proj.weight"], hf[p + "mlp.up_proj.weight"]], dim=0)
        out[p + "down.weight"] = hf[p + "mlp.down_proj.weight"]
        out[p + "attn_norm.weight"] = hf[p + "input_layernorm.weight"]
        out[p + "mlp_norm.weight"] = hf[p + "post_attention_layernorm.weight"]
        layer += 1
    if layer == 0:
        raise KeyError("the state dict has no decoder layers")
    return {k: v.contiguous() for k, v in out.items()}


_JANUS_SIDE = {
    "gen_embed.weight": "gen_embed.weight",
    "gen_aligner.layers.0.weight": "gen_aligner.fc1.weight", "gen_aligner.layers.0.bias": "gen_aligner.fc1.bias",
    "gen_aligner.layers.2.weight": "gen_aligner.fc2.weight", "gen_aligner.layers.2.bias": "gen_aligner.fc2.bias",
    "gen_head.output_mlp_projector.weight": "gen_head.fc1.weight",
    "gen_head.output_mlp_projector.bias": "gen_head.fc1.bias",
    "gen_head.vision_head.weight": "gen_head.fc2.weight", "gen_head.vision_head.bias": "gen_head.fc2.bias",
}


def janus_from_hf(state: Mapping[str, torch.Tensor], num_heads: int) -> dict[str, torch.Tensor]:
    """State dict of ``JanusNetwork`` (trunk + generation embedding, aligner and head) from a
    Janus-Pro checkpoint; understanding-side modules (vision tower, ``lm_head``) are dropped."""
    out = {f"language_model.{k}": v for k, v in llama_from_hf(state, num_heads).items()}
    missing = [k for k in _JANUS_SIDE if k not in state]
    if missing:
        raise KeyError(f"Janus checkpoint lacks {missing[:3]}")
    out.update({native: state[src].contiguous() for src, native in _JANUS_SIDE.items()})
    return out


def clip_vision_from_hf(state: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """State dict of ``ViTScorer`` (without its scalar head) from a Hugging Face
    ``CLIPVisionModelWithProjection`` / ``CLIPModel`` state dict: the strided patch convolution
    becomes a product over flattened ``(channel, row, column)`` patches, q/k/v are fused, the class
    token and the position table get their leading batch dimensions."""
    vm = "vision_model."
    if vm + "embeddings.class_embedding" not in state:
        raise KeyError("no CLIP vision tower found (vision_model.embeddings.class_embedding)")
    if "visual_projection.weight" not in state:
        raise KeyError("the checkpoint has no visual_projection (a tower without projection head)")
    conv = state[vm + "embeddings.patch_embedding.weight"]
    out: dict[str, torch.Tensor] = {
        "patch_embed.weight": conv.reshape(conv.shape[0], -1),
        "cls": state[vm + "embeddings.class_embedding"].reshape(1, 1, -1),
        "pos": state[vm + "embeddings.position_embedding.weight"].unsqueeze(0),
        "proj.weight": state["visual_projection.weight"],
    }
    for src, dst in (("pre_layrnorm", "pre_norm"), ("post_layernorm", "post_norm")):
        for leaf in ("weight", "bias"):
            out[f"{dst}.{leaf}"] = state[f"{vm}{src}.{leaf}"]
    layer = _clip_blocks(state, vm, out)
    if layer == 0:
        raise KeyError("the CLIP vision tower has no encoder layers")
    return {k: v.contiguous() for k, v in out.items()}


def _clip_blocks(state: Mapping[str, torch.Tensor], prefix: str, out: dict[str, torch.Tensor]) -> int:
    layer = 0
    while f"{prefix}encoder.layers.{layer}.self_attn.q_proj.weight" in state:
        p, q = f"{prefix}encoder.layers.{layer}.", f"blocks.{layer}."
        for leaf in ("weight", "bias"):
            out[q + f"qkv.{leaf}"] = torch.cat([state[p + f"self_attn.{n}_proj.{leaf}"] for n in "qkv"], dim=0)
            out[q + f"out.{leaf}"] = state[p + f"self_attn.out_proj.{leaf}"]
            out[q + f"n1.{leaf}"] = state[p + f"layer_norm1.{leaf}"]
            out[q + f"n2.{leaf}"] = state[p + f"layer_norm2.{leaf}"]
            out[q + f"mlp.fc1.{leaf}"] = state[p + f"mlp.fc1.{leaf}"]
            out[q + f"mlp.fc2.{leaf}"] = state[p + f"mlp.fc2.{leaf}"]
        layer += 1
    return layer


def clip_text_from_hf(state: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """State dict of ``CLIPTextTower`` from a Hugging Face ``CLIPModel`` /
    ``CLIPTextModelWithProjection`` state dict."""
    tm = "text_model."
    if tm + "embeddings.token_embedding.weight" not in state or "text_projection.weight" not in state:
        raise KeyError("no CLIP text tower with projection found (text_model.embeddings.token_embedding.weight, "
                       "text_projection.weight)")
    out: dict[str, torch.Tensor] = {
        "token_embed.weight": state[tm + "embeddings.token_embedding.weight"],
        "pos": state[tm + "embeddings.position_embedding.weight"],
        "final_norm.weight": state[tm + "final_layer_norm.weight"],
        "final_norm.bias": state[tm + "final_layer_norm.bias"],
        "proj.weight": state["text_projection.weight"],
    }
    if _clip_blocks(state, tm, out) == 0:
        raise KeyError("the CLIP text tower has no encoder layers")
    return {k: v.contiguous() for k, v in out.items()}


def clip_text_shape(state: Mapping[str, torch.Tensor]) -> dict[str, int]:
    """``CLIPTextTower`` constructor arguments read off a converted text tower state dict."""
    layers = 1 + max(int(k.split(".")[1]) for k in state if k.startswith("blocks."))
    vocab, dim = (int(v) for v in state["token_embed.weight"].shape)
    return {"layers": layers, "dim": dim, "mlp": int(state["blocks.0.mlp.fc1.weight"].shape[0]), "vocab": vocab,
            "context": int(state["pos"].shape[0]), "out_dim": int(state["proj.weight"].shape[0])}


def clip_vision_shape(state: Mapping[str, torch.Tensor]) -> dict[str, int]:
    """``ViTScorer`` constructor arguments read off a converted (native) tower state dict; the
    head count is not recorded in the weights and has to come from the checkpoint's config."""
    dim = int(state["cls"].shape[-1])
    layers = 1 + max(int(k.split(".")[1]) for k in state if k.startswith("blocks."))
    patch = int(round((state["patch_embed.weight"].shape[1] / 3) ** 0.5))
    grid = int(round((state["pos"].shape[1] - 1) ** 0.5))
    return {"layers": layers, "dim": dim, "mlp": int(state["blocks.0.mlp.fc1.weight"].shape[0]),
            "patch": patch, "image": patch * grid, "out_dim": int(state["proj.weight"].shape[0])}


def t5_encoder_from_hf(state: Mapping[str, torch.Tensor]) -> dict[str, torch.Tensor]:
    """State dict of ``T5Encoder`` from a Hugging Face ``T5EncoderModel`` / ``UMT5EncoderModel``
    state dict (gated or plain feed-forward, shared or per-layer position bias)."""
    if "encoder.block.0.layer.0.SelfAttention.q.weight" not in state:
        raise KeyError("no T5 encoder found (encoder.block.0.layer.0.SelfAttention.q.weight)")
    embed = state.get("shared.weight", state.get("encoder.embed_tokens.weight"))
    if embed is None:
        raise KeyError("the T5 checkpoint has no token embedding (shared.weight)")
    out: dict[str, torch.Tensor] = {"embed.weight": embed, "final_norm.weight": state["encoder.final_layer_norm.weight"]}
    layer = 0
    while f"encoder.block.{layer}.layer.0.SelfAttention.q.weight" in state:
        p, q = f"encoder.block.{layer}.layer.", f"blocks.{layer}."
        for n in "qkvo":
            out[q + f"{n}.weight"] = state[p + f"0.SelfAttention.{n}.weight"]
        bias = p + "0.SelfAttention.relative_attention_bias.weight"
        if bias in state:
            out[q + "rel_bias.weight"] = state[bias]
        out[q + "attn_norm.weight"] = state[p + "0.layer_norm.weight"]
        out[q + "ff_norm.weight"] = state[p + "1.layer_norm.weight"]
        if p + "1.DenseReluDense.wi_0.weight" in state:
            out[q + "wi_0.weight"] = state[p + "1.DenseReluDense.wi_0.weight"]
            out[q + "wi_1.weight"] = state[p + "1.DenseReluDense.wi_1.weight"]
        else:
            out[q + "wi_0.weight"] = state[p + "1.DenseReluDense.wi.weight"]
        out[q + "wo.weight"] = state[p + "1.DenseReluDense.wo.weight"]
        layer += 1
    return {k: v.contiguous() for k, v in out.items()}


def _load_dir(path: str) -> dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    files = sorted(f for f in os.listdir(path) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {path}")
    state: dict[str, torch.Tensor] = {}
    for name in files:
        state.update(load_file(os.path.join(path, name)))
    return state


def main(argv: list[str] | None = None) -> int:
    from safetensors.torch import save_file

    parser = argparse.ArgumentParser(description="Convert a Hugging Face LLaMA-layout checkpoint "
                                                 "directory to the native key layout.")
    parser.add_argument("kind", choices=["llama", "janus", "clip_vision"])
    parser.add_argument("source", help="directory with *.safetensors in the Hugging Face layout")
    parser.add_argument("target", help="directory to write (janus.safetensors / llama.safetensors)")
    parser.add_argument("--num-heads", type=int, default=0, help="attention heads (llama, janus)")
    args = parser.parse_args(argv)
    state = _load_dir(args.source)
    if args.kind == "clip_vision":
        native, name = clip_vision_from_hf(state), "tower"
    else:
        if args.num_heads <= 0:
            parser.error("--num-heads is required for llama and janus")
        native = (janus_from_hf if args.kind == "janus" else llama_from_hf)(state, args.num_heads)
        name = args.kind
    os.makedirs(args.target, exist_ok=True)
    save_file(native, os.path.join(args.target, f"{name}.safetensors"))
    print(f"wrote {len(native)} tensors to {os.path.join(args.target, name + '.safetensors')}")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
