"""Building blocks of the native models.

Every layer calls the functional operators in :mod:`visionrl_b200.ops`, which
run hand-written sm_100a kernels for bf16 CUDA tensors and PyTorch formulas
otherwise, so the same module definitions serve the CPU oracle runs and the
B200 runs.
"""

from __future__ import annotations

import contextlib
import math

import torch
from torch import nn

from visionrl_b200.ops import attention as attn_ops
from visionrl_b200.ops import linear as linear_ops
from visionrl_b200.ops import norm as norm_ops


class Linear(nn.Module):
    """``nn.Linear``-layout weight evaluated by :func:`visionrl_b200.ops.linear.linear`."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True,
                 init_std: float | None = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features))
        self.bias = nn.Parameter(torch.zeros(out_features)) if bias else None
        std = init_std if init_std is not None else 1.0 / math.sqrt(in_features)
        nn.init.normal_(self.weight, std=std)

    # Int4 copy of ``weight`` used for decode-sized inputs while :func:`int4_decode` is active.
    int4_shadow = None
    # Set by :mod:`visionrl_b200.parallel.fsdp` when ``weight`` holds only this rank's rows: the
    # handle gathers the full matrix inside the consuming GEMM and stages the weight gradient.
    sharded = None

    def _base(self, x, act=None, gate=None, residual=None):
        if self.sharded is not None:
            return self.sharded.linear(x, self.bias, act=act, gate=gate, residual=residual)
        shadow = self.int4_shadow
        if (shadow is not None and _INT4_DECODE_ACTIVE and not torch.is_grad_enabled()
                and x.numel() // x.shape[-1] <= 32):
            y = shadow(x)
            return linear_ops.linear_epilogue(y, act, gate, residual)
        return linear_ops.linear(x, self.weight, self.bias, act=act, gate=gate, residual=residual)

    def forward(self, x, act=None, gate=None, residual=None):
        return self._base(x, act=act, gate=gate, residual=residual)

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, bias={self.bias is not None}"
                + (", row-sharded" if self.sharded is not None else ""))

    # A sharded layer still saves and loads the FULL ``[out, in]`` matrix, so checkpoints do not
    # depend on how many ranks wrote them.
    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        if self.sharded is not None:
            destination[prefix + "weight"] = self.sharded.gather_copy()

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        handle = self.sharded
        if handle is not None:
            key = prefix + "weight"
            value = state_dict.get(key)
            if value is not None and tuple(value.shape) == (handle.n, handle.k):
                state_dict[key] = handle.local_rows(value)
            handle.rt.mark_dirty()
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)


class LoRALinear(Linear):
    """Linear with an optional low-rank adapter ``y += (alpha/r) * B(A x)``.

    ``adapter_enabled`` is flipped by :func:`adapters_disabled`; the frozen
    reference policy of LoRA training is the same module with the adapter off
    (reference behaviour: ``vrl/rollouts/evaluators/diffusion/flow_matching.py:82-109``).
    """

    def __init__(self, in_features, out_features, bias=True, init_std=None):
        super().__init__(in_features, out_features, bias, init_std)
        self.lora_A: nn.Parameter | None = None
        self.lora_B: nn.Parameter | None = None
        self.lora_scale = 0.0
        self.adapter_enabled = True
        # extra names under which ``apply_lora`` targets address this layer, e.g. a fused
        # QKV projection answers to ("to_q", "to_k", "to_v")
        self.lora_aliases: tuple = ()

    def add_adapter(self, rank: int, alpha: float, init: str = "gaussian") -> None:
        dev, dt = self.weight.device, self.weight.dtype
        a = torch.empty(rank, self.in_features, device=dev, dtype=dt)
        if init == "gaussian":
            nn.init.normal_(a, std=1.0 / rank)
        else:
            nn.init.kaiming_uniform_(a, a=math.sqrt(5))
        self.lora_A = nn.Parameter(a)
        self.lora_B = nn.Parameter(torch.zeros(self.out_features, rank, device=dev, dtype=dt))
        self.lora_scale = float(alpha) / float(rank)

    @property
    def has_adapter(self) -> bool:
        return self.lora_A is not None

    def forward(self, x, act=None, gate=None, residual=None):
        if not (self.has_adapter and self.adapter_enabled):
            return super().forward(x, act=act, gate=gate, residual=residual)
        y = self._base(x)
        if self._decode_sized(x, y):
            # a handful of rows without autograd (the decode step): two tiny kernels update y in place
            from visionrl_b200.ops import _ext

            x2 = x.reshape(-1, x.shape[-1])
            y2 = y.reshape(-1, y.shape[-1])
            _ext.load().lora_apply_rows(y2, x2 if x2.is_contiguous() else x2.contiguous(), self.lora_A,
                                        self.lora_B, float(self.lora_scale))
            return linear_ops.linear_epilogue(y, act, gate, residual)
        low = linear_ops.linear(x, self.lora_A)
        y = y + self.lora_scale * linear_ops.linear(low, self.lora_B)
        return linear_ops.linear_epilogue(y, act, gate, residual)

    def _decode_sized(self, x, y) -> bool:
        from visionrl_b200.ops import _ext

        a, b = self.lora_A, self.lora_B
        return (not torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16
                and y.dtype == torch.bfloat16 and y.is_contiguous()
                and x.numel() // x.shape[-1] <= 64 and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
                and a.is_contiguous() and b.is_contiguous() and a.shape[0] % 8 == 0 and 8 <= a.shape[0] <= 256
                and x.shape[-1] % 8 == 0 and _ext.kernels_enabled() and _ext.has("lora_apply_rows"))


_INT4_DECODE_ACTIVE = False


@contextlib.contextmanager
def int4_decode(active: bool = True):
    """While active, layers holding an ``int4_shadow`` serve decode-sized calls from it."""
    global _INT4_DECODE_ACTIVE
    previous = _INT4_DECODE_ACTIVE
    _INT4_DECODE_ACTIVE = bool(active)
    try:
        yield
    finally:
        _INT4_DECODE_ACTIVE = previous


def attach_int4_shadows(module: nn.Module, group: int = 128) -> int:
    """Quantise the frozen base weight of every eligible linear under ``module`` to int4.

    Only weights that do not receive gradients are shadowed (LoRA leaves the base frozen, so
    the copy stays valid for the whole run); returns the number of layers covered.
    """
    from visionrl_b200.ops.quant import Int4Linear

    count = 0
    for sub in module.modules():
        if isinstance(sub, Linear) and not sub.weight.requires_grad and sub.in_features % 256 == 0:
            # plain attribute, not a registered submodule: the copy must stay out of state_dict()
            object.__setattr__(sub, "int4_shadow", Int4Linear(sub, group))
            count += 1
    return count


def iter_lora_layers(module: nn.Module):
    for m in module.modules():
        if isinstance(m, LoRALinear) and m.has_adapter:
            yield m


@contextlib.contextmanager
def adapters_disabled(module: nn.Module):
    layers = list(iter_lora_layers(module))
    if not layers:
        raise RuntimeError("disable_adapter() called on a model without LoRA adapters")
    previous = [m.adapter_enabled for m in layers]
    for m in layers:
        m.adapter_enabled = False
    try:
        yield
    finally:
        for m, flag in zip(layers, previous):
            m.adapter_enabled = flag


@contextlib.contextmanager
def adapters_zeroed(module: nn.Module):
    """Inside the block every adapter's ``B`` factor is zero, so the network IS its base model —
    also for a copy of it that receives these tensors through a weight push — and afterwards the
    trained values are back.  (``adapters_disabled`` only flips a flag of this module object.)"""
    layers = list(iter_lora_layers(module))
    if not layers:
        raise RuntimeError("adapters_zeroed() called on a model without LoRA adapters")
    saved = [m.lora_B.detach().clone() for m in layers]
    with torch.no_grad():
        for m in layers:
            m.lora_B.zero_()
    try:
        yield
    finally:
        with torch.no_grad():
            for m, b in zip(layers, saved):
                m.lora_B.copy_(b)


def apply_lora(module: nn.Module, rank: int, alpha: float, target_modules, init="gaussian",
               freeze_base: bool = True) -> list[str]:
    """Attach adapters to every :class:`LoRALinear` whose qualified name ends with a target
    or whose ``lora_aliases`` contain one.  A fused projection that answers to several
    targets (q/k/v) receives a single adapter spanning the fused output."""
    targets = tuple(target_modules)
    hit: list[str] = []
    if freeze_base:
        for p in module.parameters():
            p.requires_grad_(False)
    for name, m in module.named_modules():
        if not isinstance(m, LoRALinear):
            continue
        direct = any(name == t or name.endswith("." + t) for t in targets)
        if direct or any(alias in targets for alias in m.lora_aliases):
            m.add_adapter(rank, alpha, init)
            hit.append(name)
    if not hit:
        raise ValueError(f"no LoRA target matched {list(targets)}")
    return hit


ADAPTER_WEIGHTS_NAME = "adapter_model.safetensors"
ADAPTER_CONFIG_NAME = "adapter_config.json"


def lora_state_dict(module: nn.Module) -> dict[str, torch.Tensor]:
    """``<layer>.lora_A`` / ``<layer>.lora_B`` of every adapter under ``module``, on the CPU, under
    the names ``module.load_state_dict`` knows them by.  Adapters are never sharded, so reading them
    is local to the rank."""
    out: dict[str, torch.Tensor] = {}
    for name, m in module.named_modules():
        if isinstance(m, LoRALinear) and m.has_adapter:
            prefix = f"{name}." if name else ""
            out[prefix + "lora_A"] = m.lora_A.detach().to("cpu").contiguous()
            out[prefix + "lora_B"] = m.lora_B.detach().to("cpu").contiguous()
    return out


def save_lora_adapter(module: nn.Module, directory) -> dict:
    """Write the adapters of ``module`` as ``adapter_model.safetensors`` + ``adapter_config.json``
    (the two files of the ``lora_weights/`` export a training checkpoint carries, reference
    ``vrl/trainers/checkpointing.py``); returns the config that was written."""
    import json
    import os

    from safetensors.torch import save_file

    layers = [(n, m) for n, m in module.named_modules() if isinstance(m, LoRALinear) and m.has_adapter]
    if not layers:
        raise RuntimeError("save_pretrained() called on a model without LoRA adapters")
    os.makedirs(directory, exist_ok=True)
    ranks = sorted({int(m.lora_A.shape[0]) for _, m in layers})
    config = {"peft_type": "LORA", "r": ranks[0] if len(ranks) == 1 else ranks,
              "lora_alpha": float(layers[0][1].lora_scale) * int(layers[0][1].lora_A.shape[0]),
              "target_modules": [n for n, _ in layers], "bias": "none",
              "base_model_class": type(module).__name__}
    save_file(lora_state_dict(module), os.path.join(directory, ADAPTER_WEIGHTS_NAME))
    with open(os.path.join(directory, ADAPTER_CONFIG_NAME), "w") as fh:
        json.dump(config, fh, indent=2, sort_keys=True)
        fh.write("\n")
    return config


def load_lora_adapter(module: nn.Module, directory) -> list[str]:
    """Load an export written by :func:`save_lora_adapter` into the adapters ``module`` already
    has.  Every tensor of the file must have a place of the same shape and every adapter of the
    module must be in the file; returns the keys that were loaded."""
    import os

    from safetensors.torch import load_file

    state = load_file(os.path.join(str(directory), ADAPTER_WEIGHTS_NAME))
    have = lora_state_dict(module)
    unexpected = sorted(set(state) - set(have))
    missing = sorted(set(have) - set(state))
    if unexpected:
        raise ValueError(f"unexpected LoRA keys: {unexpected[:4]}")
    if missing:
        raise ValueError(f"adapter file lacks LoRA keys: {missing[:4]}")
    for key, value in state.items():
        if tuple(value.shape) != tuple(have[key].shape):
            raise ValueError(f"LoRA tensor {key}: file has {tuple(value.shape)}, model has {tuple(have[key].shape)}")
    params = dict(module.named_parameters())
    with torch.no_grad():
        for key, value in state.items():
            params[key].copy_(value.to(params[key].device, params[key].dtype))
    return sorted(state)


class AdapterMixin:
    """Gives a network ``disable_adapter()`` / ``has_adapters`` over its LoRA layers and the
    adapter export / import of a checkpoint's ``lora_weights/`` directory."""

    def disable_adapter(self):
        return adapters_disabled(self)

    @property
    def has_adapters(self) -> bool:
        return any(True for _ in iter_lora_layers(self))

    def save_pretrained(self, directory) -> dict:
        return save_lora_adapter(self, directory)

    def load_adapter(self, directory) -> list[str]:
        return load_lora_adapter(self, directory)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim))
        self.eps = eps

    def forward(self, x):
        return norm_ops.rmsnorm(x, self.weight, self.eps)


class LayerNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-5, affine: bool = True):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim)) if affine else None
        self.bias = nn.Parameter(torch.zeros(dim)) if affine else None
        self.eps = eps

    def forward(self, x):
        return norm_ops.layernorm(x, self.weight, self.bias, self.eps)


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    """Sinusoidal embedding of (possibly fractional) timesteps, fp32, ``[B, dim]``."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, device=t.device,
                                                           dtype=torch.float32) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class TimestepEmbedder(nn.Module):
    def __init__(self, hidden: int, freq_dim: int = 256):
        super().__init__()
        self.freq_dim = freq_dim
        self.fc1 = Linear(freq_dim, hidden)
        self.fc2 = Linear(hidden, hidden)

    def forward(self, t, dtype):
        e = timestep_embedding(t, self.freq_dim).to(dtype)
        return self.fc2(self.fc1(e, act="silu"))


class MLP(nn.Module):
    def __init__(self, dim: int, hidden: int, act: str = "gelu_tanh"):
        super().__init__()
        self.fc1 = Linear(dim, hidden)
        self.fc2 = Linear(hidden, dim)
        self.act = act

    def forward(self, x, gate=None, residual=None):
        plain = type(self.fc1) is Linear and type(self.fc2) is Linear
        if plain and self.act == "gelu_tanh" and self.fc1.sharded is not None \
                and self.fc2.sharded is not None and torch.is_grad_enabled():
            from visionrl_b200.parallel.fsdp import sharded_gelu_mlp

            y = sharded_gelu_mlp(x, self.fc1, self.fc2)
            return linear_ops.linear_epilogue(y, None, gate, residual)
        if (plain and self.act == "gelu_tanh" and torch.is_grad_enabled()
                and self.fc1.sharded is None and self.fc2.sharded is None
                and self.fc1.int4_shadow is None and self.fc2.int4_shadow is None):
            y = linear_ops.gelu_mlp(x, self.fc1.weight, self.fc1.bias, self.fc2.weight, self.fc2.bias)
            return linear_ops.linear_epilogue(y, None, gate, residual)
        return self.fc2(self.fc1(x, act=self.act), gate=gate, residual=residual)


def split_heads(x: torch.Tensor, heads: int) -> torch.Tensor:
    b, s, d = x.shape
    return x.view(b, s, heads, d // heads).transpose(1, 2)


def merge_heads(x: torch.Tensor) -> torch.Tensor:
    b, h, s, d = x.shape
    return x.transpose(1, 2).reshape(b, s, h * d)


def sdpa(q, k, v, causal: bool = False):
    return attn_ops.attention(q, k, v, causal=causal)
