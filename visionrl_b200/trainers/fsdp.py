"""Sharded-training utilities under the reference's ``vrl.trainers.fsdp`` names
(``vrl/trainers/fsdp.py:35-183``).

``fsdp_wrapper`` attaches the native sharded runtime instead of wrapping modules in
``torch.distributed.fsdp``: with ``FULL_SHARD`` / ``HYBRID_SHARD`` the transformer-block weights,
their gradients and optimiser state are sharded over the shard group
(:mod:`visionrl_b200.parallel.fsdp`: all-gather inside the consuming GEMM, bucketed
reduce-scatter during backward), with ``SHARD_GRAD_OP`` only the optimiser state of flat bf16
parameters is (:mod:`visionrl_b200.parallel.sharded`), ``NO_SHARD`` replicates everything.
``save_fsdp_checkpoint`` writes rank 0's full state dict to
``checkpoint-<step>/model.safetensors`` and then barriers.
"""

from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from visionrl_b200.parallel.mesh import ProcessMesh, dist_ready
from visionrl_b200.parallel.mesh import init_distributed as _init_distributed


@dataclass
class FSDPConfig:
    sharding_strategy: str = "FULL_SHARD"       # FULL_SHARD | SHARD_GRAD_OP | HYBRID_SHARD | NO_SHARD
    backward_prefetch: str = "BACKWARD_PRE"
    cpu_offload: bool = False
    num_replicate: int = 1
    num_shard: int = 8
    mixed_precision_dtype: torch.dtype = torch.bfloat16
    use_activation_checkpointing: bool = False
    use_device_mesh: bool = False


def fsdp_wrapper(model: nn.Module, fsdp_config: FSDPConfig | None = None,
                 get_transformer_layer_cls: Any = None, ignored_modules: list[nn.Module] | None = None, *,
                 mesh: ProcessMesh | None = None, collectives: str = "fused") -> nn.Module:
    """Prepare ``model`` for sharded training and return it (same object).

    Arguments as in the reference (``vrl/trainers/fsdp.py:49-54``): ``get_transformer_layer_cls()``
    returns the block classes whose instances are the sharding units (default: the model's
    ``blocks`` / ``layers`` list), ``ignored_modules`` are left whole.  The returned module carries
    ``model.sharded_runtime`` — the object trainers pass as ``grad_sync`` so that gradient
    reduction, clipping and the sharded AdamW update run as one fused step.
    """
    from visionrl_b200.parallel.sharded import ShardedGradSync

    config = fsdp_config or FSDPConfig()
    if mesh is None:
        hybrid = config.sharding_strategy == "HYBRID_SHARD" and config.num_replicate > 1
        mesh = ProcessMesh.build(replicate=config.num_replicate if hybrid else 1)
    if config.use_activation_checkpointing:
        enable = getattr(model, "enable_gradient_checkpointing", None)
        inner = getattr(model, "transformer", None)
        if callable(enable):
            enable(True)
        elif inner is not None and callable(getattr(inner, "enable_gradient_checkpointing", None)):
            inner.enable_gradient_checkpointing(True)
    shard = config.sharding_strategy != "NO_SHARD"
    param_runtime = None
    if config.sharding_strategy in ("FULL_SHARD", "HYBRID_SHARD") and mesh.world_size > 1:
        from visionrl_b200.parallel.fsdp import shard_model

        first = next(model.parameters(), None)
        device = first.device if first is not None else torch.device("cpu")
        param_runtime = shard_model(model, mesh, device, collectives=collectives,
                                    units=sharding_units(model, get_transformer_layer_cls, ignored_modules))
        model.param_runtime = param_runtime
    model.sharded_runtime = ShardedGradSync(mesh, shard_optimizer=shard, collectives=collectives,
                                            param_runtime=param_runtime)
    return model


def sharding_units(model: nn.Module, get_transformer_layer_cls: Any = None,
                   ignored_modules: list[nn.Module] | None = None) -> list[nn.Module] | None:
    """The blocks to shard: instances of the classes ``get_transformer_layer_cls()`` returns (or the
    model's own block list when no classes are named: ``None``), minus everything inside an ignored
    module."""
    from visionrl_b200.parallel.fsdp import find_units

    ignored = {id(m) for root in (ignored_modules or []) for m in root.modules()}
    if get_transformer_layer_cls is None:
        if not ignored:
            return None
        units = find_units(model)
    else:
        classes = tuple(get_transformer_layer_cls() if callable(get_transformer_layer_cls)
                        else get_transformer_layer_cls)
        units = [m for m in model.modules() if isinstance(m, classes)] if classes else []
    return [u for u in units if id(u) not in ignored]


def save_fsdp_checkpoint(save_dir: str, model: nn.Module, global_step: int, rank: int | None = None) -> str:
    """Rank 0 writes the full state dict to ``<save_dir>/checkpoint-<global_step>/model.safetensors``
    (every rank takes part in gathering sharded weights), then all ranks meet at a barrier.  Argument
    order as in the reference (``vrl/trainers/fsdp.py:106-111``); returns the directory."""
    if rank is None:
        rank = dist.get_rank() if dist_ready() else 0
    path = os.path.join(save_dir, f"checkpoint-{global_step}")
    state = model.state_dict()
    if rank == 0:
        from safetensors.torch import save_file

        os.makedirs(path, exist_ok=True)
        save_file({k: v.detach().cpu().contiguous() for k, v in state.items()}, os.path.join(path, "model.safetensors"))
    del state
    if dist_ready():
        dist.barrier()
    return path


class OptimizerOffloadHook:
    """Keeps optimiser state in host memory between steps: the pre-step hook brings every state
    tensor back to its parameter's device, the post-step hook parks it on the host again
    (reference: ``vrl/trainers/fsdp.py:131-160``).  The flat moment buffers of
    ``visionrl_b200.ops.optim.FusedAdamW`` are handled the same way."""

    def __init__(self) -> None:
        self.cpu_states: dict[Any, dict[str, torch.Tensor]] = {}

    @staticmethod
    def _flat_entries(optimizer: Any) -> list:
        return list(getattr(optimizer, "_flat", []) or [])

    def pre_step_hook(self, optimizer: Any, args: Any = None, kwargs: Any = None) -> None:
        for group in optimizer.param_groups:
            for param in group["params"]:
                parked = self.cpu_states.pop(param, None)
                if parked and param in optimizer.state:
                    for key, tensor in parked.items():
                        optimizer.state[param][key] = tensor.to(param.device, non_blocking=True)
        for i, entry in enumerate(self._flat_entries(optimizer)):
            parked = self.cpu_states.pop(("flat", i), None)
            if parked:
                for key, tensor in parked.items():
                    entry[key] = tensor.to(entry["param"].device, non_blocking=True)

    def post_step_hook(self, optimizer: Any, args: Any = None, kwargs: Any = None) -> None:
        for group in optimizer.param_groups:
            for param in group["params"]:
                state = optimizer.state.get(param)
                if not state:
                    continue
                parked = {}
                for key, value in state.items():
                    if isinstance(value, torch.Tensor) and value.numel() > 1:
                        parked[key] = value.to("cpu", non_blocking=True)
                        state[key] = torch.empty(0, device=param.device, dtype=value.dtype)
                if parked:
                    self.cpu_states[param] = parked
        for i, entry in enumerate(self._flat_entries(optimizer)):
            parked = {}
            for key in ("exp_avg", "exp_avg_sq"):
                value = entry.get(key)
                if isinstance(value, torch.Tensor) and value.numel():
                    parked[key] = value.to("cpu", non_blocking=True)
                    entry[key] = torch.empty(0, device=value.device, dtype=value.dtype)
            if parked:
                self.cpu_states[("flat", i)] = parked


def register_optimizer_offload_hooks(optimizer: torch.optim.Optimizer) -> tuple[list[Any], OptimizerOffloadHook]:
    """Register the two hooks; returns ``([pre_handle, post_handle], hook)`` as the reference does.
    State that already exists is parked at once."""
    hook = OptimizerOffloadHook()
    handles = [optimizer.register_step_pre_hook(hook.pre_step_hook),
               optimizer.register_step_post_hook(hook.post_step_hook)]
    hook.post_step_hook(optimizer)
    return handles, hook


def init_distributed(backend: str | None = None) -> tuple[bool, int, int, int]:
    """``env://`` rendezvous (NCCL on GPUs, gloo otherwise) →
    ``(is_distributed, rank, world_size, local_rank)``; ``(False, 0, 1, 0)`` without a launcher
    (reference: ``vrl/trainers/fsdp.py:172-183``)."""
    rank, world, local = _init_distributed(backend)
    return dist_ready(), rank, world, local


__all__ = ["FSDPConfig", "OptimizerOffloadHook", "fsdp_wrapper", "init_distributed",
           "register_optimizer_offload_hooks", "save_fsdp_checkpoint", "sharding_units"]
