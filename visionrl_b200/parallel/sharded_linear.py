"""One row-sharded linear weight whose all-gather is fused into the consuming GEMM (kernel F1).

This is the single-layer form, kept for micro-benchmarks and kernel tests; whole models are
sharded by :mod:`visionrl_b200.parallel.fsdp`, which drives the same kernel from a shared ring of
gather buffers.

Every rank keeps ``N / world`` rows of a ``[N, K]`` weight in symmetric memory.  A forward call
launches ONE kernel: 128 extra threads per CTA copy the peers' rows into the local full-weight
buffer over NVLink (own rows first) while the tensor-core warps already work on the tiles whose
rows have arrived; per-shard arrival counters with bounded waits order the two.  The NCCL
formulation of the same step — ``all_gather_into_tensor`` followed by a GEMM — is kept as the
baseline (`collectives="nccl"`) and as the oracle of the tests.  The reference has the all-gather
only implicitly, inside FSDP1 (``vrl/trainers/fsdp.py:69-87``).
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist

from visionrl_b200.ops.linear import linear_reference


class ShardedLinearWeight:
    """One ``[N, K]`` bf16 weight (and optional bias) sharded by rows over the pool's group."""

    def __init__(self, pool: Any, out_features: int, in_features: int, device: Any,
                 bias: bool = False, collectives: str = "fused") -> None:
        if out_features % pool.world:
            raise ValueError(f"out_features ({out_features}) must divide by the group size ({pool.world})")
        self.pool, self.world, self.rank = pool, pool.world, pool.rank
        self.out_features, self.in_features = out_features, in_features
        self.rows = out_features // pool.world
        self.collectives = collectives
        self.shard = pool.allocate(self.rows * in_features, torch.bfloat16, device, "weight_shard") \
            .view(self.rows, in_features)
        self.full = torch.empty(out_features, in_features, device=device, dtype=torch.bfloat16)
        self.ready = torch.zeros(16, device=device, dtype=torch.int32)
        self.bias = torch.zeros(out_features, device=device, dtype=torch.bfloat16) if bias else None
        self.kernel_launches = 0

    def load_full(self, weight: torch.Tensor) -> None:
        """Keep this rank's rows of a replicated ``[N, K]`` tensor (test / initialisation helper)."""
        lo = self.rank * self.rows
        self.shard.copy_(weight[lo:lo + self.rows].to(torch.bfloat16))

    def forward(self, x: torch.Tensor, act: str | None = None) -> torch.Tensor:
        """``act(x @ W.T + bias)`` with ``W`` gathered from all ranks.

        Every rank's shard must be final before any rank calls this (the optimizer step that
        wrote it is followed by a barrier).
        """
        from visionrl_b200.ops import _ext
        from visionrl_b200.ops.linear import _ACTS

        x2 = x.reshape(-1, x.shape[-1])
        fused = (self.collectives == "fused" and x2.is_cuda and x2.dtype == torch.bfloat16
                 and _ext.kernels_enabled() and _ext.has("gemm_allgather"))
        if fused:
            y = _ext.load().gemm_allgather(x2.contiguous(), self.pool.peer_pointers(self.shard.view(-1)),
                                           self.full, self.ready, self.bias, _ACTS[act], self.rank,
                                           self.world, None, None, 0, False)[0]
            self.kernel_launches += 1
        else:
            dist.all_gather_into_tensor(self.full.view(-1), self.shard.reshape(-1).contiguous(),
                                        group=self.pool.group)
            y = linear_reference(x2, self.full, self.bias, act)
        return y.view(*x.shape[:-1], self.out_features)


__all__ = ["ShardedLinearWeight"]
