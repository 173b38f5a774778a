"""Ulysses sequence parallelism for the video DiT (F3).

Token-wise layers run on a contiguous ``S/P`` slice of the sequence.  Around attention the
layout changes from (all heads, local tokens) to (local heads, all tokens) and back.  On B200
both exchanges are peer stores issued by the producing kernel into the consumer's symmetric
buffer — the head split / QK-norm / RoPE epilogue of the QKV projection writes straight into the
destination rank's ``[B, H/P, S, Dh]`` buffers, and the attention output is written straight
into each rank's merged-head ``[B, S/P, H*Dh]`` buffer that its output projection reads.  A
symmetric-memory barrier orders producer stores before consumer loads.  Without CUDA (gloo
tests) and as the measured baseline the same exchange is an ``all_to_all_single``.
"""

from __future__ import annotations

from typing import Any

import torch
import torch.distributed as dist


def _all_to_all_heads(x: torch.Tensor, group: Any, world: int) -> torch.Tensor:
    """``[B, H, S_loc, D]`` → ``[B, H/P, S, D]`` through the library collective."""
    b, h, s, d = x.shape
    send = x.reshape(b, world, h // world, s, d).permute(1, 0, 2, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[r] holds sequence slice r of this rank's head group
    return recv.permute(1, 2, 0, 3, 4).reshape(b, h // world, world * s, d)


def _all_to_all_seq(x: torch.Tensor, group: Any, world: int) -> torch.Tensor:
    """``[B, H/P, S, D]`` → ``[B, H, S_loc, D]`` through the library collective."""
    b, hp, s, d = x.shape
    s_loc = s // world
    send = x.reshape(b, hp, world, s_loc, d).permute(2, 0, 1, 3, 4).contiguous()
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    return recv.permute(1, 0, 2, 3, 4).reshape(b, world * hp, s_loc, d)


class _HeadExchange(torch.autograd.Function):
    """to_heads in forward, to_seq in backward (and vice versa with ``inverse``)."""

    @staticmethod
    def forward(ctx, x, sp, inverse):
        ctx.sp, ctx.inverse = sp, inverse
        return sp._seq_to_local(x) if inverse else sp._heads_to_local(x)

    @staticmethod
    def backward(ctx, g):
        sp = ctx.sp
        g = g.contiguous()
        return (sp._heads_to_local(g) if ctx.inverse else sp._seq_to_local(g)), None, None


class SequenceParallel:
    def __init__(self, mesh: Any, pool: Any | None = None) -> None:
        self.mesh = mesh
        self.group = mesh.sp_group
        self.world = mesh.sp
        self.rank = mesh.sp_rank
        self.pool = pool
        self._buffers: dict[tuple, torch.Tensor] = {}
        self.kernel_launches = 0

    # -- sequence sharding of token tensors -------------------------------------------------
    def shard_sequence(self, x: torch.Tensor) -> torch.Tensor:
        s = x.shape[1]
        if s % self.world != 0:
            raise ValueError(f"sequence length {s} is not divisible by sp={self.world}")
        n = s // self.world
        return x[:, self.rank * n:(self.rank + 1) * n].contiguous()

    def shard_rows(self, x: torch.Tensor) -> torch.Tensor:
        n = x.shape[0] // self.world
        return x[self.rank * n:(self.rank + 1) * n].contiguous()

    def gather_sequence(self, x: torch.Tensor) -> torch.Tensor:
        parts = [torch.empty_like(x) for _ in range(self.world)]
        dist.all_gather(parts, x.contiguous(), group=self.group)
        parts[self.rank] = x          # keep the autograd path of the local slice
        return torch.cat(parts, dim=1)

    # -- exchanges ---------------------------------------------------------------------------
    def _use_kernels(self, x: torch.Tensor) -> bool:
        from visionrl_b200.ops import _ext

        return (self.pool is not None and x.is_cuda and x.element_size() == 2
                and _ext.kernels_enabled() and _ext.has("ulysses_scatter"))

    def _buffer(self, kind: str, shape: tuple, dtype, device) -> torch.Tensor:
        key = (kind, shape, dtype)
        buf = self._buffers.get(key)
        if buf is None:
            numel = 1
            for v in shape:
                numel *= v
            buf = self.pool.allocate(numel, dtype, device, kind).view(shape)
            self._buffers[key] = buf
        return buf

    def _heads_to_local(self, x: torch.Tensor) -> torch.Tensor:
        b, h, s, d = x.shape
        if not self._use_kernels(x):
            return _all_to_all_heads(x, self.group, self.world)
        from visionrl_b200.ops import _ext

        out = self._buffer("to_heads", (b, h // self.world, s * self.world, d), x.dtype, x.device)
        self.pool.barrier()        # the previous consumer of `out` on every peer is done
        _ext.load().ulysses_scatter(x.contiguous(), self.pool.peer_pointers(out), b, h, s, d,
                                    self.world, self.rank, True)
        self.pool.barrier()        # every peer's stores into `out` have landed
        self.kernel_launches += 1
        return out.clone()

    def _seq_to_local(self, x: torch.Tensor) -> torch.Tensor:
        b, hp, s, d = x.shape
        if not self._use_kernels(x):
            return _all_to_all_seq(x, self.group, self.world)
        from visionrl_b200.ops import _ext

        s_loc, h = s // self.world, hp * self.world
        out = self._buffer("to_seq", (b, s_loc, h, d), x.dtype, x.device)
        self.pool.barrier()
        _ext.load().ulysses_scatter(x.contiguous(), self.pool.peer_pointers(out), b, h, s_loc, d,
                                    self.world, self.rank, False)
        self.pool.barrier()
        self.kernel_launches += 1
        return out.permute(0, 2, 1, 3).contiguous()     # [B, H, S_loc, D]

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """``q, k, v`` ``[B, H, S/P, D]`` → attention over the full sequence → ``[B, H, S/P, D]``."""
        from visionrl_b200.ops.attention import attention

        if self.world == 1:
            return attention(q, k, v)
        qh = _HeadExchange.apply(q, self, False)
        kh = _HeadExchange.apply(k, self, False)
        vh = _HeadExchange.apply(v, self, False)
        o = attention(qh, kh, vh)
        return _HeadExchange.apply(o, self, True)


def attach_sequence_parallel(policy: Any, mesh: Any, pool: Any | None = None) -> SequenceParallel:
    """Switch a video policy to sequence-parallel execution over ``mesh.sp_group``."""
    heads = int(policy.arch["num_heads"])
    if heads % mesh.sp != 0:
        raise ValueError(f"num_heads={heads} is not divisible by sp={mesh.sp}")
    if pool is None and torch.cuda.is_available() and mesh.sp > 1:
        from visionrl_b200.ops import _ext

        if _ext.kernels_enabled() and _ext.available():
            from visionrl_b200.parallel.symm import SymmetricPool

            pool = SymmetricPool(mesh, group=mesh.sp_group)
    sp = SequenceParallel(mesh, pool)
    policy.sequence_parallel = sp
    return sp
