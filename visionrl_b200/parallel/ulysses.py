"""Ulysses sequence parallelism for the video DiT (F3).

Token-wise layers run on a contiguous ``S/P`` slice of the sequence.  Around attention the
layout changes from (all heads, local tokens) to (local heads, all tokens) and back.  What
happens at each stage, per attention layer:

*Fused path* (``fused_attention``; bf16 on CUDA with a symmetric pool):

1. the kernel that finishes the QKV projection — head split, QK-RMSNorm, RoPE — stores every
   head straight into the ``[B, S, H/P, Dh]`` q / k / v buffers of the rank that owns the head
   (plain peer stores over NVLink; ``qkv_prepare_fwd_peers``).  No separate exchange kernel, no
   staging copy;
2. one flag store per peer says "my rows of exchange n are in" and one bounded flag wait holds
   the stream until every peer has said so.  Buffers are double-buffered by exchange parity and
   a second flag ("exchange n has been read") gates their reuse two exchanges later, so no
   barrier is ever on the critical path;
3. attention runs on the local heads over the full sequence.  Without gradients its epilogue
   stores each output row into the ``[B, S/P, H, Dh]`` buffer of the rank that owns the token
   (``flash_attn_fwd_peers``) and the output projection reads that buffer as a merged-head
   ``[B, S/P, H·Dh]`` view; with gradients the output is kept locally for the backward pass and
   sent by one token-major exchange kernel;
4. backward mirrors this with token-major exchange kernels (``ulysses_exchange_tm``): dO to the
   head owners, dQ / dK / dV back to the token owners, then the QKV-prepare backward.

*Library path* (CPU / gloo tests, ``collectives: nccl`` baseline): the same two layout changes
as ``all_to_all_single`` calls around a local attention.

The final ``gather_sequence`` of the model output is an all-gather of the small ``[B, S/P, C]``
velocity patches (NCCL / gloo).  The reference has no sequence parallelism at all
(``vrl/models/families/wan_2_1/official_policy.py:304-314`` passes ``use_sp: False``).
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


_KINDS = ("qkv", "o", "do", "dqkv")


class SequenceParallel:
    def __init__(self, mesh: Any, pool: Any | None = None) -> None:
        self.mesh = mesh
        self.group = mesh.sp_group
        self.world = mesh.sp
        self.rank = mesh.sp_rank
        self.pool = pool
        self._buffers: dict[tuple, torch.Tensor] = {}
        self.kernel_launches = 0
        self.fused_layers = 0
        # exchange counters per buffer kind (identical on every rank: exchanges are collective)
        self._count = {k: 0 for k in _KINDS}
        self._pending_read: tuple | None = None      # an output view whose consumer is not enqueued yet
        self._flag_base = pool.reserve_slots(len(_KINDS) * 2 * 2 * 16) if pool is not None else 0

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

    # -- flags and buffers of the fused path ------------------------------------------------------
    def _use_kernels(self, x: torch.Tensor) -> bool:
        from visionrl_b200.ops import _ext

        return (self.pool is not None and x.is_cuda and x.element_size() == 2
                and _ext.kernels_enabled() and _ext.has("ulysses_exchange_tm"))

    def _buffer(self, kind: str, slot: int, shape: tuple, dtype, device) -> torch.Tensor:
        key = (kind, slot, shape, dtype)
        buf = self._buffers.get(key)
        if buf is None:
            numel = 1
            for v in shape:
                numel *= v
            buf = self.pool.allocate(numel, dtype, device, kind).view(shape)
            self._buffers[key] = buf
        return buf

    def _flag(self, kind: str, slot: int, which: int) -> int:
        """First of the 16 flag slots (one per rank) of (kind, buffer slot, ready=0 / read=1)."""
        return self._flag_base + ((_KINDS.index(kind) * 2 + slot) * 2 + which) * 16

    def _begin(self, kind: str) -> tuple[int, int]:
        """Start exchange ``n`` of ``kind``: returns ``(n, slot)`` once the destination buffers of
        that slot may be overwritten on every peer (they were last used by exchange ``n - 2``)."""
        if self._pending_read is not None:
            # whatever consumes the previous layer's output view has been enqueued by now
            pending, self._pending_read = self._pending_read, None
            self._read(*pending)
        self._count[kind] += 1
        n = self._count[kind]
        slot = n & 1
        if n > 2:
            self.pool.wait(self._flag(kind, slot, 1), self.world, n - 2)
            self.kernel_launches += 1
        return n, slot

    def _written(self, kind: str, slot: int, n: int) -> None:
        """This rank's stores of exchange ``n`` are enqueued: publish, then wait for every peer's."""
        self.pool.signal(self._flag(kind, slot, 0) + self.rank, n)
        self.pool.wait(self._flag(kind, slot, 0), self.world, n)
        self.kernel_launches += 2

    def _read(self, kind: str, slot: int, n: int) -> None:
        """Everything enqueued so far has consumed this rank's buffers of exchange ``n``."""
        self.pool.signal(self._flag(kind, slot, 1) + self.rank, n)
        self.kernel_launches += 1

    def _exchange_tm(self, kind: str, src: torch.Tensor, batch: int, s_loc: int, chunk: int,
                     to_heads: bool, count: int = 1) -> list[torch.Tensor]:
        """Token-major exchange of ``count`` tensors packed in ``src`` (list of contiguous tensors)."""
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        n, slot = self._begin(kind)
        outs = []
        for i, t in enumerate(src):
            shape = (batch, s_loc * self.world, chunk) if to_heads else (batch, s_loc, self.world, chunk)
            dst = self._buffer(f"{kind}{i}", slot, shape, t.dtype, t.device)
            ext.ulysses_exchange_tm(t, self.pool.peer_pointers(dst), batch, s_loc, chunk, self.world,
                                    self.rank, to_heads)
            outs.append(dst)
        self.kernel_launches += len(outs)
        self._written(kind, slot, n)
        return outs, n, slot

    # -- library exchanges ---------------------------------------------------------------------------
    def _heads_to_local(self, x: torch.Tensor) -> torch.Tensor:
        return _all_to_all_heads(x, self.group, self.world)

    def _seq_to_local(self, x: torch.Tensor) -> torch.Tensor:
        return _all_to_all_seq(x, self.group, self.world)

    def attention(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor) -> torch.Tensor:
        """``q, k, v`` ``[B, H, S/P, D]`` → attention over the full sequence → ``[B, H, S/P, D]``
        (library exchanges; the fused path starts one step earlier, at :meth:`fused_attention`)."""
        from visionrl_b200.ops.attention import attention

        if self.world == 1:
            return attention(q, k, v)
        qh = _HeadExchange.apply(q, self, False)
        kh = _HeadExchange.apply(k, self, False)
        vh = _HeadExchange.apply(v, self, False)
        o = attention(qh, kh, vh)
        return _HeadExchange.apply(o, self, True)

    # -- fused path ------------------------------------------------------------------------------------
    def can_fuse(self, qkv: torch.Tensor, heads: int) -> bool:
        from visionrl_b200.ops import _ext

        dh = qkv.shape[-1] // (3 * heads)
        return (self.world > 1 and self._use_kernels(qkv) and qkv.dtype == torch.bfloat16
                and dh in (64, 128) and heads % self.world == 0 and qkv.shape[-1] <= 16384
                and _ext.has("qkv_prepare_fwd_peers") and _ext.has("flash_attn_fwd_peers"))

    def fused_attention(self, qkv: torch.Tensor, heads: int, q_weight, k_weight, rope, eps: float = 1e-6):
        """Fused QKV post-processing + exchange + attention + exchange.

        ``qkv`` is the projection output ``[B, S/P, 3·H·Dh]`` of this rank's tokens; the result is
        the attention output of the same tokens with merged heads, ``[B, S/P, H·Dh]`` — what the
        output projection consumes."""
        cos, sin = rope if rope is not None else (None, None)
        return _FusedUlyssesFn.apply(qkv, q_weight, k_weight, cos, sin, self, int(heads), float(eps))


class _FusedUlyssesFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, q_weight, k_weight, cos, sin, sp: SequenceParallel, heads: int, eps: float):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        pool, world, rank = sp.pool, sp.world, sp.rank
        qkv = qkv.contiguous()
        b, s_loc, d3 = qkv.shape
        dh = d3 // (3 * heads)
        hp, s_full = heads // world, s_loc * world
        scale = dh ** -0.5
        needs_grad = any(ctx.needs_input_grad[:3])
        # 1. QKV post-processing whose stores ARE the heads exchange
        n, slot = sp._begin("qkv")
        bufs = [sp._buffer(f"qkv{i}", slot, (b, s_full, hp, dh), qkv.dtype, qkv.device) for i in range(3)]
        rstd = ext.qkv_prepare_fwd_peers(qkv, q_weight, k_weight, cos, sin, heads, eps,
                                         pool.peer_pointers(bufs[0]), pool.peer_pointers(bufs[1]),
                                         pool.peer_pointers(bufs[2]), world, s_full, rank * s_loc)
        sp._written("qkv", slot, n)
        qh, kh, vh = (t.transpose(1, 2) for t in bufs)           # [B, H/P, S, Dh] views
        sp.kernel_launches += 1
        sp.fused_layers += 1
        if not needs_grad:
            # 2a. attention whose epilogue stores ARE the sequence exchange
            m, oslot = sp._begin("o")
            obuf = sp._buffer("o0", oslot, (b, s_loc, heads, dh), qkv.dtype, qkv.device)
            ext.flash_attn_fwd_peers(qh, kh, vh, scale, pool.peer_pointers(obuf), world, rank, heads)
            sp._read("qkv", slot, n)
            sp._written("o", oslot, m)
            sp.kernel_launches += 1
            # the consumer of this view is enqueued before the next exchange starts, and the next
            # exchange is what declares this one read (see the `_read` at its start)
            sp._pending_read = ("o", oslot, m)
            return obuf.view(b, s_loc, heads * dh)
        # 2b. with gradients: local output (the backward pass needs it), then a token-major exchange
        out_h, lse = ext.flash_attn_fwd(qh, kh, vh, scale, False, 0)       # [B, H/P, S, Dh] view, token-major
        saved_q, saved_k, saved_v = (t.clone() for t in (qh, kh, vh))     # the exchange buffers get reused
        sp._read("qkv", slot, n)
        (obuf,), m, oslot = sp._exchange_tm("o", [out_h.transpose(1, 2).reshape(b, s_full, hp * dh)], b, s_loc,
                                             hp * dh, to_heads=False)
        merged = obuf.view(b, s_loc, heads * dh).clone()
        sp._read("o", oslot, m)
        ctx.save_for_backward(qkv, q_weight, k_weight, cos, sin, rstd, saved_q, saved_k, saved_v, out_h, lse)
        ctx.sp, ctx.heads, ctx.scale = sp, heads, scale
        return merged

    @staticmethod
    def backward(ctx, grad):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        sp: SequenceParallel = ctx.sp
        qkv, q_weight, k_weight, cos, sin, rstd, qh, kh, vh, out_h, lse = ctx.saved_tensors
        heads, world = ctx.heads, sp.world
        b, s_loc, d3 = qkv.shape
        dh = d3 // (3 * heads)
        hp, s_full = heads // world, s_loc * world
        # dO: token owners -> head owners
        (dobuf,), n, slot = sp._exchange_tm("do", [grad.contiguous().view(b, s_loc, world, hp * dh)], b, s_loc,
                                             hp * dh, to_heads=True)
        do_h = dobuf.view(b, s_full, hp, dh).transpose(1, 2)
        dq, dk, dv = ext.flash_attn_bwd(do_h, qh, kh, vh, out_h, lse, ctx.scale, False)
        sp._read("do", slot, n)
        # dQ, dK, dV: head owners -> token owners (token-major [B, S, H/P, Dh] storage)
        packed = [t.transpose(1, 2).reshape(b, s_full, hp * dh) for t in (dq, dk, dv)]
        gbufs, m, gslot = sp._exchange_tm("dqkv", packed, b, s_loc, hp * dh, to_heads=False)
        gq, gk, gv = (t.view(b, s_loc, heads, dh).transpose(1, 2) for t in gbufs)
        gqkv, gqw, gkw = ext.qkv_prepare_bwd(gq, gk, gv, qkv, q_weight, k_weight, cos, sin, rstd, int(heads), 0)
        sp._read("dqkv", gslot, m)
        gqw = None if q_weight is None else gqw.to(q_weight.dtype)
        gkw = None if k_weight is None else gkw.to(k_weight.dtype)
        return gqkv, gqw, gkw, None, None, None, None, None


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
