"""Linear layer on the tcgen05 GEMM (kernel K1) with fused epilogues.

``y = epilogue(x @ w.T + bias)`` where ``w`` is ``[N, K]`` (``nn.Linear`` layout).
Epilogues: ``act`` ∈ {None, "gelu_tanh", "silu"} and the adaLN gate-residual
``y = residual + gate[b] * y`` with a per-sample ``gate[B, N]``.  bf16 CUDA inputs
run the hand-written sm_100a kernel (TMA → shared memory → ``tcgen05.mma`` with
the accumulator in tensor memory → epilogue from ``tcgen05.ld``); anything else
(CPU, fp32) takes the PyTorch oracle below.  The backward pass forms ``dX`` and
``dW`` with the same kernel through its transposed-operand variants.
"""

from __future__ import annotations

import contextlib

import torch
import torch.nn.functional as F

_ACTS = {None: 0, "none": 0, "gelu_tanh": 1, "silu": 2}


def linear_reference(x, w, bias=None, act=None, gate=None, residual=None):
    y = F.linear(x, w, bias)
    if act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif act == "silu":
        y = F.silu(y)
    if gate is not None:
        y = residual + gate.unsqueeze(1) * y if y.dim() == 3 else residual + gate * y
    return y


def linear_epilogue(y, act=None, gate=None, residual=None):
    """The epilogue alone, for callers that add a side product before it."""
    if act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif act == "silu":
        y = F.silu(y)
    if gate is not None:
        y = gate_residual(y, gate, residual)
    return y


def _use_kernel(x, w) -> bool:
    from visionrl_b200.ops import _ext

    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and x.shape[-1] % 8 == 0 and w.shape[0] % 8 == 0 and _ext.kernels_enabled())


def gemm_nt(a, b, bias=None, act=None, gate=None, residual=None, rows_per_gate: int = 0,
            out_dtype=None):
    """``a[M,K] @ b[N,K].T`` on the sm_100a kernel (no autograd)."""
    from visionrl_b200.ops import _ext

    return _ext.load().gemm_bf16(
        a, b, bias, gate, residual, _ACTS[act], int(rows_per_gate), False, False,
        out_dtype == torch.float32,
    )


def gemm_nn(a, b):
    """``a[M,K] @ b[K,N]`` (``b`` row-major, i.e. MN-major operand)."""
    from visionrl_b200.ops import _ext

    return _ext.load().gemm_bf16(a, b, None, None, None, 0, 0, False, True, False)


def gemm_tn(a, b, out_fp32: bool = False):
    """``a[K,M].T @ b[K,N]`` — both operands MN-major (weight gradients)."""
    from visionrl_b200.ops import _ext

    return _ext.load().gemm_bf16(a, b, None, None, None, 0, 0, True, True, out_fp32)


# While the trainer's backward pass runs, weight gradients are added straight into the parameters'
# existing ``.grad`` buffers by the GEMM epilogue (no temporary, no separate accumulation kernel).
# Functional uses of autograd (``torch.autograd.grad``) never enable this.
_ACCUMULATE_IN_PLACE = [False]


@contextlib.contextmanager
def accumulate_weight_grads_in_place(enabled: bool = True):
    previous = _ACCUMULATE_IN_PLACE[0]
    _ACCUMULATE_IN_PLACE[0] = bool(enabled)
    try:
        yield
    finally:
        _ACCUMULATE_IN_PLACE[0] = previous


def _weight_grad(gy2, x2, param):
    """``gy2.T @ x2`` — returned, or added into ``param.grad`` in place (then ``None``)."""
    from visionrl_b200.ops import _ext

    grad = param.grad if (_ACCUMULATE_IN_PLACE[0] and param is not None and param.is_leaf) else None
    if (grad is not None and grad.dtype == torch.bfloat16
            and grad.is_contiguous() and grad.shape == (gy2.shape[1], x2.shape[1])
            and grad.data_ptr() % 16 == 0 and _ext.has("gemm_bf16_acc")):
        _ext.load().gemm_bf16_acc(gy2, x2, grad, True, True)
        return None
    return gemm_tn(gy2, x2)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, bias):
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        y = gemm_nt(x2, w, bias)
        ctx.save_for_backward(x2, w)
        ctx.weight_param = w            # the parameter object itself (its .grad buffer is the target)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = gemm_nn(gy2, w).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw = _weight_grad(gy2, x2, ctx.weight_param)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from visionrl_b200.ops import _ext

            gb = _ext.load().colsum(gy2).to(gy2.dtype)
        return gx, gw, gb


class _GateResidualFn(torch.autograd.Function):
    """``residual + gate[:, None, :] * y`` for ``[B, S, D]`` activations and a ``[B, D]`` gate."""

    @staticmethod
    def forward(ctx, y, gate, residual):
        from visionrl_b200.ops import _ext

        y = y.contiguous()
        out = _ext.load().gate_residual_fwd(y, gate, residual.contiguous())
        ctx.save_for_backward(y, gate)
        return out

    @staticmethod
    def backward(ctx, g):
        from visionrl_b200.ops import _ext

        y, gate = ctx.saved_tensors
        gy, ggate = _ext.load().gate_residual_bwd(g, y, gate)
        return gy, ggate.to(gate.dtype), g


def gate_residual(y, gate, residual):
    """Differentiable adaLN-Zero gate: one fused kernel each way on bf16 CUDA tensors."""
    from visionrl_b200.ops import _ext

    if (y.is_cuda and y.dim() == 3 and gate.dim() == 2 and y.dtype == torch.bfloat16
            and gate.dtype == torch.bfloat16 and residual.dtype == torch.bfloat16
            and y.shape[-1] % 8 == 0 and y.shape[-1] <= 2048 and _ext.kernels_enabled()
            and _ext.has("gate_residual_fwd")):
        return _GateResidualFn.apply(y, gate, residual)
    return residual + (gate.unsqueeze(1) if y.dim() == 3 else gate) * y


class _GeluMLPFn(torch.autograd.Function):
    """``fc2(gelu_tanh(fc1(x)))`` with the activation folded into the GEMM epilogues.

    Forward: the first GEMM stores both the pre-activation ``h`` and ``gelu(h)`` from one pass
    over the accumulator.  Backward: the GEMM that forms ``d gelu(h)`` multiplies by
    ``gelu'(h)`` in its epilogue, so no stand-alone activation kernel runs in either direction.
    """

    @staticmethod
    def forward(ctx, x, w1, b1, w2, b2):
        from visionrl_b200.ops import _ext

        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        a, h = _ext.load().gemm_bf16_dual(x2, w1, b1, _ACTS["gelu_tanh"])
        y = gemm_nt(a, w2, b2)
        ctx.save_for_backward(x2, w1, w2, h, a)
        ctx.w1_param, ctx.w2_param = w1, w2
        ctx.has_b1, ctx.has_b2 = b1 is not None, b2 is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, gy):
        from visionrl_b200.ops import _ext

        ext = _ext.load()
        x2, w1, w2, h, a = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        # gh = (gy @ w2) * gelu'(h): w2 is [out, hidden] row-major, i.e. the MN-major B operand
        gh = ext.gemm_bf16(gy2, w2, None, None, h, 3, 0, False, True, False)
        gx = gw1 = gb1 = gw2 = gb2 = None
        if ctx.needs_input_grad[3]:
            gw2 = _weight_grad(gy2, a, ctx.w2_param)
        if ctx.has_b2 and ctx.needs_input_grad[4]:
            gb2 = ext.colsum(gy2).to(gy2.dtype)
        if ctx.needs_input_grad[1]:
            gw1 = _weight_grad(gh, x2, ctx.w1_param)
        if ctx.has_b1 and ctx.needs_input_grad[2]:
            gb1 = ext.colsum(gh).to(gh.dtype)
        if ctx.needs_input_grad[0]:
            gx = gemm_nn(gh, w1).view(ctx.x_shape)
        return gx, gw1, gb1, gw2, gb2


def gelu_mlp(x, w1, b1, w2, b2):
    """Two-layer GELU-tanh MLP; fused epilogues when gradients are needed on bf16 CUDA tensors."""
    from visionrl_b200.ops import _ext

    needs_grad = torch.is_grad_enabled() and any(
        t is not None and t.requires_grad for t in (x, w1, b1, w2, b2))
    if (needs_grad and _use_kernel(x, w1) and w2.dtype == torch.bfloat16 and w1.shape[0] % 8 == 0
            and w2.shape[0] % 8 == 0 and _ext.has("gemm_bf16_dual")):
        return _GeluMLPFn.apply(x, w1, b1, w2, b2)
    return linear(linear(x, w1, b1, act="gelu_tanh"), w2, b2)


def linear(x, w, bias=None, act=None, gate=None, residual=None):
    """Differentiable linear with optional fused epilogue (fused only without grad)."""
    if not _use_kernel(x, w):
        return linear_reference(x, w, bias, act, gate, residual)
    needs_grad = torch.is_grad_enabled() and (
        x.requires_grad or w.requires_grad or (bias is not None and bias.requires_grad)
        or (gate is not None and gate.requires_grad)
        or (residual is not None and residual.requires_grad)
    )
    if not needs_grad:
        x2 = x.reshape(-1, x.shape[-1])
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x.shape[-2] if (gate is not None and x.dim() == 3) else (1 if gate is not None else 0)
        if gate is not None and gate.dim() != 2:
            gate = gate.reshape(-1, w.shape[0])
        res2 = None if residual is None else residual.reshape(-1, w.shape[0])
        y = gemm_nt(x2, w, bias, act, gate, res2, rows)
        return y.view(*x.shape[:-1], w.shape[0])
    y = _LinearFn.apply(x, w, bias)
    if act == "gelu_tanh":
        y = F.gelu(y, approximate="tanh")
    elif act == "silu":
        y = F.silu(y)
    if gate is not None:
        y = gate_residual(y, gate, residual)
    return y
