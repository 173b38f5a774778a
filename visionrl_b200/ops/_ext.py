"""Loader of the in-tree CUDA extension (``visionrl_b200/_C*.so``).

The extension is compiled ahead of time for ``sm_100a`` only (see
:func:`visionrl_b200.ops.build.build_extension`) and shipped next to the Python
sources.  :func:`load` fails loudly when a CUDA device is present and the
binary is missing, so a GPU run can never fall back to eager PyTorch silently.
"""

from __future__ import annotations

import importlib
import os
import threading

_lock = threading.Lock()
_module = None
_proxy = None
_error: Exception | None = None

# kernels launched per extension call (used for launch accounting in benchmarks)
_LAUNCHES = {
    "sde_step_fwd": 2, "sde_rollout_step": 2, "sde_step_bwd": 1, "token_loss_fwd": 1, "per_sample_mse": 2,
    "sum_squares": 2, "colsum": 1, "ulysses_scatter": 1, "ulysses_exchange_tm": 1, "p2p_broadcast_versioned": 2, "wait_flag": 1, "adamw_flat": 1, "adaln_fwd": 1, "adaln_bwd": 1, "rmsnorm_fwd": 1,
    "rmsnorm_bwd": 1, "qkv_prepare_fwd": 1, "qkv_prepare_fwd_peers": 1, "qkv_prepare_bwd": 1, "gemm_bf16": 1,
    "flash_attn_bwd": 3, "token_logprob_fwd": 1, "token_logprob_bwd": 1,
    "decode_attention": 1, "decode_qkv_rope_append": 1, "swiglu_rows": 1, "add_rmsnorm_rows": 1, "rs_sum_slice": 1, "adamw_slice_broadcast": 1, "int4_gemv": 1,
    "sample_tokens": 1, "lse_chunk_update": 1, "softmax_grad_chunk": 1, "group_advantages": 1,
    "flag_signal": 1, "flag_wait": 1, "flag_barrier": 1, "bucket_reduce_acc": 1, "p2p_gather_rows": 1, "p2p_gather_table": 1, "p2p_broadcast_table": 1,
    "head_logprob_fwd": 2, "head_softmax_grad": 1, "gemm_bf16_out": 1, "groupnorm_nhwc": 2, "gemm_bf16_acc": 1, "gemm_allgather": 1, "int4_gemm": 2, "gemm_bf16_dual": 1, "gate_residual_fwd": 1, "gate_residual_bwd": 1, "flash_attn_fwd": 1, "flash_attn_fwd_peers": 1, "moe_gate_topk": 1, "moe_permute": 1, "moe_gather_rows": 1, "moe_combine": 1, "moe_combine_bwd": 2, "moe_segment_colsum": 1, "lora_apply_rows": 2, "gemm_grouped": 1, "gemm_grouped_wgrad": 1,
}
launch_count = 0
_kernels_enabled = os.environ.get("VRL_FORCE_TORCH_OPS", "0") != "1"


def kernels_enabled() -> bool:
    """False while the PyTorch-library baseline mode is active (benchmark comparison arm)."""
    return _kernels_enabled


def set_kernels_enabled(flag: bool) -> None:
    global _kernels_enabled
    _kernels_enabled = bool(flag)


class _CountingProxy:
    """Forwards attribute access to the extension and counts kernel launches per call."""

    def __init__(self, module):
        self._module = module
        self._wrapped: dict = {}

    def __getattr__(self, name):
        fn = self._wrapped.get(name)
        if fn is None:
            raw = getattr(self._module, name)
            n = _LAUNCHES.get(name, 0)
            if n == 0 or not callable(raw):
                return raw

            def fn(*args, _raw=raw, _n=n, **kwargs):
                global launch_count
                launch_count += _n
                return _raw(*args, **kwargs)

            self._wrapped[name] = fn
        return fn

    def __dir__(self):
        return dir(self._module)


class ExtensionUnavailable(RuntimeError):
    pass


def load():
    """Import ``visionrl_b200._C`` once; raise :class:`ExtensionUnavailable` otherwise."""
    global _module, _error, _proxy
    if _proxy is not None:
        return _proxy
    with _lock:
        if _proxy is not None:
            return _proxy
        try:
            import torch  # noqa: F401  (libtorch must be loaded before the extension)

            _module = importlib.import_module("visionrl_b200._C")
        except Exception as exc:  # pragma: no cover - depends on the build
            _error = exc
            raise ExtensionUnavailable(
                "visionrl_b200._C is not built; run `python -c \"import __graft_entry__ as g; "
                "g.build()\"` (or `python -m visionrl_b200.ops.build`) first"
            ) from exc
        _proxy = _CountingProxy(_module)
    return _proxy


def has(name: str) -> bool:
    """True when the built extension exports ``name``."""
    try:
        return hasattr(load()._module, name)
    except ExtensionUnavailable:
        return False


def available() -> bool:
    try:
        load()
        return True
    except ExtensionUnavailable:
        return False
