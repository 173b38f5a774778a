"""What every trainer of this package has in common.

`Trainer` is the asynchronous step contract of the online trainers (reference:
``vrl/trainers/base.py``).  `raise_on_kernel_timeout` is the check every trainer runs after a
step on a GPU: the package's kernels never spin without limit, a wait that gives up writes a code
into a status word and the kernel returns, so the host has to look at those words or a step with
invalid results would pass silently.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from typing import Any

import torch

from visionrl_b200.algorithms.types import TrainStepMetrics

KERNEL_STATUS_WORDS = (
    "bf16 GEMM (1 = TMA producer, 2 = MMA issuer, 3 = epilogue)",
    "attention (flash forward / backward; 31 = decode attention's copy ring)",
    "int4 GEMM",
)


def describe_kernel_status(words) -> list[str]:
    """One line per non-zero status word, in the order the extension reports them."""
    return [f"{name}: status {int(word)}" for name, word in zip(KERNEL_STATUS_WORDS, words) if int(word) != 0]


def raise_on_kernel_timeout(device: torch.device | str, grad_sync: Any = None, where: str = "training step") -> int:
    """Read the kernels' status words (one 16-byte copy) and, when `grad_sync` has one, the
    collective runtime's; raise if a bounded wait gave up.  Returns the bytes read from the device
    so callers can keep their device-to-host accounting exact.  A CPU device reads nothing."""
    if torch.device(device).type != "cuda":
        return 0
    from visionrl_b200.ops import _ext

    if not (_ext.kernels_enabled() and _ext.available()):
        return 0
    read = 16
    bad = describe_kernel_status(_ext.load().kernel_status_all())
    if bad:
        raise RuntimeError("a kernel gave up waiting on one of its barriers; this step's "
                           "results are invalid (" + "; ".join(bad) + ")")
    check = getattr(grad_sync, "check", None)
    if callable(check):
        check(where)
        read += 16
    return read


class Trainer(ABC):
    """One call of `step` is a whole iteration: collect, reward, advantages, update."""

    @abstractmethod
    async def step(self) -> TrainStepMetrics: ...

    @abstractmethod
    def state_dict(self) -> dict: ...

    @abstractmethod
    def load_state_dict(self, state: dict, *, strict: bool = True) -> None: ...
