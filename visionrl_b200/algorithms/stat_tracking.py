"""Per-prompt reward statistics (float64 on the host).

``update`` buckets a batch's rewards by prompt string, extends each prompt's
history and returns advantages of the requested kind: ``grpo`` is
``(r - mean) / (std + 1e-4)`` with the population std of the prompt's history,
``rwr`` the raw reward, ``sft`` a one-hot on the bucket maximum and ``dpo`` ±1 on
the bucket max/min.  ``clear`` drops histories but remembers which prompts were
ever seen (reference: ``vrl/algorithms/stat_tracking.py:21-118``).
"""

from __future__ import annotations

from typing import Any

import numpy as np

_KINDS = ("grpo", "rwr", "sft", "dpo")


class PerPromptStatTracker:
    def __init__(self, global_std: bool = False) -> None:
        self.global_std = global_std
        self.stats: dict[str, Any] = {}
        self.history_prompts: set[int] = set()

    def update(self, prompts, rewards, type: str = "grpo") -> np.ndarray:  # noqa: A002
        if type not in _KINDS:
            raise ValueError(f"Unknown advantage type: {type}")
        if hasattr(rewards, "detach"):
            rewards = rewards.detach().cpu().numpy()
        rewards = np.asarray(rewards, dtype=np.float64)
        prompts = np.asarray(prompts)
        names, inverse = np.unique(prompts, return_inverse=True)
        rows = [np.flatnonzero(inverse == g) for g in range(len(names))]

        for name, idx in zip(names, rows):
            history = list(self.stats.get(name, []))
            history.extend(rewards[idx])
            self.stats[name] = np.stack(history)
            self.history_prompts.add(hash(name))

        advantages = np.zeros_like(rewards)
        global_std = np.std(rewards, axis=0, keepdims=True) + 1e-4
        for name, idx in zip(names, rows):
            bucket = rewards[idx]
            history = self.stats[name]
            if type == "grpo":
                mean = np.mean(history, axis=0, keepdims=True)
                std = global_std if self.global_std else np.std(history, axis=0, keepdims=True) + 1e-4
                advantages[idx] = (bucket - mean) / std
            elif type == "rwr":
                advantages[idx] = bucket
            elif type == "sft":
                advantages[idx] = (bucket == bucket.max()).astype(np.float64)
            else:
                hi, lo = int(np.argmax(bucket)), int(np.argmin(bucket))
                if hi == lo:
                    lo, hi = 0, 1
                signs = np.zeros_like(bucket)
                signs[hi], signs[lo] = 1.0, -1.0
                advantages[idx] = signs
        return advantages

    def get_stats(self) -> tuple[float, int]:
        if not self.stats:
            return 0.0, 0
        sizes = [len(v) for v in self.stats.values()]
        return sum(sizes) / len(sizes), len(self.history_prompts)

    def clear(self) -> None:
        self.stats = {}
