"""Trainer interface (reference: ``vrl/trainers/base.py``)."""

from __future__ import annotations

from abc import ABC, abstractmethod

from visionrl_b200.algorithms.types import TrainStepMetrics


class Trainer(ABC):
    @abstractmethod
    async def step(self) -> TrainStepMetrics:
        """collect → reward → advantage → update."""

    @abstractmethod
    def state_dict(self) -> dict:
        """Serialisable trainer state."""

    @abstractmethod
    def load_state_dict(self, state: dict, *, strict: bool = True) -> None:
        """Restore from :meth:`state_dict`."""
