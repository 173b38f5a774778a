"""Training entry point of a one-process-per-GPU job.

    python -m vrl.scripts.train --config experiment/<name> [key=value ...]
    torchrun --nproc-per-node 8 -m vrl.scripts.train --config experiment/<name> [key=value ...]

The same command line serves a single process and every rank of a ``torchrun`` launch: the
launcher's ``RANK`` / ``WORLD_SIZE`` decide which.  What this layer adds around the recipe named
by the config is the part that is the same for every rank and every model family:

* log lines carry the rank, and only rank 0 logs at INFO (the others from WARNING up), so an
  eight-rank job reads like one;
* the YAML (plus ``key=value`` overrides) is loaded once per rank, the recipe is looked up from
  ``trainer.entrypoint`` (``"package.module:function"``) and called with the config; a coroutine
  is driven to completion on a fresh event loop;
* whatever happens, the rank leaves its process group on the way out, so a failed rank does not
  keep its peers' collectives waiting on a half-open communicator, and the exit status is
  non-zero for the launcher to see.

No model family and no algorithm kind is named here: both belong to the config and the recipe
(the reference keeps its CLI equally blind, ``vrl/scripts/train.py:28-85``).
"""

from __future__ import annotations

import argparse
import asyncio
import importlib
import inspect
import logging
import os
import sys
from dataclasses import dataclass
from typing import Any, Callable

from visionrl_b200.config.cli import LOG_FORMAT

_SYNTAX = "trainer.entrypoint must use 'module:function' import path syntax"


@dataclass(frozen=True, slots=True)
class TrainTarget:
    """Where the recipe lives: ``import_path`` is ``"package.module:function"``."""

    import_path: str

    @property
    def module(self) -> str:
        return self.import_path.partition(":")[0]

    @property
    def function(self) -> str:
        return self.import_path.partition(":")[2]

    def load(self) -> Callable[[Any], Any]:
        if ":" not in self.import_path or not self.module or not self.function:
            raise ValueError(_SYNTAX)
        recipe = getattr(importlib.import_module(self.module), self.function, None)
        if not callable(recipe):
            raise ValueError(f"{self.import_path} does not name a callable")
        return recipe


def resolve_train_target(cfg: Any) -> TrainTarget:
    trainer = cfg.get("trainer") if hasattr(cfg, "get") else getattr(cfg, "trainer", None)
    path = None if trainer is None else (trainer.get("entrypoint") if hasattr(trainer, "get")
                                         else getattr(trainer, "entrypoint", None))
    if path is None:
        raise ValueError("config missing required field: trainer.entrypoint")
    if not isinstance(path, str) or not path.strip():
        raise ValueError("trainer.entrypoint must be a non-empty import path")
    return TrainTarget(path.strip())


def _import_callable(import_path: str) -> Callable[[Any], Any]:
    return TrainTarget(import_path).load()


def run_config(cfg: Any) -> Any:
    """Call the recipe the config names; the caller drives the result if it is awaitable."""
    return resolve_train_target(cfg).load()(cfg)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        prog="vrl-train", description="Run the training recipe named by a YAML config "
                                      "(alone, or as every rank of a torchrun launch).")
    parser.add_argument("--config", required=True,
                        help="config name below configs/ (e.g. experiment/<name>) or a filesystem path")
    parser.add_argument("overrides", nargs="*", metavar="key=value",
                        help="dotted overrides applied after the file, e.g. actor.optim.lr=2e-4")
    return parser


def _launcher_rank() -> tuple[int, int]:
    try:
        return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    except ValueError:
        return 0, 1


def _configure_logging(rank: int, world: int) -> None:
    fmt = LOG_FORMAT if world <= 1 else LOG_FORMAT.replace("%(name)s", f"[rank {rank}] %(name)s")
    logging.basicConfig(level=logging.INFO if rank == 0 else logging.WARNING, format=fmt)


def _leave_process_group() -> None:
    try:
        import torch.distributed as dist

        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001 - leaving must not mask the error that brought us here
        logging.getLogger(__name__).debug("process group teardown failed", exc_info=True)


def main(argv: list[str] | None = None) -> int:
    from visionrl_b200.config.loader import load_config

    rank, world = _launcher_rank()
    _configure_logging(rank, world)
    args = build_parser().parse_args(argv)
    try:
        outcome = run_config(load_config(args.config, overrides=args.overrides))
        if inspect.isawaitable(outcome):
            asyncio.run(outcome)
    finally:
        _leave_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
