"""Unified training entry point: ``python -m vrl.scripts.train --config experiment/<name> [k=v ...]``.

Loads one YAML (with overrides), imports ``trainer.entrypoint`` (``"module:function"``) and
runs it, awaiting the result when it is a coroutine.  Nothing here knows about model
families or algorithm kinds (reference: ``vrl/scripts/train.py:28-85``).
"""

from __future__ import annotations

import argparse
import asyncio
import importlib
import inspect
import logging
from dataclasses import dataclass
from typing import Any

from visionrl_b200.config.cli import LOG_FORMAT


@dataclass(frozen=True, slots=True)
class TrainTarget:
    import_path: str


def resolve_train_target(cfg: Any) -> TrainTarget:
    try:
        path = cfg.trainer.entrypoint
    except Exception as exc:  # noqa: BLE001
        raise ValueError("config missing required field: trainer.entrypoint") from exc
    if not isinstance(path, str) or not path.strip():
        raise ValueError("trainer.entrypoint must be a non-empty import path")
    return TrainTarget(path.strip())


def _import_callable(import_path: str) -> Any:
    if ":" not in import_path:
        raise ValueError("trainer.entrypoint must use 'module:function' import path syntax")
    module_name, attr = import_path.split(":", 1)
    return getattr(importlib.import_module(module_name), attr)


def run_config(cfg: Any) -> Any:
    return _import_callable(resolve_train_target(cfg).import_path)(cfg)


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description="Run a YAML-driven training job.")
    parser.add_argument("--config", required=True,
                        help="YAML config name under configs/ or a filesystem path")
    parser.add_argument("overrides", nargs="*",
                        help="dotlist overrides, e.g. trainer.seed=42 actor.optim.lr=2e-4")
    return parser


def main(argv: list[str] | None = None) -> None:
    from visionrl_b200.config.loader import load_config

    logging.basicConfig(level=logging.INFO, format=LOG_FORMAT)
    args = build_parser().parse_args(argv)
    result = run_config(load_config(args.config, overrides=args.overrides))
    if inspect.isawaitable(result):
        asyncio.run(result)


if __name__ == "__main__":
    main()
