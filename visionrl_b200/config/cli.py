"""Argparse helper shared by scripts that want a default experiment
(reference: ``vrl/config/cli.py:11-32``)."""

from __future__ import annotations

import argparse
import logging

LOG_FORMAT = "%(asctime)s %(name)s %(levelname)s %(message)s"


def parse_and_load(default_config: str, description: str, argv: list[str] | None = None):
    from visionrl_b200.config.loader import load_config

    logging.basicConfig(level=logging.INFO, format=LOG_FORMAT)
    parser = argparse.ArgumentParser(description=description)
    parser.add_argument("--config", default=default_config,
                        help="experiment name below configs/ or a filesystem path")
    parser.add_argument("overrides", nargs="*", help="dotlist overrides, e.g. trainer.seed=42")
    args = parser.parse_args(argv)
    return load_config(args.config, overrides=args.overrides)
