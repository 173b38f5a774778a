"""Command-line front end shared by the per-family scripts: ``--config`` (with the script's own
default experiment) plus trailing ``key=value`` overrides, resolved into a loaded config.

Logging is set up the way the training entry point does it, so a script started as one rank of a
multi-process launch tags its lines with the rank and keeps the non-zero ranks quiet.  The
reference's helper has the same two arguments (``vrl/config/cli.py:11-32``).
"""

from __future__ import annotations

import argparse
import logging
import os

LOG_FORMAT = "%(asctime)s %(name)s %(levelname)s %(message)s"


def build_parser(default_config: str, description: str) -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(description=description)
    parser.add_argument("--config", default=default_config,
                        help="experiment name below configs/ or a filesystem path")
    parser.add_argument("overrides", nargs="*", metavar="key=value",
                        help="dotted overrides applied after the file, e.g. trainer.seed=42")
    return parser


def configure_logging() -> None:
    rank, world = os.environ.get("RANK", "0"), os.environ.get("WORLD_SIZE", "1")
    many = world.isdigit() and int(world) > 1
    fmt = LOG_FORMAT.replace("%(name)s", f"[rank {rank}] %(name)s") if many else LOG_FORMAT
    logging.basicConfig(level=logging.INFO if rank in ("0", "") else logging.WARNING, format=fmt)


def parse_and_load(default_config: str, description: str, argv: list[str] | None = None):
    from visionrl_b200.config.loader import load_config

    configure_logging()
    args = build_parser(default_config, description).parse_args(argv)
    return load_config(args.config, overrides=args.overrides)
