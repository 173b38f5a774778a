"""``"package.module:attr"`` import helper."""

from __future__ import annotations

import importlib
from typing import Any


def import_from_path(path: str) -> Any:
    if ":" not in path:
        raise ValueError(f"import path must look like 'module:attr', got {path!r}")
    module, attr = path.split(":", 1)
    return getattr(importlib.import_module(module), attr)
