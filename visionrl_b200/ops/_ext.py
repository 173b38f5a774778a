"""Loader of the in-tree CUDA extension (``visionrl_b200/_C*.so``).

The extension is compiled ahead of time for ``sm_100a`` only (see
:func:`visionrl_b200.ops.build.build_extension`) and shipped next to the Python
sources.  :func:`load` fails loudly when a CUDA device is present and the
binary is missing, so a GPU run can never fall back to eager PyTorch silently.
"""

from __future__ import annotations

import importlib
import threading

_lock = threading.Lock()
_module = None
_error: Exception | None = None


class ExtensionUnavailable(RuntimeError):
    pass


def load():
    """Import ``visionrl_b200._C`` once; raise :class:`ExtensionUnavailable` otherwise."""
    global _module, _error
    if _module is not None:
        return _module
    with _lock:
        if _module is not None:
            return _module
        try:
            import torch  # noqa: F401  (libtorch must be loaded before the extension)

            _module = importlib.import_module("visionrl_b200._C")
        except Exception as exc:  # pragma: no cover - depends on the build
            _error = exc
            raise ExtensionUnavailable(
                "visionrl_b200._C is not built; run `python -c \"import __graft_entry__ as g; "
                "g.build()\"` (or `python -m visionrl_b200.ops.build`) first"
            ) from exc
    return _module


def available() -> bool:
    try:
        load()
        return True
    except ExtensionUnavailable:
        return False
