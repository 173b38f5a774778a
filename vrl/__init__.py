"""``vrl`` — import alias for :mod:`visionrl_b200`.

``import vrl.algorithms.grpo`` returns the very same module object as
``import visionrl_b200.algorithms.grpo``; ``python -m vrl.scripts.train``
runs :mod:`visionrl_b200.scripts.train`.  The alias keeps every import path,
console entry point and YAML ``trainer.entrypoint`` string of the reference
project (``vrl/scripts/train.py``, ``pyproject.toml:44-45``) valid.
"""

from __future__ import annotations

import importlib
import importlib.abc
import importlib.util
import sys

_ALIAS = "vrl"
_TARGET = "visionrl_b200"


def _target_name(fullname: str) -> str:
    return _TARGET + fullname[len(_ALIAS):]


class _AliasLoader(importlib.abc.Loader):
    def __init__(self, target: str) -> None:
        self._target = target

    def create_module(self, spec):  # noqa: D401 - importlib protocol
        module = importlib.import_module(self._target)
        return module

    def exec_module(self, module) -> None:  # already executed under its real name
        return None

    # runpy (``python -m vrl.x``) asks the loader for code by the alias name.
    def get_code(self, fullname: str):
        spec = importlib.util.find_spec(self._target)
        if spec is None or spec.loader is None:
            raise ImportError(self._target)
        return spec.loader.get_code(self._target)

    def get_source(self, fullname: str):
        spec = importlib.util.find_spec(self._target)
        return spec.loader.get_source(self._target) if spec and spec.loader else None

    def is_package(self, fullname: str) -> bool:
        spec = importlib.util.find_spec(self._target)
        return bool(spec and spec.submodule_search_locations is not None)


class _AliasFinder(importlib.abc.MetaPathFinder):
    def find_spec(self, fullname, path=None, target=None):
        if fullname != _ALIAS and not fullname.startswith(_ALIAS + "."):
            return None
        if fullname == _ALIAS:
            return None
        real = _target_name(fullname)
        try:
            real_spec = importlib.util.find_spec(real)
        except (ImportError, ValueError):
            return None
        if real_spec is None:
            return None
        spec = importlib.util.spec_from_loader(
            fullname,
            _AliasLoader(real),
            origin=real_spec.origin,
            is_package=real_spec.submodule_search_locations is not None,
        )
        if spec is not None:
            spec.has_location = real_spec.has_location
        if spec is not None and real_spec.submodule_search_locations is not None:
            spec.submodule_search_locations = list(real_spec.submodule_search_locations)
        return spec


def _install() -> None:
    for finder in sys.meta_path:
        if isinstance(finder, _AliasFinder):
            return
    sys.meta_path.insert(0, _AliasFinder())


_install()

from visionrl_b200 import __version__  # noqa: E402,F401
