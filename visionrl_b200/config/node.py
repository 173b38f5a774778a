"""Minimal attribute-access config tree on top of PyYAML.

The reference loads its YAML through OmegaConf (``vrl/config/loader.py:28``).
That package is not a dependency here: :class:`DictConfig` is a ``dict``
subclass with attribute access, recursive merge, dotlist overrides with
YAML-typed values and ``${a.b.c}`` interpolation — the subset of OmegaConf the
recipes and tests rely on.  Lists are :class:`ListConfig` (a ``list`` subclass)
so ``isinstance`` checks on either container keep working.
"""

from __future__ import annotations

import copy
import re
from pathlib import Path
from typing import Any, Iterable, Mapping

import yaml

_INTERP = re.compile(r"\$\{([^}]+)\}")


class ListConfig(list):
    """YAML sequence node."""


class DictConfig(dict):
    """YAML mapping node with ``cfg.a.b`` access."""

    def __getattr__(self, key: str) -> Any:
        if key.startswith("__") and key.endswith("__"):
            raise AttributeError(key)
        try:
            return self[key]
        except KeyError as exc:
            raise AttributeError(f"Missing key {key}") from exc

    def __setattr__(self, key: str, value: Any) -> None:
        self[key] = wrap(value)

    def __delattr__(self, key: str) -> None:
        try:
            del self[key]
        except KeyError as exc:
            raise AttributeError(key) from exc

    def __setitem__(self, key: str, value: Any) -> None:
        super().__setitem__(key, wrap(value))

    def copy(self) -> "DictConfig":  # type: ignore[override]
        return copy.deepcopy(self)


def wrap(value: Any) -> Any:
    """Convert plain containers into config nodes (recursively)."""
    if isinstance(value, (DictConfig, ListConfig)):
        return value
    if isinstance(value, Mapping):
        node = DictConfig()
        for k, v in value.items():
            dict.__setitem__(node, str(k), wrap(v))
        return node
    if isinstance(value, (list, tuple)):
        return ListConfig(wrap(v) for v in value)
    return value


def to_container(value: Any, resolve: bool = True) -> Any:
    """Convert config nodes back into plain ``dict`` / ``list`` objects."""
    if isinstance(value, Mapping):
        return {k: to_container(v, resolve) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return [to_container(v, resolve) for v in value]
    return value


def merge(base: Any, *others: Any) -> Any:
    """Recursive merge; mappings merge key-wise, everything else is replaced."""
    out = wrap(copy.deepcopy(base))
    for other in others:
        out = _merge_two(out, wrap(other))
    return out


def _merge_two(a: Any, b: Any) -> Any:
    if isinstance(a, DictConfig) and isinstance(b, DictConfig):
        for k, v in b.items():
            if k in a and isinstance(a[k], DictConfig) and isinstance(v, DictConfig):
                dict.__setitem__(a, k, _merge_two(a[k], v))
            else:
                dict.__setitem__(a, k, copy.deepcopy(v))
        return a
    return copy.deepcopy(b)


class _Loader(yaml.SafeLoader):
    """SafeLoader that also reads ``1e-4`` (no dot) as a float, like YAML 1.2."""


_Loader.add_implicit_resolver(
    "tag:yaml.org,2002:float",
    re.compile(
        r"""^(?:[-+]?(?:[0-9][0-9_]*)\.[0-9_]*(?:[eE][-+]?[0-9]+)?
        |[-+]?(?:[0-9][0-9_]*)(?:[eE][-+]?[0-9]+)
        |\.[0-9_]+(?:[eE][-+]?[0-9]+)?
        |[-+]?\.(?:inf|Inf|INF)
        |\.(?:nan|NaN|NAN))$""",
        re.X,
    ),
    list("-+0123456789."),
)


def parse_yaml_text(text: str) -> Any:
    return yaml.load(text, Loader=_Loader)


def load_yaml(path: str | Path) -> Any:
    with open(path, "r", encoding="utf-8") as fh:
        data = yaml.load(fh, Loader=_Loader)
    return wrap({} if data is None else data)


def create(value: Any = None) -> Any:
    if value is None:
        return DictConfig()
    if isinstance(value, str):
        return wrap(parse_yaml_text(value) or {})
    return wrap(copy.deepcopy(value))


def from_dotlist(items: Iterable[str]) -> DictConfig:
    """``["a.b=1", "c=[1,2]"]`` → nested config with YAML-typed values."""
    root = DictConfig()
    for item in items:
        if "=" not in item:
            key, raw = item, None
        else:
            key, raw = item.split("=", 1)
        key = key.strip().lstrip("+")
        if not key:
            raise ValueError(f"bad override (empty key): {item!r}")
        value = None if raw is None else parse_yaml_text(raw) if raw.strip() != "" else ""
        node = root
        parts = key.split(".")
        for part in parts[:-1]:
            if part not in node or not isinstance(node[part], DictConfig):
                dict.__setitem__(node, part, DictConfig())
            node = node[part]
        node[parts[-1]] = value
    return root


def select(cfg: Any, path: str, default: Any = None) -> Any:
    node = cfg
    for key in path.split("."):
        if isinstance(node, Mapping) and key in node:
            node = node[key]
        elif isinstance(node, list) and key.lstrip("-").isdigit() and int(key) < len(node):
            node = node[int(key)]
        else:
            return default
    return node


def resolve(cfg: Any) -> Any:
    """Resolve ``${dotted.path}`` interpolations in place."""

    def _lookup(path: str, stack: tuple[str, ...]) -> Any:
        if path in stack:
            raise ValueError(f"interpolation cycle: {' -> '.join(stack + (path,))}")
        sentinel = object()
        value = select(cfg, path, sentinel)
        if value is sentinel:
            raise KeyError(f"interpolation key not found: {path}")
        return _resolve_value(value, stack + (path,))

    def _resolve_value(value: Any, stack: tuple[str, ...]) -> Any:
        if isinstance(value, str):
            whole = _INTERP.fullmatch(value)
            if whole:
                return _lookup(whole.group(1).strip(), stack)
            if _INTERP.search(value):
                return _INTERP.sub(lambda m: str(_lookup(m.group(1).strip(), stack)), value)
            return value
        if isinstance(value, DictConfig):
            for k in list(value.keys()):
                dict.__setitem__(value, k, _resolve_value(value[k], stack))
            return value
        if isinstance(value, ListConfig):
            for i in range(len(value)):
                value[i] = _resolve_value(value[i], stack)
            return value
        return value

    return _resolve_value(cfg, ())


def to_yaml(cfg: Any) -> str:
    return yaml.safe_dump(to_container(cfg), sort_keys=False, default_flow_style=False)


def save_yaml(cfg: Any, path: str | Path) -> None:
    Path(path).parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w", encoding="utf-8") as fh:
        fh.write(to_yaml(cfg))


class OmegaConf:
    """Name-compatible facade for the handful of OmegaConf calls recipes use."""

    create = staticmethod(create)
    merge = staticmethod(merge)
    load = staticmethod(load_yaml)
    to_container = staticmethod(to_container)
    from_dotlist = staticmethod(from_dotlist)
    resolve = staticmethod(resolve)
    select = staticmethod(select)
    to_yaml = staticmethod(to_yaml)
    save = staticmethod(save_yaml)


__all__ = [
    "DictConfig",
    "ListConfig",
    "OmegaConf",
    "create",
    "from_dotlist",
    "load_yaml",
    "merge",
    "resolve",
    "save_yaml",
    "select",
    "to_container",
    "to_yaml",
    "wrap",
]
