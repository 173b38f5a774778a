"""YAML experiment loader with a ``defaults:`` overlay and fail-fast validation.

Behavioural contract (reference: ``vrl/config/loader.py:36-126,151-189,210-271,
377-444,447-580``):

* a YAML file may carry a top-level ``defaults:`` list; every entry names
  another YAML below the configs root (leading ``/`` optional, ``.yaml``
  appended, ``{group: option}`` read as ``group/option``); entries merge in
  list order and the file's own body goes last unless ``_self_`` moves it;
* overrides use dotlist syntax (``trainer.seed=42``) with YAML-typed values;
* ``require`` / ``optional_none`` raise ``ValueError`` naming the dotted path;
* ``algorithm.kind`` ∈ {``grpo``, ``token_grpo``, ``diffusion_dpo``} is the only
  algorithm dispatch key.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

from visionrl_b200.config.node import (
    DictConfig,
    ListConfig,
    OmegaConf,
    from_dotlist,
    load_yaml,
    merge,
    resolve,
    to_container,
)

CONFIGS_ROOT = Path(__file__).resolve().parents[2] / "configs"

_SELF = "_self_"
_YAML_SUFFIXES = (".yaml", ".yml")

_GRPO_FIELDS = frozenset(
    {"eps_clip", "init_kl_coef", "eps", "adv_clip_max", "global_std", "flow_kl_use_dt"}
)
_TOKEN_GRPO_EXTRA_FIELDS = frozenset({"mask_key", "kl_estimator"})
_DPO_FIELDS = frozenset({"beta", "sft_weight"})
_KINDS = ("grpo", "token_grpo", "diffusion_dpo")

# reward name -> kwargs that must be spelled out when its weight is positive
_REWARD_REQUIRED_KWARGS: dict[str, tuple[str, ...]] = {
    "aesthetic": ("model_name",),
    "clipscore": ("model_name",),
    "pickscore": ("processor_name", "model_name"),
    "ocr": ("debug_dir",),  # may be "", but the key has to be written
}

_COMMON_REQUIRED_FIELDS: tuple[str, ...] = tuple(
    [f"actor.optim.{k}" for k in
     ("lr", "adam_beta1", "adam_beta2", "weight_decay", "eps", "use_8bit_adam", "allow_tf32")]
    + [f"actor.{k}" for k in
       ("max_norm", "ppo_epochs", "bf16", "gradient_checkpointing", "timestep_fraction")]
    + [f"actor.ema.{k}" for k in ("enable", "decay", "update_interval")]
    + [f"trainer.{k}" for k in
       ("entrypoint", "total_epochs", "save_freq", "log_freq", "output_dir", "seed",
        "profile", "resume_from", "resume_strict")]
    + ["trainer.debug.first_step", "trainer.debug.grad_split"]
)
_GRPO_DIFFUSION_REQUIRED: tuple[str, ...] = tuple(
    f"rollout.{k}" for k in
    ("n", "rollout_batch_size", "noise_level", "sample_batch_size", "sde.type",
     "sde.window_size", "sde.window_range", "same_latent")
)
_TOKEN_GRPO_REQUIRED: tuple[str, ...] = tuple(
    f"rollout.{k}" for k in
    ("n_samples_per_prompt", "rollout_batch_size", "rescale_to_unit", "max_text_length")
)
_DPO_REQUIRED: tuple[str, ...] = (
    "actor.mixed_precision", "actor.gradient_checkpointing", "actor.train_batch_size",
    "actor.gradient_accumulation_steps", "actor.scale_lr", "actor.use_adafactor",
    "actor.prediction_type", "data.random_crop", "data.no_hflip",
    "data.dataloader_num_workers", "data.resolution", "trainer.max_train_steps",
    "trainer.checkpointing_steps", "trainer.log_interval", "rollout.n",
    "rollout.rollout_batch_size",
)


# --------------------------------------------------------------------------- loading
def _default_path(entry: Any, root: Path) -> Path:
    if isinstance(entry, dict):
        if len(entry) != 1:
            raise ValueError(f"defaults dict must have exactly one key: {dict(entry)}")
        (group, option), = entry.items()
        entry = f"{group}/{option}"
    rel = str(entry).lstrip("/")
    if not rel.endswith(_YAML_SUFFIXES):
        rel += ".yaml"
    return root / rel


def _load_one(path: Path, root: Path, seen: frozenset[Path] = frozenset()) -> DictConfig:
    path = path.resolve()
    if path in seen:
        raise RuntimeError(f"Cyclic defaults: {path}")
    seen = seen | {path}
    body = load_yaml(path)
    if not isinstance(body, DictConfig):
        raise TypeError(f"{path}: top-level must be a mapping")
    defaults = body.pop("defaults", None)
    if defaults is None:
        return body
    if not isinstance(defaults, (list, ListConfig)):
        raise TypeError(f"{path}: 'defaults' must be a list")
    merged = DictConfig()
    placed_self = False
    for entry in defaults:
        if entry == _SELF:
            merged, placed_self = merge(merged, body), True
        else:
            merged = merge(merged, _load_one(_default_path(entry, root), root, seen))
    return merged if placed_self else merge(merged, body)


def load_config(
    path: str | Path,
    overrides: list[str] | None = None,
    root: Path | None = None,
) -> DictConfig:
    """Load ``path`` (absolute, existing-relative, or a name under the configs root)."""
    root = Path(root or CONFIGS_ROOT).resolve()
    candidate = Path(path)
    if not candidate.is_absolute() and not candidate.exists():
        rel = str(path).lstrip("/")
        if not rel.endswith(_YAML_SUFFIXES):
            rel += ".yaml"
        candidate = root / rel
    cfg = _load_one(candidate, root)
    if overrides:
        cfg = merge(cfg, from_dotlist(list(overrides)))
    resolve(cfg)
    return cfg


# ----------------------------------------------------------------- required access
def _walk(cfg: Any, path: str) -> tuple[bool, Any]:
    node = cfg
    for key in path.split("."):
        if not isinstance(node, dict) or key not in node:
            return False, None
        node = node[key]
    return True, node


def _plain(node: Any) -> Any:
    return to_container(node) if isinstance(node, (dict, list)) else node


def require(cfg: DictConfig, path: str) -> Any:
    """Value at dotted ``path``; absent or ``None`` raises with the path in the text."""
    found, node = _walk(cfg, path)
    if not found:
        raise ValueError(f"config missing required field: {path}")
    if node is None:
        raise ValueError(f"config missing required field: {path} (got None)")
    return _plain(node)


def optional_none(cfg: DictConfig, path: str) -> Any | None:
    """Like :func:`require` but an explicit YAML ``null`` is a legal value."""
    found, node = _walk(cfg, path)
    if not found:
        raise ValueError(f"config missing required field: {path}")
    return None if node is None else _plain(node)


def _path_exists(cfg: DictConfig, path: str) -> bool:
    return _walk(cfg, path)[0]


# ---------------------------------------------------------------------- validation
def validate_reward_config(cfg: DictConfig) -> None:
    if "reward" not in cfg:
        raise ValueError("config missing required field: reward")
    reward = cfg["reward"]
    if not isinstance(reward, dict) or "components" not in reward:
        raise ValueError("config missing required field: reward.components")
    components = to_container(reward["components"]) or {}
    if not isinstance(components, dict):
        raise ValueError("reward.components must be a mapping of name -> weight")
    kwargs = to_container(reward.get("kwargs")) or {}
    for name, sub in kwargs.items():
        if sub is not None and not isinstance(sub, dict):
            raise ValueError(
                f"reward.kwargs.{name} must be a mapping, got {type(sub).__name__}"
            )
    for name, needed in _REWARD_REQUIRED_KWARGS.items():
        if name not in components:
            continue
        try:
            weight = float(components[name])
        except (TypeError, ValueError) as exc:
            raise ValueError(
                f"reward.components.{name} must be numeric, got {components[name]!r}"
            ) from exc
        if weight <= 0:
            continue
        sub = kwargs.get(name)
        if not isinstance(sub, dict):
            raise ValueError(
                f"config missing required field: reward.kwargs.{name} "
                f"(component {name!r} has weight {weight} > 0)"
            )
        for key in needed:
            if key not in sub:
                raise ValueError(f"config missing required field: reward.kwargs.{name}.{key}")


def _resolve_algorithm_kind(algo: Any) -> str:
    if "adv_estimator" in algo:
        raise ValueError("algorithm.adv_estimator is no longer supported; use algorithm.kind")
    kind = algo.get("kind")
    if kind is None:
        raise ValueError("algorithm.kind required")
    kind = str(kind)
    if kind not in _KINDS:
        raise ValueError(
            f"unknown algorithm.kind={kind!r}; expected grpo / token_grpo / diffusion_dpo"
        )
    return kind


def validate_training_config(cfg: DictConfig) -> None:
    """Presence checks only — nothing here touches the filesystem."""
    for path in _COMMON_REQUIRED_FIELDS:
        require(cfg, path)
    entrypoint = require(cfg, "trainer.entrypoint")
    if not isinstance(entrypoint, str) or not entrypoint.strip():
        raise ValueError("trainer.entrypoint must be a non-empty import path")
    if "reward" in cfg:
        validate_reward_config(cfg)
    if "algorithm" not in cfg:
        raise ValueError("config missing required field: algorithm")
    kind = _resolve_algorithm_kind(cfg["algorithm"])
    if kind == "grpo":
        for path in _GRPO_DIFFUSION_REQUIRED:
            require(cfg, path)
        if str(require(cfg, "rollout.sde.type")) not in ("sde", "cps"):
            raise ValueError("rollout.sde.type must be 'sde' or 'cps'")
    elif kind == "token_grpo":
        for path in _TOKEN_GRPO_REQUIRED:
            require(cfg, path)
        if _path_exists(cfg, "model.family") and cfg["model"]["family"] == "nextstep_1":
            require(cfg, "rollout.noise_level")
    else:
        for path in _DPO_REQUIRED:
            require(cfg, path)
        optional_none(cfg, "data.max_train_samples")


# -------------------------------------------------------------------- typed builders
def build_trainer_config(cfg: DictConfig):
    from visionrl_b200.trainers.types import DebugConfig, EMAConfig, OptimConfig, TrainerConfig

    if _path_exists(cfg, "rollout.n_samples_per_prompt"):
        group = require(cfg, "rollout.n_samples_per_prompt")
    elif _path_exists(cfg, "rollout.n"):
        group = require(cfg, "rollout.n")
    else:
        raise ValueError(
            "config missing rollout group size: expected rollout.n or "
            "rollout.n_samples_per_prompt"
        )
    actor = {k: require(cfg, f"actor.{k}") for k in
             ("max_norm", "ppo_epochs", "bf16", "gradient_checkpointing", "timestep_fraction")}
    run = {k: require(cfg, f"trainer.{k}") for k in
           ("total_epochs", "save_freq", "log_freq", "output_dir", "seed", "resume_from",
            "resume_strict", "profile")}
    return TrainerConfig(
        optim=OptimConfig(**require(cfg, "actor.optim")),
        ema=EMAConfig(**require(cfg, "actor.ema")),
        debug=DebugConfig(**require(cfg, "trainer.debug")),
        n=group,
        rollout_batch_size=require(cfg, "rollout.rollout_batch_size"),
        **actor,
        **run,
    )


def build_algorithm_config(cfg: DictConfig):
    if "algorithm" not in cfg:
        raise ValueError("config missing `algorithm` section")
    kind = _resolve_algorithm_kind(cfg["algorithm"])
    raw = to_container(cfg["algorithm"]) or {}
    if kind == "grpo":
        from visionrl_b200.algorithms.grpo import GRPOConfig

        return GRPOConfig(**{k: v for k, v in raw.items() if k in _GRPO_FIELDS})
    if kind == "token_grpo":
        from visionrl_b200.algorithms.grpo_token import TokenGRPOConfig

        allowed = _GRPO_FIELDS | _TOKEN_GRPO_EXTRA_FIELDS
        return TokenGRPOConfig(**{k: v for k, v in raw.items() if k in allowed})
    from visionrl_b200.algorithms.dpo import DiffusionDPOConfig

    return DiffusionDPOConfig(**{k: v for k, v in raw.items() if k in _DPO_FIELDS})


def build_reward_config(cfg: DictConfig) -> tuple[dict[str, float], dict[str, dict]]:
    validate_reward_config(cfg)
    components = to_container(cfg["reward"]["components"]) or {}
    weights = {name: float(w) for name, w in components.items() if float(w) > 0}
    kwargs = to_container(cfg["reward"].get("kwargs")) or {}
    return weights, {k: (v or {}) for k, v in kwargs.items()}


def build_configs(cfg: DictConfig) -> dict[str, Any]:
    validate_training_config(cfg)
    out: dict[str, Any] = {
        "trainer": build_trainer_config(cfg),
        "algorithm": build_algorithm_config(cfg),
        "raw": cfg,
    }
    if "reward" in cfg:
        out["reward"] = build_reward_config(cfg)
    return out


__all__ = [
    "CONFIGS_ROOT",
    "DictConfig",
    "ListConfig",
    "OmegaConf",
    "build_algorithm_config",
    "build_configs",
    "build_reward_config",
    "build_trainer_config",
    "load_config",
    "optional_none",
    "require",
    "validate_reward_config",
    "validate_training_config",
]
