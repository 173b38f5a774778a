"""Training checkpoints.

Layout of ``<output_dir>/checkpoint-<N>/`` (reference: ``vrl/trainers/checkpointing.py:17-410``):

* ``checkpoint.pt`` — ``torch.save`` of ``{schema_version: 1, family, trainer, model:
  {trainable_modules: {name: cpu_state_dict}}, progress, rng}``; the only resume source;
* ``checkpoint_meta.json`` — human-readable summary (steps, epochs, LoRA flag);
* ``lora_weights/`` (optional) — adapter export of modules exposing ``save_pretrained``.

With sharded parameters the caller passes a bundle whose modules return fully
assembled state dicts, so a checkpoint written by N ranks loads on any other N.
"""

from __future__ import annotations

import json
import os
import logging
import re
from dataclasses import dataclass
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

import torch

from visionrl_b200.rollouts.runtime.config import cfg_get, cfg_path

logger = logging.getLogger(__name__)

CHECKPOINT_SCHEMA_VERSION = 1
TRAINING_CHECKPOINT_NAME = "checkpoint.pt"
LORA_WEIGHTS_NAME = "lora_weights"
CHECKPOINT_META_NAME = "checkpoint_meta.json"


def _nonneg(value: Any, name: str) -> int:
    try:
        out = int(value)
    except (TypeError, ValueError) as exc:
        raise ValueError(f"{name} must be an integer, got {value!r}") from exc
    if out < 0:
        raise ValueError(f"{name} must be >= 0, got {out}")
    return out


def _dict_field(container: dict, key: str, label: str, default: Any = None) -> dict:
    value = container.get(key, default)
    if not isinstance(value, dict):
        raise TypeError(f"checkpoint payload missing dict field: {label}"
                        if default is None else f"checkpoint payload field {label} must be a dict")
    return value


@dataclass(frozen=True, slots=True)
class TrainingCheckpoint:
    checkpoint_dir: Path
    checkpoint_path: Path
    payload: dict[str, Any]
    meta: dict[str, Any]

    @property
    def trainer_state(self) -> dict[str, Any]:
        return _dict_field(self.payload, "trainer", "trainer")

    @property
    def trainable_state(self) -> dict[str, Any]:
        return _dict_field(_dict_field(self.payload, "model", "model"), "trainable_modules",
                           "model.trainable_modules")

    @property
    def progress(self) -> dict[str, Any]:
        return _dict_field(self.payload, "progress", "progress", {})

    @property
    def rng_state(self) -> dict[str, Any]:
        return _dict_field(self.payload, "rng", "rng", {})

    @property
    def next_epoch(self) -> int:
        if "next_epoch" in self.progress:
            return _nonneg(self.progress["next_epoch"], "progress.next_epoch")
        return infer_next_epoch(self.checkpoint_dir, self.trainer_state, self.meta)

    @property
    def next_step(self) -> int:
        if "next_step" in self.progress:
            return _nonneg(self.progress["next_step"], "progress.next_step")
        for key in ("global_step", "step"):
            if key in self.trainer_state:
                return _nonneg(self.trainer_state[key], f"trainer.{key}")
        return self.next_epoch


def _to_cpu(value: Any) -> Any:
    if isinstance(value, torch.Tensor):
        return value.detach().cpu()
    if isinstance(value, dict):
        return {k: _to_cpu(v) for k, v in value.items()}
    if isinstance(value, (list, tuple)):
        return type(value)(_to_cpu(v) for v in value)
    return value


def _modules(bundle: Any) -> dict[str, Any]:
    modules = getattr(bundle, "trainable_modules", None)
    if not isinstance(modules, dict) or not modules:
        raise ValueError("RuntimeBundle.trainable_modules must be a non-empty dict")
    return modules


def export_trainable_state(bundle: Any) -> dict[str, dict[str, Any]]:
    out = {}
    for name, module in _modules(bundle).items():
        if not callable(getattr(module, "state_dict", None)):
            raise TypeError(f"trainable module {name!r} does not expose state_dict()")
        out[name] = _to_cpu(module.state_dict())
    return out


def join_trainable_state_gathers(bundle: Any) -> None:
    """What a rank that does NOT write the checkpoint has to do while the writer exports the model:
    row-sharded weights are saved at their full shape, and gathering them is a collective (or needs
    the peers' shards to stay put), so every rank walks the same state dicts in the same order and
    throws the result away.  Modules without sharded layers are skipped."""
    for module in _modules(bundle).values():
        layers = getattr(module, "modules", None)
        if callable(layers) and any(getattr(m, "sharded", None) is not None for m in layers()):
            module.state_dict()


def load_trainable_state(bundle: Any, state: dict[str, Any], *, strict: bool = True) -> None:
    modules = _modules(bundle)
    missing, extra = sorted(set(modules) - set(state)), sorted(set(state) - set(modules))
    if strict and (missing or extra):
        raise ValueError(f"checkpoint trainable module keys mismatch: missing={missing}, extra={extra}")
    for name, module in modules.items():
        if name not in state:
            continue
        if not callable(getattr(module, "load_state_dict", None)):
            raise TypeError(f"trainable module {name!r} does not expose load_state_dict()")
        module.load_state_dict(state[name], strict=strict)


def capture_rng_state(**generators: torch.Generator) -> dict[str, Any]:
    import random

    import numpy as np

    state: dict[str, Any] = {
        "torch": torch.get_rng_state(),
        "generators": {name: g.get_state() for name, g in generators.items()},
        "python_random": random.getstate(),
        "numpy": np.random.get_state(),
    }
    if torch.cuda.is_available():
        state["cuda"] = torch.cuda.get_rng_state_all()
    return state


def restore_rng_state(state: dict[str, Any] | None, **generators: torch.Generator) -> None:
    if not state:
        return
    import random

    import numpy as np

    if "torch" in state:
        torch.set_rng_state(state["torch"])
    if "cuda" in state and torch.cuda.is_available():
        try:
            torch.cuda.set_rng_state_all(state["cuda"])
        except Exception:  # noqa: BLE001 - device count may differ from the saving run
            logger.warning("could not restore CUDA RNG state (device count changed?)")
    named = state.get("generators", {})
    if isinstance(named, dict):
        for name, g in generators.items():
            if name in named:
                g.set_state(named[name])
    if "python_random" in state:
        random.setstate(state["python_random"])
    if "numpy" in state:
        np.random.set_state(state["numpy"])


def write_checkpoint_meta(checkpoint_dir: str | Path, *, family: str, trainer_state: dict[str, Any],
                          completed_epoch: int, next_epoch: int, uses_lora: bool) -> dict[str, Any]:
    meta = {
        "schema_version": CHECKPOINT_SCHEMA_VERSION, "family": family,
        "trainer_step": int(trainer_state.get("step", 0)),
        "global_step": int(trainer_state.get("global_step", 0)),
        "completed_epoch": int(completed_epoch), "next_epoch": int(next_epoch),
        "uses_lora": bool(uses_lora),
    }
    path = Path(checkpoint_dir)
    path.mkdir(parents=True, exist_ok=True)
    (path / CHECKPOINT_META_NAME).write_text(json.dumps(meta, indent=2, sort_keys=True) + "\n")
    return meta


def read_checkpoint_meta(checkpoint_dir: str | Path) -> dict[str, Any]:
    meta_path = Path(checkpoint_dir) / CHECKPOINT_META_NAME
    if not meta_path.exists():
        return {}
    raw = json.loads(meta_path.read_text())
    if not isinstance(raw, dict):
        raise TypeError(f"{meta_path} must contain a JSON object")
    return raw


def infer_next_epoch(checkpoint_dir: str | Path, trainer_state: dict[str, Any],
                     meta: dict[str, Any] | None) -> int:
    meta = meta or {}
    if "next_epoch" in meta:
        return _nonneg(meta["next_epoch"], "checkpoint_meta.next_epoch")
    if "step" in trainer_state:
        return _nonneg(trainer_state["step"], "trainer_state.step")
    match = re.fullmatch(r"checkpoint-(\d+)", Path(checkpoint_dir).name)
    if match:
        return _nonneg(match.group(1), "checkpoint directory suffix")
    raise ValueError("cannot infer next_epoch: checkpoint_meta.next_epoch and trainer_state.step "
                     "are missing")


def save_training_checkpoint(checkpoint_dir: str | Path, *, trainer: Any, bundle: Any, family: str,
                             progress: dict[str, Any], rng_state: dict[str, Any] | None = None,
                             export_modules: dict[str, Any] | None = None) -> dict[str, Any]:
    path = Path(checkpoint_dir)
    path.mkdir(parents=True, exist_ok=True)
    trainer_state = trainer.state_dict()
    payload = {
        "schema_version": CHECKPOINT_SCHEMA_VERSION, "family": family, "trainer": trainer_state,
        "model": {"trainable_modules": export_trainable_state(bundle)},
        "progress": dict(progress), "rng": rng_state or capture_rng_state(),
    }
    # written under a temporary name and renamed, and the meta file is written last: a checkpoint
    # directory that has its meta file is complete, whatever interrupted the run
    partial = path / (TRAINING_CHECKPOINT_NAME + ".partial")
    torch.save(payload, partial)
    os.replace(partial, path / TRAINING_CHECKPOINT_NAME)
    for name, module in (export_modules or {}).items():
        if not callable(getattr(module, "save_pretrained", None)):
            raise TypeError(f"export module {name!r} does not expose save_pretrained()")
        module.save_pretrained(path / name)
    meta = write_checkpoint_meta(
        path, family=family, trainer_state=trainer_state,
        completed_epoch=int(progress.get("completed_epoch", progress.get("next_epoch", 0))),
        next_epoch=int(progress.get("next_epoch", progress.get("next_step", 0))),
        uses_lora=bool((export_modules or {}).get(LORA_WEIGHTS_NAME)),
    )
    meta["checkpoint_file"] = TRAINING_CHECKPOINT_NAME
    (path / CHECKPOINT_META_NAME).write_text(json.dumps(meta, indent=2, sort_keys=True) + "\n")
    return meta


def load_training_checkpoint(path: str | Path) -> TrainingCheckpoint:
    raw = Path(path).expanduser().resolve()
    file = raw if raw.is_file() else raw / TRAINING_CHECKPOINT_NAME
    if not file.exists():
        raise FileNotFoundError(f"training checkpoint file not found: {file}")
    payload = torch.load(file, map_location="cpu", weights_only=False)
    if not isinstance(payload, dict):
        raise TypeError(f"{file} must contain a dict payload")
    version = int(payload.get("schema_version", 0))
    if version != CHECKPOINT_SCHEMA_VERSION:
        raise ValueError(f"unsupported checkpoint schema_version={version}; "
                         f"expected {CHECKPOINT_SCHEMA_VERSION}")
    return TrainingCheckpoint(file.parent, file, payload, read_checkpoint_meta(file.parent))


AUTO_RESUME = "auto"


def latest_checkpoint(output_dir: str | Path) -> Path | None:
    """The complete checkpoint directory below ``output_dir`` that is furthest along, or ``None``.

    Complete means that both the payload and the meta file are there (the meta file is written
    last).  Directories are ranked by the ``next_epoch`` recorded in their meta file, the newer
    file winning a tie (``checkpoint-3`` and ``checkpoint-final`` of a three-epoch run)."""
    root = Path(output_dir).expanduser()
    if not root.is_dir():
        return None
    best: tuple[int, float, Path] | None = None
    for child in root.iterdir():
        payload, meta_file = child / TRAINING_CHECKPOINT_NAME, child / CHECKPOINT_META_NAME
        if not (child.is_dir() and payload.is_file() and meta_file.is_file()):
            continue
        try:
            meta = json.loads(meta_file.read_text())
            progress = int(meta["next_epoch"])
        except (OSError, ValueError, KeyError, TypeError):
            continue
        key = (progress, payload.stat().st_mtime, child)
        if best is None or key[:2] > best[:2]:
            best = key
    return None if best is None else best[2]


def load_training_checkpoint_from_config(cfg: Any) -> TrainingCheckpoint | None:
    """``trainer.resume_from`` names a checkpoint directory (or file); ``auto`` means the latest
    complete checkpoint below ``trainer.output_dir`` and a fresh start when there is none — the
    setting under which a relaunched job (``torchrun --max-restarts``, or the restart loop of
    ``visionrl_b200.scripts.elastic``) carries on where the failed one stopped."""
    resume = str(cfg_path(cfg, "trainer.resume_from", "") or "").strip()
    if resume.lower() == AUTO_RESUME:
        found = latest_checkpoint(str(cfg_path(cfg, "trainer.output_dir", "") or "."))
        if found is None:
            logger.info("trainer.resume_from=auto: no complete checkpoint below %s, starting fresh",
                        cfg_path(cfg, "trainer.output_dir", "."))
            return None
        logger.info("trainer.resume_from=auto: resuming from %s", found)
        return load_training_checkpoint(found)
    return load_training_checkpoint(resume) if resume else None


def prepare_model_config_for_training_resume(cfg: Any, checkpoint: TrainingCheckpoint | None, *,
                                             strict: bool = True) -> None:
    """A full resume restores adapters from ``checkpoint.pt``; a warm-start ``model.lora.path``
    on top of it is rejected (strict) or cleared (non-strict)."""
    if checkpoint is None:
        return
    lora_path = cfg_path(cfg, "model.lora.path", None)
    if lora_path is None or not str(lora_path or "").strip():
        return
    if strict:
        raise ValueError("trainer.resume_from cannot be combined with model.lora.path; "
                         "checkpoint.pt is the resume source of truth")
    node = cfg_path(cfg, "model.lora", None)
    try:
        node["path"] = ""
    except TypeError:
        setattr(node, "path", "")


def restore_training_checkpoint(checkpoint: TrainingCheckpoint | None, *, trainer: Any, bundle: Any,
                                strict: bool = True) -> None:
    if checkpoint is None:
        return
    saved = checkpoint.payload.get("family")
    current = getattr(bundle, "metadata", {}).get("family")
    if strict and saved and current and str(saved) != str(current):
        raise ValueError(f"checkpoint family mismatch: checkpoint={saved!r}, bundle={current!r}")
    load_trainable_state(bundle, checkpoint.trainable_state, strict=strict)
    trainer.load_state_dict(checkpoint.trainer_state, strict=strict)


def save_resolved_config(cfg: Any, output_dir: str | Path, *, resumed: bool) -> None:
    from visionrl_b200.config.node import save_yaml

    path = Path(output_dir)
    path.mkdir(parents=True, exist_ok=True)
    target = path / "resolved_config.yaml"
    if resumed and target.exists():
        stamp = datetime.now(timezone.utc).strftime("%Y%m%d_%H%M%S")
        target = path / f"resume_config_{stamp}.yaml"
    save_yaml(cfg, target)


def prepare_metrics_csv(csv_path: str | Path, header: str, *, resume: bool) -> None:
    path = Path(csv_path)
    if resume and path.exists():
        return
    if resume:
        logger.warning("Resume requested but metrics file does not exist; creating %s", path)
    path.parent.mkdir(parents=True, exist_ok=True)
    path.write_text(header)


def sample_prompt_indices(rng: torch.Generator, *, num_examples: int,
                          rollout_batch_size: int) -> list[int]:
    if num_examples < 1:
        raise ValueError("prompt manifest must contain at least one example")
    if rollout_batch_size < 1:
        raise ValueError("rollout_batch_size must be >= 1")
    return torch.randperm(num_examples, generator=rng)[:rollout_batch_size].tolist()


__all__ = [
    "CHECKPOINT_META_NAME", "CHECKPOINT_SCHEMA_VERSION", "LORA_WEIGHTS_NAME",
    "TRAINING_CHECKPOINT_NAME", "TrainingCheckpoint", "capture_rng_state",
    "AUTO_RESUME", "export_trainable_state", "join_trainable_state_gathers", "infer_next_epoch",
    "latest_checkpoint", "load_trainable_state",
    "load_training_checkpoint", "load_training_checkpoint_from_config", "prepare_metrics_csv",
    "prepare_model_config_for_training_resume", "read_checkpoint_meta", "restore_rng_state",
    "restore_training_checkpoint", "sample_prompt_indices", "save_resolved_config",
    "save_training_checkpoint", "write_checkpoint_meta",
]
