"""OCR text-match reward with a pluggable recognition engine.

For every scored frame ``reward = 1 - min(lev(text, target), len(target)) / len(target)`` on
whitespace-stripped, lower-cased strings; a single image gets full credit when the target is
a substring of the recognised text; videos score every 4th frame and average the frames
with positive reward; no target → 0 (reference: ``vrl/rewards/ocr.py:27-216``).

``engine`` is any callable ``frame[H, W, 3] uint8 → str``.  Without one, ``paddleocr`` /
``rapidocr_onnxruntime`` are tried in that order on first use.  The Levenshtein distance is
built in.
"""

from __future__ import annotations

import re
from pathlib import Path
from typing import Any, Callable

from visionrl_b200.algorithms.types import Rollout
from visionrl_b200.rewards.base import RewardFunction


def _normalize_ocr_text(text: str) -> str:
    return text.replace(" ", "").lower()


def _normalize_text(text: str) -> str:
    cleaned = re.sub(r"[^a-z0-9\s]+", "", text.lower())
    return re.sub(r"\s+", " ", cleaned).strip()


def _edit_distance(a: str, b: str) -> int:
    if a == b:
        return 0
    if not a or not b:
        return len(a) + len(b)
    row = list(range(len(b) + 1))
    for i, ca in enumerate(a, 1):
        diag, row[0] = row[0], i
        for j, cb in enumerate(b, 1):
            diag, row[j] = row[j], min(row[j] + 1, row[j - 1] + 1, diag + (ca != cb))
    return row[-1]


def _normalized_edit_distance(a: str, b: str) -> float:
    if not a and not b:
        return 0.0
    return _edit_distance(a, b) / max(len(a), len(b), 1)


def _safe_filename_fragment(text: str, max_len: int = 24) -> str:
    """Letters and digits of ``text`` joined by single underscores, at most ``max_len`` characters;
    ``"empty"`` when nothing is left."""
    return re.sub(r"[^A-Za-z0-9]+", "_", text).strip("_")[:max_len] or "empty"


def _import_engine(path: str) -> Callable[[Any], str]:
    import importlib

    module, _, name = path.partition(":")
    if not module or not name:
        raise ValueError(f"OCR engine {path!r}: expected 'package.module:function'")
    engine = getattr(importlib.import_module(module), name, None)
    if not callable(engine):
        raise ValueError(f"OCR engine {path!r} does not name a callable")
    return engine


def _default_engine() -> Callable[[Any], str]:
    try:
        from paddleocr import PaddleOCR

        ocr = PaddleOCR(use_angle_cls=False, lang="en", use_gpu=False, show_log=False)

        def run(frame) -> str:
            result = ocr.ocr(frame, cls=False)
            if result and result[0]:
                return "".join(r[1][0] if r[1][1] > 0 else "" for r in result[0])
            return ""

        return run
    except ImportError:
        pass
    try:
        from rapidocr_onnxruntime import RapidOCR

        ocr2 = RapidOCR()

        def run2(frame) -> str:
            result, _ = ocr2(frame)
            return "".join(r[1] for r in result) if result else ""

        return run2
    except ImportError as exc:
        raise ImportError("OCRReward needs an OCR engine: install paddleocr or "
                          "rapidocr_onnxruntime, or pass engine=<callable>") from exc


class OCRReward(RewardFunction):
    frame_interval: int = 4

    def __init__(self, device: str = "cuda", debug_dir: str | None = None,
                 engine: Callable[[Any], str] | str | None = None) -> None:
        self._device = device
        # a callable frame -> text, or its import path ("package.module:function") so that a YAML
        # config can name one (``reward.kwargs.ocr.engine``)
        self._engine = _import_engine(engine) if isinstance(engine, str) and engine else engine
        self._debug_dir = Path(debug_dir) if debug_dir else None
        self._debug_counter = 0
        if self._debug_dir is not None:
            self._debug_dir.mkdir(parents=True, exist_ok=True)

    def _ensure_loaded(self) -> None:
        if self._engine is None:
            self._engine = _default_engine()

    def _read(self, frame: Any) -> str:
        """Text of one frame.  The engine is a callable ``frame -> text``, or an object with the
        ``ocr(frame, cls=False)`` method of PaddleOCR (lines of ``[box, (text, confidence)]``)."""
        engine = self._engine
        if callable(engine):
            return str(engine(frame))
        result = engine.ocr(frame, cls=False)
        if result and result[0]:
            return "".join(line[1][0] if line[1][1] > 0 else "" for line in result[0])
        return ""

    def _frames(self, output: Any) -> tuple[list, bool]:
        import numpy as np
        import torch

        if not isinstance(output, torch.Tensor):
            arr = np.asarray(output)
            return [arr], arr.ndim == 3
        raw = (output * 255).round().clamp(0, 255).to(torch.uint8)
        if raw.ndim == 3:
            return [raw.permute(1, 2, 0).cpu().numpy()], True
        if raw.ndim != 4:
            raise ValueError(f"OCRReward expected image/video tensor with 3 or 4 dims, got {raw.ndim}")
        video = raw.permute(1, 2, 3, 0) if raw.shape[0] <= 4 else raw.permute(0, 2, 3, 1)
        return list(video.cpu().numpy()[:: self.frame_interval]), False

    async def score(self, rollout: Rollout) -> float:
        target_raw = rollout.metadata.get("target_text", "")
        target = _normalize_ocr_text(target_raw) if target_raw else ""
        if not target:
            return 0.0
        self._ensure_loaded()
        frames, single = self._frames(rollout.trajectory.output)
        positive: list[float] = []
        best = (0.0, None, "")
        for frame in frames:
            seen_raw = self._read(frame)
            seen = _normalize_ocr_text(seen_raw)
            dist = 0 if single and target in seen else _edit_distance(seen, target)
            reward = 1.0 - min(dist, len(target)) / len(target)
            if reward > 0:
                positive.append(reward)
            if reward > best[0]:
                best = (reward, frame, seen_raw)
        value = sum(positive) / len(positive) if positive else 0.0
        if self._debug_dir is not None and best[1] is not None:
            self._dump(best[1], target_raw, best[2], value)
        return value

    def _dump(self, frame: Any, target: str, seen: str, value: float) -> None:
        try:
            from PIL import Image

            stem = f"{self._debug_counter:06d}_{_safe_filename_fragment(target)}_score{value:.3f}"
            self._debug_counter += 1
            Image.fromarray(frame).save(self._debug_dir / f"{stem}.png")
            (self._debug_dir / f"{stem}.txt").write_text(
                f"target: {target}\nocr:    {seen}\nscore:  {value:.4f}\n", encoding="utf-8")
        except Exception:  # noqa: BLE001 - debugging aid only
            pass

    async def score_batch(self, rollouts: list[Rollout]) -> list[float]:
        return [await self.score(r) for r in rollouts]
