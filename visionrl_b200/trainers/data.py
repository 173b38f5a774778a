"""Prompt sources: manifest loading, datasets and the K-repeat distributed sampler
(reference: ``vrl/trainers/data.py:19-166``).

Manifests are ``.jsonl`` (one object per line with ``PromptExample`` fields) or
``.txt`` (one prompt per line; the OCR target is the text between the first pair of
double quotes).  ``synthetic:<n>[:<seed>]`` yields ``n`` generated prompts without
touching the filesystem.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

import torch
from torch.utils.data import Dataset, Sampler


@dataclass(slots=True)
class PromptExample:
    prompt: str
    target_text: str = ""
    references: list[str] = field(default_factory=list)
    task_type: str = "text_to_video"
    request_overrides: dict[str, Any] = field(default_factory=dict)
    metadata: dict[str, Any] = field(default_factory=dict)


_WORDS = ("amber", "birch", "cobalt", "dune", "ember", "fjord", "glade", "harbor", "iris", "jade",
          "kelp", "lotus", "mesa", "nectar", "onyx", "pearl", "quartz", "reef", "slate", "tundra")


def synthetic_prompts(count: int, seed: int = 0) -> list[PromptExample]:
    gen = torch.Generator().manual_seed(seed)
    out = []
    for i in range(count):
        picks = torch.randint(0, len(_WORDS), (4,), generator=gen).tolist()
        target = _WORDS[picks[0]]
        text = f'a sign that says "{target}" near a {_WORDS[picks[1]]} {_WORDS[picks[2]]}, {_WORDS[picks[3]]} light #{i}'
        out.append(PromptExample(prompt=text, target_text=target))
    return out


def load_prompt_manifest(path: str | Path) -> list[PromptExample]:
    text = str(path)
    if text.startswith("synthetic:"):
        parts = text.split(":")
        return synthetic_prompts(int(parts[1]), int(parts[2]) if len(parts) > 2 else 0)
    p = Path(path)
    if p.suffix == ".jsonl":
        return list(JsonlPromptDataset(p).examples)
    if p.suffix == ".txt":
        examples = []
        for line in p.read_text(encoding="utf-8").splitlines():
            line = line.strip()
            if not line:
                continue
            pieces = line.split('"')
            examples.append(PromptExample(prompt=line,
                                          target_text=pieces[1] if len(pieces) >= 3 else ""))
        return examples
    raise ValueError(f"Unsupported manifest suffix: {p.suffix}")


def _collate(examples: list[dict[str, Any]]) -> tuple[list[str], list[dict]]:
    return [e["prompt"] for e in examples], [e["metadata"] for e in examples]


class JsonlPromptDataset(Dataset):
    def __init__(self, path: str | Path) -> None:
        self.examples: list[PromptExample] = []
        with open(path, encoding="utf-8") as fh:
            for line in fh:
                if line.strip():
                    self.examples.append(PromptExample(**json.loads(line)))

    def __len__(self) -> int:
        return len(self.examples)

    def __getitem__(self, idx: int) -> dict[str, Any]:
        ex = self.examples[idx]
        return {"prompt": ex.prompt, "metadata": ex.metadata, "example": ex}

    collate_fn = staticmethod(_collate)


class TextPromptDataset(Dataset):
    def __init__(self, path: str) -> None:
        with open(path, encoding="utf-8") as fh:
            self.prompts = [line.strip() for line in fh if line.strip()]

    def __len__(self) -> int:
        return len(self.prompts)

    def __getitem__(self, idx: int) -> dict[str, Any]:
        return {"prompt": self.prompts[idx], "metadata": {}}

    collate_fn = staticmethod(_collate)


class DistributedKRepeatSampler(Sampler):
    """Every iteration draws ``M = replicas * batch / K`` unique prompts, repeats each ``K``
    times, shuffles with a seed shared by all ranks and hands rank ``r`` its slice — so
    the ranks together always hold complete groups.  Iterates forever."""

    def __init__(self, dataset: Dataset, batch_size: int, k: int, num_replicas: int, rank: int,
                 seed: int = 0) -> None:
        self.dataset, self.batch_size, self.k = dataset, batch_size, k
        self.num_replicas, self.rank, self.seed = num_replicas, rank, seed
        self.total_samples = num_replicas * batch_size
        if self.total_samples % k != 0:
            raise AssertionError(f"k ({k}) must divide num_replicas*batch_size ({self.total_samples})")
        self.m = self.total_samples // k
        self.epoch = 0

    def __iter__(self):
        while True:
            gen = torch.Generator().manual_seed(self.seed + self.epoch)
            chosen = torch.randperm(len(self.dataset), generator=gen)[: self.m].tolist()
            repeated = [i for i in chosen for _ in range(self.k)]
            order = torch.randperm(len(repeated), generator=gen).tolist()
            mixed = [repeated[i] for i in order]
            lo = self.rank * self.batch_size
            yield mixed[lo: lo + self.batch_size]

    def set_epoch(self, epoch: int) -> None:
        self.epoch = epoch
