"""Preference-pair data for Diffusion-DPO (reference: ``vrl/trainers/pickapic.py:26-141``).

``PreferenceBatch.pixel_values`` is ``[B, 6, H, W]`` with the winner in channels 0-2 and
the loser in channels 3-5; ``stacked_winner_then_loser()`` gives the ``[2B, 3, H, W]``
layout the DPO loss expects.  ``SyntheticLatentPairs`` yields seed-generated latent
pairs directly (no image files, no VAE encode).
"""

from __future__ import annotations

import io
from collections.abc import Iterable
from dataclasses import dataclass
from typing import Any

import torch
from torch.utils.data import Dataset


@dataclass(slots=True)
class PreferenceBatch:
    pixel_values: torch.Tensor
    captions: list[str]

    def split_winner_loser(self) -> tuple[torch.Tensor, torch.Tensor]:
        c = self.pixel_values.shape[1] // 2
        return self.pixel_values[:, :c], self.pixel_values[:, c:]

    def stacked_winner_then_loser(self) -> torch.Tensor:
        return torch.cat(self.split_winner_loser(), dim=0)


@dataclass(slots=True)
class LatentPreferenceBatch:
    """Winner / loser latents that skip the pixel encoder."""

    winner: torch.Tensor
    loser: torch.Tensor
    captions: list[str]

    def latents_winner_then_loser(self) -> torch.Tensor:
        return torch.cat([self.winner, self.loser], dim=0)


class SyntheticLatentPairs(Dataset):
    """``num_pairs`` latent pairs drawn from a seed; the winner is a low-noise and the
    loser a high-noise perturbation of one shared base sample."""

    def __init__(self, latent_shape: tuple, num_pairs: int = 64, seed: int = 0):
        self.latent_shape, self.num_pairs, self.seed = tuple(latent_shape), num_pairs, seed

    def __len__(self) -> int:
        return self.num_pairs

    def __getitem__(self, idx: int) -> dict[str, Any]:
        g = torch.Generator().manual_seed(self.seed * 1_000_003 + idx)
        base = torch.randn(self.latent_shape, generator=g)
        return {"winner": base + 0.1 * torch.randn(self.latent_shape, generator=g),
                "loser": base + 0.5 * torch.randn(self.latent_shape, generator=g),
                "caption": f"synthetic preference pair {idx}"}


def collate_latent_pairs(examples: Iterable[dict[str, Any]]) -> LatentPreferenceBatch:
    items = list(examples)
    return LatentPreferenceBatch(torch.stack([e["winner"] for e in items]),
                                 torch.stack([e["loser"] for e in items]),
                                 [e["caption"] for e in items])


class PickAPicPreferenceDataset(Dataset):
    """HF ``datasets`` rows → tensors in ``[-1, 1]``; ties (label 0.5) are dropped."""

    def __init__(self, hf_dataset: Any, resolution: int = 512, random_crop: bool = False,
                 no_hflip: bool = False) -> None:
        from torchvision import transforms

        keep = [i for i, label in enumerate(hf_dataset["label_0"]) if label in (0, 1)]
        if len(keep) < len(hf_dataset):
            hf_dataset = hf_dataset.select(keep)
        self._ds = hf_dataset
        steps: list[Any] = [
            transforms.Resize(resolution, interpolation=transforms.InterpolationMode.BILINEAR),
            transforms.RandomCrop(resolution) if random_crop else transforms.CenterCrop(resolution),
        ]
        if not no_hflip:
            steps.append(transforms.RandomHorizontalFlip())
        steps += [transforms.ToTensor(), transforms.Normalize([0.5], [0.5])]
        self._tx = transforms.Compose(steps)

    def __len__(self) -> int:
        return len(self._ds)

    def __getitem__(self, idx: int) -> dict[str, Any]:
        from PIL import Image

        row = self._ds[idx]
        first_wins = row["label_0"] == 1
        win, lose = (row["jpg_0"], row["jpg_1"]) if first_wins else (row["jpg_1"], row["jpg_0"])
        load = lambda raw: self._tx(Image.open(io.BytesIO(raw)).convert("RGB"))  # noqa: E731
        return {"pixel_values": torch.cat([load(win), load(lose)], dim=0), "caption": row["caption"]}


def collate_preference(examples: Iterable[dict[str, Any]]) -> PreferenceBatch:
    items = list(examples)
    pixels = torch.stack([e["pixel_values"] for e in items]).contiguous().float()
    return PreferenceBatch(pixel_values=pixels, captions=[e["caption"] for e in items])


def load_pickapic(split: str = "train", cache_dir: str | None = None, streaming: bool = False,
                  max_samples: int | None = None, resolution: int = 512, random_crop: bool = False,
                  no_hflip: bool = False,
                  dataset_name: str = "yuvalkirstain/pickapic_v2") -> PickAPicPreferenceDataset:
    from datasets import load_dataset

    ds = load_dataset(dataset_name, split=split, cache_dir=cache_dir, streaming=streaming)
    if max_samples is not None and not streaming:
        ds = ds.select(range(min(max_samples, len(ds))))
    return PickAPicPreferenceDataset(ds, resolution=resolution, random_crop=random_crop,
                                     no_hflip=no_hflip)
