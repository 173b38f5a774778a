"""The post-step check of the kernels' status words, exercised on CPU against a stand-in for the
compiled extension: nothing is read on a CPU device, a clean read costs 16 bytes (32 with the
collective runtime's own word), a non-zero word raises and names the kernel."""

import types

import pytest
import torch

from visionrl_b200.ops import _ext
from visionrl_b200.trainers import base


class _GradSync:
    def __init__(self):
        self.calls = []

    def check(self, where):
        self.calls.append(where)


@pytest.fixture
def fake_extension(monkeypatch):
    words = [0, 0, 0]
    module = types.SimpleNamespace(kernel_status_all=lambda: list(words))
    monkeypatch.setattr(_ext, "available", lambda: True)
    monkeypatch.setattr(_ext, "kernels_enabled", lambda: True)
    monkeypatch.setattr(_ext, "load", lambda: module)
    return words


def test_cpu_device_reads_nothing(fake_extension):
    fake_extension[0] = 2
    assert base.raise_on_kernel_timeout(torch.device("cpu")) == 0


def test_clean_words_cost_sixteen_bytes_and_the_collective_word_sixteen_more(fake_extension):
    assert base.raise_on_kernel_timeout("cuda") == 16
    sync = _GradSync()
    assert base.raise_on_kernel_timeout(torch.device("cuda", 0), sync, "training step 7") == 32
    assert sync.calls == ["training step 7"]


@pytest.mark.parametrize("index,fragment", [(0, "bf16 GEMM"), (1, "attention"), (2, "int4 GEMM")])
def test_a_word_that_is_set_raises_and_names_its_kernel(fake_extension, index, fragment):
    fake_extension[index] = 31 if index == 1 else 2
    sync = _GradSync()
    with pytest.raises(RuntimeError, match="gave up waiting") as err:
        base.raise_on_kernel_timeout("cuda", sync)
    assert fragment in str(err.value) and f"status {fake_extension[index]}" in str(err.value)
    assert sync.calls == [], "the collective check is not reached once a kernel reported"


def test_kernels_switched_off_reads_nothing(fake_extension, monkeypatch):
    monkeypatch.setattr(_ext, "kernels_enabled", lambda: False)
    fake_extension[2] = 1
    assert base.raise_on_kernel_timeout("cuda") == 0


def test_describe_lists_only_the_words_that_are_set():
    assert base.describe_kernel_status([0, 0, 0]) == []
    lines = base.describe_kernel_status([3, 0, 1])
    assert len(lines) == 2 and lines[0].endswith("status 3") and lines[1] == "int4 GEMM: status 1"
