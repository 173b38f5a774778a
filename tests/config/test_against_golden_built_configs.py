"""Typed configs and validation outcomes against the reference loader's.  ``tests/golden/built_configs.json``
was produced by the reference's own ``load_config`` + ``build_configs`` on its own YAML tree (run on
top of this repository's ``OmegaConf`` facade, which also shows that the facade serves that loader):
the trainer, algorithm and reward configs of its ten experiments, and what eight broken variants of
one experiment lead to (accepted, or the exception type and the start of its message)."""

import dataclasses
import json
import os

import pytest

from visionrl_b200.config import loader as L

with open(os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "built_configs.json")) as fh:
    GOLDEN = json.load(fh)

BREAKS = {"no_entrypoint": ["trainer.entrypoint=null"], "bad_kind": ["algorithm.kind=ppo"], "neg_lr": ["actor.optim.lr=-1"],
          "zero_n": ["rollout.n=0"], "bad_reward": ["reward.components.unknown_reward=1.0"],
          "all_zero_rewards": ["reward.components.ocr=0.0"], "bad_sde": ["rollout.sde.type=foo"],
          "clip_model_missing": ["reward.components.aesthetic=1.0", "reward.kwargs.aesthetic.model_name=null"]}


def _dump(o):
    if dataclasses.is_dataclass(o):
        return {"__class__": type(o).__name__, **{k: _dump(getattr(o, k)) for k in o.__dataclass_fields__}}
    if isinstance(o, dict):
        return {str(k): _dump(v) for k, v in o.items()}
    if isinstance(o, (list, tuple)):
        return [_dump(v) for v in o]
    if isinstance(o, (str, int, float, bool)) or o is None:
        return o
    return str(type(o).__name__)


@pytest.mark.parametrize("name", sorted(k for k in GOLDEN if not k.startswith("break/")))
def test_typed_configs_of_the_experiment_match(name):
    built = L.build_configs(L.load_config(f"experiment/{name}"))
    assert _dump({k: v for k, v in built.items() if k != "raw"}) == GOLDEN[name]


@pytest.mark.parametrize("case", sorted(BREAKS))
def test_a_broken_config_ends_the_same_way(case):
    try:
        L.build_configs(L.load_config("experiment/sd3_5_ocr_grpo", overrides=BREAKS[case]))
        outcome = "accepted"
    except Exception as exc:  # noqa: BLE001 - the outcome is what is compared
        outcome = type(exc).__name__ + ": " + str(exc)[:160]
    assert outcome == GOLDEN["break/" + case]
