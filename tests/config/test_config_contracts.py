"""Fail-fast rules of the config layer that the recipes rely on (reference expectations:
``tests/config/test_load_all_experiments.py:106-400``): the entry point comes from the YAML and
nowhere else, resume fields have base defaults and take overrides, model-backed rewards name
their weights explicitly, and the algorithm is chosen by ``algorithm.kind`` alone."""

import pytest

from vrl.config.loader import (CONFIGS_ROOT, build_algorithm_config, build_configs, build_reward_config,
                               load_config, optional_none, validate_reward_config, validate_training_config)
from vrl.config.node import OmegaConf
from vrl.scripts.train import resolve_train_target

EXPERIMENTS = sorted(p.stem for p in (CONFIGS_ROOT / "experiment").glob("*.yaml"))
REQUIRED_REWARD_KWARGS = {"aesthetic": ("model_name",), "clipscore": ("model_name",), "pickscore": ("model_name",)}


def test_entrypoint_must_be_in_the_yaml_and_non_empty():
    with pytest.raises(ValueError, match=r"trainer\.entrypoint"):
        resolve_train_target(OmegaConf.create({"trainer": {}}))
    with pytest.raises(ValueError, match="non-empty"):
        resolve_train_target(OmegaConf.create({"trainer": {"entrypoint": ""}}))
    with pytest.raises(ValueError, match="non-empty"):
        resolve_train_target(OmegaConf.create({"trainer": {"entrypoint": 3}}))
    target = resolve_train_target(OmegaConf.create({"trainer": {"entrypoint": " pkg.mod:fn "}}))
    assert (target.import_path, target.module, target.function) == ("pkg.mod:fn", "pkg.mod", "fn")


def test_resume_fields_come_from_the_base_yaml_and_take_overrides():
    cfg = load_config("experiment/sd3_5_ocr_grpo")
    built = build_configs(cfg)["trainer"]
    assert cfg.trainer.resume_from == "" and cfg.trainer.resume_strict is True
    assert built.resume_from == "" and built.resume_strict is True
    over = load_config("experiment/sd3_5_ocr_grpo", overrides=["trainer.resume_from=/tmp/checkpoint-10",
                                                               "trainer.resume_strict=false"])
    built = build_configs(over)["trainer"]
    assert built.resume_from == "/tmp/checkpoint-10" and built.resume_strict is False


def test_algorithm_is_chosen_by_kind_alone():
    cfg = load_config("experiment/sd3_5_ocr_grpo")
    assert "adv_estimator" not in cfg.algorithm
    assert type(build_algorithm_config(cfg)).__name__ == "GRPOConfig"
    only_estimator = load_config("experiment/sd3_5_ocr_grpo")
    del only_estimator.algorithm["kind"]
    only_estimator.algorithm["adv_estimator"] = "grpo"
    with pytest.raises(ValueError):
        build_algorithm_config(only_estimator)


@pytest.mark.parametrize("experiment,component", [("wan_2_1_1_3b_grpo", "aesthetic"), ("janus_pro_1b_grpo", "pickscore")])
def test_model_backed_rewards_must_name_their_model(experiment, component):
    cfg = load_config(f"experiment/{experiment}")
    assert float(cfg.reward.components.get(component, 0.0)) > 0
    del cfg.reward.kwargs[component]["model_name"]
    with pytest.raises(ValueError) as err:
        validate_reward_config(cfg)
    assert component in str(err.value) and "model_name" in str(err.value)


@pytest.mark.parametrize("name", EXPERIMENTS)
def test_every_experiment_validates_and_spells_out_reward_kwargs(name):
    cfg = load_config(f"experiment/{name}")
    validate_training_config(cfg)
    if "reward" not in cfg:
        return
    assert "ocr_debug_dir" not in cfg.reward                          # lives under reward.kwargs.ocr.debug_dir
    weights, kwargs = build_reward_config(cfg)
    for component, needed in REQUIRED_REWARD_KWARGS.items():
        if component in weights:
            assert isinstance(kwargs.get(component), dict)
            for key in needed:
                assert key in kwargs[component], f"{name}: reward.kwargs.{component}.{key}"


def test_dpo_accepts_an_explicit_null_sample_cap_but_needs_a_step_budget():
    cfg = load_config("experiment/wan_2_1_1_3b_dpo")
    cfg.data.max_train_samples = None
    assert optional_none(cfg, "data.max_train_samples") is None
    validate_training_config(cfg)
    del cfg.trainer["max_train_steps"]
    with pytest.raises(ValueError, match=r"trainer\.max_train_steps"):
        validate_training_config(cfg)


EXPECTED_PATHS = {
    "cosmos_predict2_2b_grpo": ("datasets/drawbench/train_192.txt", "outputs/cosmos_pred2_2b_grpo"),
    "janus_pro_1b_grpo": ("datasets/janus/prompts.txt", "outputs/janus_pro_1b_grpo"),
    "janus_pro_1b_ocr_grpo": ("datasets/ocr/train.txt", "outputs/janus_pro_1b_ocr_grpo"),
    "nextstep_1_ocr_grpo": ("datasets/ocr/train.txt", "outputs/nextstep_1_ocr_grpo"),
    "sd3_5_ocr_grpo": ("datasets/ocr/train.txt", "outputs/sd3_5_ocr_grpo"),
    "wan_2_1_14b_grpo": ("datasets/wan/prompts.txt", "outputs/wan_14b_grpo"),
    "wan_2_1_1_3b_dpo": (None, "outputs/wan_1_3b_dpo"),
    "wan_2_1_1_3b_grpo": ("datasets/wan/prompts.txt", "outputs/wan_1_3b_grpo"),
    "wan_2_1_1_3b_multi_reward_grpo": ("datasets/wan/prompts.txt", "outputs/wan_1_3b_multi_reward_grpo"),
    "wan_2_1_1_3b_ocr_grpo": ("datasets/ocr/train.txt", "outputs/wan_1_3b_ocr_grpo"),
}


@pytest.mark.parametrize("name", sorted(EXPECTED_PATHS))
def test_experiments_name_the_manifest_and_output_directory_of_their_recipe(name):
    cfg = load_config(f"experiment/{name}")
    manifest, out = EXPECTED_PATHS[name]
    data = cfg.get("data")
    assert (data.get("manifest") if data is not None else None) == manifest
    assert cfg.trainer.output_dir == out


def test_every_experiment_has_a_plain_output_directory_and_a_textual_manifest():
    import re
    from pathlib import Path

    from visionrl_b200.config.loader import CONFIGS_ROOT

    for file in sorted(Path(CONFIGS_ROOT, "experiment").glob("*.yaml")):
        cfg = load_config(f"experiment/{file.stem}")
        assert re.fullmatch(r"outputs/\w+", str(cfg.trainer.output_dir)), file.stem
        manifest = cfg.get("data").get("manifest") if cfg.get("data") is not None else None
        assert manifest is None or (isinstance(manifest, str) and re.fullmatch(r"(synthetic:\d+(:\d+)?|[\w./-]+\.(txt|jsonl))",
                                                                               manifest)), (file.stem, manifest)


def test_shipped_manifests_exist_and_parse():
    from pathlib import Path

    from visionrl_b200.config.loader import CONFIGS_ROOT
    from visionrl_b200.trainers.data import load_prompt_manifest

    repo = Path(CONFIGS_ROOT).parent
    not_shipped = {"datasets/drawbench/train_192.txt"}            # a published prompt set, see datasets/README.md
    seen = set()
    for file in sorted(Path(CONFIGS_ROOT, "experiment").glob("*.yaml")):
        data = load_config(f"experiment/{file.stem}").get("data")
        manifest = data.get("manifest") if data is not None else None
        if manifest is None or manifest.startswith("synthetic:") or manifest in not_shipped:
            continue
        seen.add(manifest)
        examples = load_prompt_manifest(repo / manifest)
        assert len(examples) >= 32 and all(e.prompt for e in examples), manifest
        if "/ocr/" in manifest:
            assert all(e.target_text and e.target_text in e.prompt for e in examples)
    assert seen == {"datasets/ocr/train.txt", "datasets/wan/prompts.txt", "datasets/janus/prompts.txt"}
