"""Every experiment YAML loads, validates and dispatches to the right typed configs."""

from pathlib import Path

import pytest

from vrl.algorithms.dpo import DiffusionDPOConfig
from vrl.algorithms.grpo import GRPOConfig
from vrl.algorithms.grpo_token import TokenGRPOConfig
from vrl.config.loader import (
    CONFIGS_ROOT, build_algorithm_config, build_configs, build_reward_config, load_config,
    optional_none, require, validate_training_config,
)
from vrl.scripts.train import _import_callable, build_parser, resolve_train_target, run_config
from vrl.trainers.types import TrainerConfig

EXPERIMENTS = sorted(p.stem for p in (CONFIGS_ROOT / "experiment").glob("*.yaml"))
KIND_TO_CLASS = {"grpo": GRPOConfig, "token_grpo": TokenGRPOConfig, "diffusion_dpo": DiffusionDPOConfig}
ENTRYPOINTS = {
    "sd3_5_ocr_grpo": "vrl.scripts.sd3_5.train:train_sd3_5_grpo",
    "wan_2_1_1_3b_grpo": "vrl.scripts.wan_2_1.train:train_wan_2_1_grpo",
    "wan_2_1_14b_grpo": "vrl.scripts.wan_2_1.train:train_wan_2_1_grpo",
    "wan_2_1_1_3b_dpo": "vrl.scripts.wan_2_1.train_dpo:train_wan_2_1_dpo",
    "cosmos_predict2_2b_grpo": "vrl.scripts.cosmos.train:train_cosmos_predict2_grpo",
    "janus_pro_1b_grpo": "vrl.scripts.janus_pro.train:train_janus_pro_grpo",
    "janus_pro_1b_ocr_grpo": "vrl.scripts.janus_pro.train:train_janus_pro_ocr_grpo",
    "nextstep_1_ocr_grpo": "vrl.scripts.nextstep_1.train:train_nextstep_1_ocr_grpo",
}


def test_reference_experiment_set_is_present():
    assert set(ENTRYPOINTS) <= set(EXPERIMENTS)
    assert {"tiny_dit_grpo", "sd3_5_shape_grpo", "wan_2_1_1_3b_shape_grpo", "wan_2_1_14b_shape_grpo",
            "janus_pro_1b_shape_grpo", "wan_2_1_1_3b_shape_dpo"} <= set(EXPERIMENTS)


@pytest.mark.parametrize("name", EXPERIMENTS)
def test_experiment_loads_validates_and_dispatches(name):
    cfg = load_config(f"experiment/{name}")
    built = build_configs(cfg)
    assert isinstance(built["trainer"], TrainerConfig)
    kind = cfg.algorithm.kind
    assert type(built["algorithm"]) is KIND_TO_CLASS[kind]
    target = resolve_train_target(cfg)
    assert callable(_import_callable(target.import_path))
    if name in ENTRYPOINTS:
        assert target.import_path == ENTRYPOINTS[name]
    if "reward" in cfg:
        weights, kwargs = built["reward"]
        assert weights and all(w > 0 for w in weights.values())


def test_sd3_max_sequence_length_and_cli_override_reach_typed_config():
    cfg = load_config("experiment/sd3_5_ocr_grpo", ["actor.optim.lr=3e-5", "trainer.seed=7"])
    assert cfg.sampling.max_sequence_length == 128
    tc = build_configs(cfg)["trainer"]
    assert tc.optim.lr == pytest.approx(3e-5) and tc.seed == 7


@pytest.mark.parametrize("name,path", [
    ("sd3_5_ocr_grpo", "trainer.output_dir"), ("sd3_5_ocr_grpo", "actor.optim.lr"),
    ("nextstep_1_ocr_grpo", "rollout.noise_level"), ("wan_2_1_1_3b_dpo", "trainer.max_train_steps"),
    ("sd3_5_ocr_grpo", "rollout.sde.type"), ("janus_pro_1b_grpo", "rollout.max_text_length"),
])
def test_missing_required_field_names_the_dotted_path(name, path):
    cfg = load_config(f"experiment/{name}")
    node = cfg
    keys = path.split(".")
    for k in keys[:-1]:
        node = node[k]
    del node[keys[-1]]
    with pytest.raises(ValueError, match=path.replace(".", r"\.")):
        validate_training_config(cfg)


def test_algorithm_kind_rules():
    cfg = load_config("experiment/sd3_5_ocr_grpo")
    cfg.algorithm["adv_estimator"] = "grpo"
    with pytest.raises(ValueError, match="adv_estimator"):
        build_algorithm_config(cfg)
    del cfg.algorithm["adv_estimator"]
    cfg.algorithm.kind = "ppo"
    with pytest.raises(ValueError, match="unknown algorithm.kind"):
        build_algorithm_config(cfg)
    cfg.rollout.sde.type = "ode"
    cfg.algorithm.kind = "grpo"
    with pytest.raises(ValueError, match="sde.type"):
        validate_training_config(cfg)


def test_reward_validation():
    cfg = load_config("experiment/wan_2_1_1_3b_multi_reward_grpo")
    weights, kwargs = build_reward_config(cfg)
    assert weights == {"aesthetic": 0.5, "clipscore": 0.5} and "ocr" not in weights
    del cfg.reward.kwargs.clipscore["model_name"]
    with pytest.raises(ValueError, match=r"reward\.kwargs\.clipscore\.model_name"):
        build_reward_config(cfg)
    cfg.reward.components["aesthetic"] = "high"
    with pytest.raises(ValueError, match="numeric"):
        build_reward_config(cfg)


def test_require_and_optional_none():
    cfg = load_config("experiment/wan_2_1_1_3b_dpo")
    assert optional_none(cfg, "data.max_train_samples") is None
    with pytest.raises(ValueError, match="got None"):
        require(cfg, "data.max_train_samples")
    with pytest.raises(ValueError, match="data.nope"):
        optional_none(cfg, "data.nope")
    assert require(cfg, "rollout.n") == 1


def test_defaults_overlay_features(tmp_path):
    (tmp_path / "a.yaml").write_text("x: {p: 1, q: 2}\nlist: [1, 2]\n")
    (tmp_path / "grp").mkdir()
    (tmp_path / "grp" / "b.yaml").write_text("x: {q: 3}\nref: ${x.p}\n")
    (tmp_path / "top.yaml").write_text(
        "defaults:\n  - /a\n  - {grp: b}\nx: {r: 4}\nlist: [9]\nlr: 1e-4\n")
    cfg = load_config(tmp_path / "top.yaml", root=tmp_path, overrides=["x.p=7", "new.key=[1,2]"])
    assert cfg.x == {"p": 7, "q": 3, "r": 4} and cfg.list == [9] and cfg.ref == 7
    assert cfg.new.key == [1, 2] and isinstance(cfg.lr, float)
    (tmp_path / "self_first.yaml").write_text("defaults:\n  - _self_\n  - /a\nx: {p: 100}\n")
    assert load_config(tmp_path / "self_first.yaml", root=tmp_path).x.p == 1
    (tmp_path / "c1.yaml").write_text("defaults: [/c2]\n")
    (tmp_path / "c2.yaml").write_text("defaults: [/c1]\n")
    with pytest.raises(RuntimeError, match="Cyclic"):
        load_config(tmp_path / "c1.yaml", root=tmp_path)


def test_cli_layer_has_no_family_or_kind_dispatch():
    source = Path(__import__("visionrl_b200.scripts.train", fromlist=["x"]).__file__).read_text()
    for word in ("sd3_5", "wan_2_1", "cosmos", "janus", "nextstep", "token_grpo", "diffusion_dpo"):
        assert word not in source
    args = build_parser().parse_args(["--config", "experiment/x", "a=1", "b.c=2"])
    assert args.config == "experiment/x" and args.overrides == ["a=1", "b.c=2"]
    with pytest.raises(ValueError, match="module:function"):
        _import_callable("no_colon_here")
    with pytest.raises(ValueError, match="entrypoint"):
        run_config(load_config("base/trainer"))
