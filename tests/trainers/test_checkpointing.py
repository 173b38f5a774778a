"""Checkpoint format and resume helpers (reference expectations:
``tests/trainers/test_checkpointing.py:20-125`` and ``tests/scripts/test_sd3_resume.py:16-77``)."""

import json
from types import SimpleNamespace

import pytest
import torch
from torch import nn

from visionrl_b200.config.node import OmegaConf
from visionrl_b200.trainers import checkpointing as ck


class _Trainer:
    def __init__(self):
        self.state = {"step": 3, "global_step": 12, "total_reward": 1.5, "total_loss": 0.25}
        self.loaded = None

    def state_dict(self):
        return dict(self.state)

    def load_state_dict(self, state, *, strict=True):
        self.loaded = (dict(state), strict)


def _bundle(seed=0, family="sd3_5"):
    torch.manual_seed(seed)
    return SimpleNamespace(trainable_modules={"transformer": nn.Linear(3, 2)}, metadata={"family": family})


class _LoraExport:
    def save_pretrained(self, path):
        path.mkdir(parents=True, exist_ok=True)
        (path / "adapter_config.json").write_text("{}")


def test_round_trip_files_keys_and_state(tmp_path):
    trainer, bundle = _Trainer(), _bundle(0)
    meta = ck.save_training_checkpoint(
        tmp_path / "checkpoint-3", trainer=trainer, bundle=bundle, family="sd3_5",
        progress={"completed_epoch": 2, "next_epoch": 3, "global_step": 12},
        export_modules={ck.LORA_WEIGHTS_NAME: _LoraExport()})
    d = tmp_path / "checkpoint-3"
    assert (d / "checkpoint.pt").exists() and (d / "checkpoint_meta.json").exists()
    assert (d / "lora_weights" / "adapter_config.json").exists()
    on_disk = json.loads((d / "checkpoint_meta.json").read_text())
    assert on_disk == meta
    assert {"schema_version", "family", "trainer_step", "global_step", "completed_epoch", "next_epoch",
            "uses_lora", "checkpoint_file"} <= set(on_disk)
    assert on_disk["uses_lora"] is True and on_disk["checkpoint_file"] == "checkpoint.pt"

    payload = torch.load(d / "checkpoint.pt", map_location="cpu", weights_only=False)
    assert payload["schema_version"] == 1 and payload["family"] == "sd3_5"
    assert set(payload) == {"schema_version", "family", "trainer", "model", "progress", "rng"}
    assert set(payload["model"]["trainable_modules"]) == {"transformer"}
    assert {"torch", "python_random", "numpy"} <= set(payload["rng"])

    loaded = ck.load_training_checkpoint(d)
    assert loaded.next_epoch == 3
    other_trainer, other = _Trainer(), _bundle(1)
    assert not torch.equal(other.trainable_modules["transformer"].weight,
                           bundle.trainable_modules["transformer"].weight)
    ck.restore_training_checkpoint(loaded, trainer=other_trainer, bundle=other)
    assert torch.equal(other.trainable_modules["transformer"].weight,
                       bundle.trainable_modules["transformer"].weight)
    assert other_trainer.loaded[0]["global_step"] == 12 and other_trainer.loaded[1] is True
    # the file itself is an accepted path too
    assert ck.load_training_checkpoint(d / "checkpoint.pt").payload["family"] == "sd3_5"


def test_missing_file_bad_schema_and_key_mismatch(tmp_path):
    with pytest.raises(FileNotFoundError):
        ck.load_training_checkpoint(tmp_path / "nope")
    bad = tmp_path / "bad"
    bad.mkdir()
    torch.save({"schema_version": 99}, bad / "checkpoint.pt")
    with pytest.raises(ValueError):
        ck.load_training_checkpoint(bad)
    trainer, bundle = _Trainer(), _bundle()
    ck.save_training_checkpoint(tmp_path / "c", trainer=trainer, bundle=bundle, family="sd3_5",
                                progress={"next_epoch": 1})
    loaded = ck.load_training_checkpoint(tmp_path / "c")
    wrong = SimpleNamespace(trainable_modules={"other": nn.Linear(3, 2)}, metadata={"family": "sd3_5"})
    with pytest.raises(ValueError):
        ck.restore_training_checkpoint(loaded, trainer=_Trainer(), bundle=wrong)
    other_family = _bundle(family="wan_2_1")
    with pytest.raises(ValueError):
        ck.restore_training_checkpoint(loaded, trainer=_Trainer(), bundle=other_family)


def test_next_epoch_fallbacks_and_meta_type(tmp_path):
    d = tmp_path / "checkpoint-7"
    d.mkdir()
    assert ck.infer_next_epoch(d, {"step": 5}, {}) == 5          # trainer step first
    assert ck.infer_next_epoch(d, {}, {}) == 7                    # then the directory suffix
    with pytest.raises(ValueError):
        ck.infer_next_epoch(tmp_path / "checkpoint-final", {}, {})
    assert ck.infer_next_epoch(d, {"step": 5}, {"next_epoch": 9}) == 9   # explicit meta wins
    (d / "checkpoint_meta.json").write_text("[1, 2]")
    with pytest.raises(TypeError):
        ck.read_checkpoint_meta(d)


def test_prompt_rng_restore_reproduces_next_sample(tmp_path):
    gen = torch.Generator().manual_seed(123)
    ck.sample_prompt_indices(gen, num_examples=50, rollout_batch_size=4)
    state = ck.capture_rng_state(prompt_generator=gen)
    expected = ck.sample_prompt_indices(gen, num_examples=50, rollout_batch_size=4)
    fresh = torch.Generator().manual_seed(999)
    ck.restore_rng_state(state, prompt_generator=fresh)
    assert ck.sample_prompt_indices(fresh, num_examples=50, rollout_batch_size=4) == expected
    with pytest.raises(ValueError):
        ck.sample_prompt_indices(fresh, num_examples=0, rollout_batch_size=4)


def test_metrics_csv_is_appended_not_rewritten_on_resume(tmp_path):
    path = tmp_path / "metrics.csv"
    ck.prepare_metrics_csv(path, "epoch,loss\n", resume=False)
    with path.open("a") as fh:
        fh.write("0,1.0\n")
    ck.prepare_metrics_csv(path, "epoch,loss\n", resume=True)
    assert path.read_text() == "epoch,loss\n0,1.0\n"
    ck.prepare_metrics_csv(path, "epoch,loss\n", resume=False)
    assert path.read_text() == "epoch,loss\n"


def test_strict_resume_conflicts_with_lora_path(tmp_path):
    trainer, bundle = _Trainer(), _bundle()
    ck.save_training_checkpoint(tmp_path / "c", trainer=trainer, bundle=bundle, family="sd3_5",
                                progress={"next_epoch": 1})
    loaded = ck.load_training_checkpoint(tmp_path / "c")
    cfg = OmegaConf.create({"model": {"lora": {"path": "/some/adapter"}},
                            "trainer": {"resume_from": str(tmp_path / "c")}})
    with pytest.raises(ValueError):
        ck.prepare_model_config_for_training_resume(cfg, loaded, strict=True)
    ck.prepare_model_config_for_training_resume(cfg, loaded, strict=False)
    assert not cfg.model.lora.path
    assert ck.load_training_checkpoint_from_config(cfg).payload["family"] == "sd3_5"
    assert ck.load_training_checkpoint_from_config(OmegaConf.create({"trainer": {"resume_from": ""}})) is None


def test_resolved_config_written_and_resume_copy_kept(tmp_path):
    cfg = OmegaConf.create({"a": {"b": 1}})
    ck.save_resolved_config(cfg, tmp_path, resumed=False)
    assert (tmp_path / "resolved_config.yaml").exists()
    ck.save_resolved_config(cfg, tmp_path, resumed=True)
    assert len(list(tmp_path.glob("resume_config_*.yaml"))) == 1


def test_a_checkpoint_written_by_the_reference_implementation_restores_here(tmp_path):
    """``tests/golden/reference_checkpoint`` was written by the reference's own
    ``save_training_checkpoint`` (a 2x2 linear layer seeded with 0, optimiser and averaged state, the
    prompt generator seeded with 123 and advanced by one permutation of five).  It must load, restore
    and continue here exactly as there; and a checkpoint written here carries the same meta file."""
    import json
    import os
    import types

    from torch import nn

    from visionrl_b200.trainers import checkpointing as ck

    golden = os.path.join(os.path.dirname(os.path.dirname(__file__)), "golden", "reference_checkpoint")
    loaded = ck.load_training_checkpoint(golden)
    assert loaded.meta["next_epoch"] == 4 and loaded.meta["family"] == "sd3_5" and loaded.meta["schema_version"] == 1

    class Trainer:
        def load_state_dict(self, state, strict=True):
            self.loaded = state

        def state_dict(self):
            return self.loaded

    trainer, net = Trainer(), nn.Linear(2, 2)
    bundle = types.SimpleNamespace(trainable_modules={"transformer": net}, metadata={"family": "sd3_5"})
    ck.restore_training_checkpoint(loaded, trainer=trainer, bundle=bundle, strict=True)
    torch.manual_seed(0)
    assert torch.equal(net.weight, nn.Linear(2, 2).weight)
    assert sorted(trainer.loaded) == ["ema", "global_step", "optimizer", "step", "total_loss", "total_reward"]
    assert float(trainer.loaded["optimizer"]["state"][0]["exp_avg_sq"][0, 0]) == 2.0
    generator = torch.Generator().manual_seed(0)
    ck.restore_rng_state(loaded.payload["rng"], prompt_generator=generator)
    assert torch.randperm(5, generator=generator).tolist() == [0, 3, 2, 4, 1]

    # written here from the restored pieces: the same meta file, key for key
    ck.save_training_checkpoint(tmp_path / "again", trainer=trainer, bundle=bundle, family="sd3_5",
                                progress={"completed_epoch": 4, "next_epoch": 4, "global_step": 7})
    ours = json.loads((tmp_path / "again" / "checkpoint_meta.json").read_text())
    theirs = json.loads(open(os.path.join(golden, "checkpoint_meta.json")).read())
    assert ours == theirs
