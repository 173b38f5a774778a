"""The tiny flow-matching DiT recipe through the public CLI entry on CPU: rollout, reward,
advantages, replay, clipped loss with LoRA-off reference KL, optimizer step, CSV, checkpoints,
resume.  This is the always-on end-to-end check of the whole stack."""

import asyncio
import csv
import inspect
import json

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.scripts.train import run_config


def _train(cfg):
    result = run_config(cfg)
    if inspect.isawaitable(result):
        asyncio.new_event_loop().run_until_complete(result)


def _overrides(out, **extra):
    base = {
        "trainer.output_dir": str(out), "trainer.total_epochs": 2, "trainer.save_freq": 1,
        "sampling.num_steps": 4, "rollout.n": 2, "rollout.rollout_batch_size": 2,
        "rollout.sample_batch_size": 2, "distributed.rollout.gpus_per_worker": 0,
    }
    base.update(extra)
    return [f"{k}={v}" for k, v in base.items()]


@pytest.mark.timeout(600)
def test_tiny_dit_grpo_trains_checkpoints_and_resumes(tmp_path, caplog):
    out = tmp_path / "run"
    caplog.set_level("INFO")
    _train(load_config("experiment/tiny_dit_grpo", overrides=_overrides(out)))

    rows = list(csv.reader((out / "metrics.csv").open()))
    assert rows[0][:6] == ["epoch", "loss", "policy_loss", "kl_penalty", "reward_mean", "reward_std"]
    assert [r[0] for r in rows[1:]] == ["0", "1"]
    assert all(torch.isfinite(torch.tensor(float(v))) for r in rows[1:] for v in r[1:10])
    assert (out / "resolved_config.yaml").exists()
    # one performance line per epoch, apart from the fixed-column CSV
    perf = [json.loads(line) for line in (out / "perf.jsonl").read_text().splitlines()]
    assert [p["epoch"] for p in perf] == [0, 1]
    assert all(p["step_ms"] > 0 and p["samples"] == 4 and p["samples_per_sec"] > 0 and p["n_ranks"] == 1
               for p in perf)
    for name in ("checkpoint-1", "checkpoint-final"):
        assert (out / name / "checkpoint.pt").exists() and (out / name / "checkpoint_meta.json").exists()
        # the adapters are also exported by themselves, loadable through model.lora.path
        assert (out / name / "lora_weights" / "adapter_model.safetensors").exists()
        assert (out / name / "lora_weights" / "adapter_config.json").exists()
    meta = json.loads((out / "checkpoint-final" / "checkpoint_meta.json").read_text())
    assert meta["family"] == "sd3_5" and meta["next_epoch"] == 2 and meta["schema_version"] == 1
    payload = torch.load(out / "checkpoint-final" / "checkpoint.pt", map_location="cpu", weights_only=False)
    assert set(payload["model"]["trainable_modules"]) == {"transformer"}
    keys = list(payload["model"]["trainable_modules"]["transformer"])
    assert keys and all("lora" in k for k in keys if "lora" in k)
    assert "optimizer" in payload["trainer"]

    # the rollout log-probability is reproduced exactly by the first replay
    first_step = [r.message for r in caplog.records if "first-step" in r.message.lower()
                  or "first_step" in r.message.lower()]
    assert first_step, "debug.first_step should log the rollout/replay log-prob difference"

    # resume for one more epoch: CSV is appended, the resolved config of the first run is kept
    _train(load_config("experiment/tiny_dit_grpo", overrides=_overrides(
        out, **{"trainer.total_epochs": 3, "trainer.resume_from": str(out / "checkpoint-final")})))
    rows = list(csv.reader((out / "metrics.csv").open()))
    assert [r[0] for r in rows[1:]] == ["0", "1", "2"]
    assert len(list(out.glob("resume_config_*.yaml"))) == 1
