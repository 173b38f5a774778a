"""The Cosmos video, NextStep-1 continuous-token and Wan Diffusion-DPO recipes through the public
entry point on CPU, each with its architecture shrunk to a few thousand parameters by overrides.
Every stage of the real recipe runs: config composition, model build with LoRA, rollout (or pair
loading), reward, advantages, replay, loss, optimizer step, metrics file and checkpoint."""

import asyncio
import csv
import inspect
import json
import math

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.scripts.train import run_config


def _train(cfg):
    result = run_config(cfg)
    if inspect.isawaitable(result):
        asyncio.new_event_loop().run_until_complete(result)


TINY_VIDEO_ARCH = [
    "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2", "model.arch.ffn_dim=128",
    "model.arch.text_dim=32", "model.arch.freq_dim=32",
    "sampling.num_frames=5", "sampling.height=32", "sampling.width=32", "sampling.max_sequence_length=8",
    "actor.bf16=false",
]
TINY_VIT_REWARD = [
    "reward.components.vit_scalar=1.0", "reward.kwargs.vit_scalar.preset=vit_tiny", "reward.kwargs.vit_scalar.seed=0",
    "data.manifest=synthetic:8:0", "distributed.rollout.gpus_per_worker=0",
]


def _rows(out):
    rows = list(csv.reader((out / "metrics.csv").open()))
    return rows[0], rows[1:]


def _finite(header, row, names):
    return all(math.isfinite(float(row[header.index(n)])) for n in names)


@pytest.mark.timeout(600)
def test_cosmos_video_recipe_trains_on_cpu(tmp_path):
    out = tmp_path / "cosmos"
    _train(load_config("experiment/cosmos_predict2_2b_grpo", overrides=TINY_VIDEO_ARCH + TINY_VIT_REWARD + [
        "model.random_init=true", "+model.dtype=float32", "model.lora.rank=4", "model.lora.alpha=8",
        "sampling.num_steps=3", "rollout.n=2", "rollout.rollout_batch_size=1", "rollout.sample_batch_size=2",
        "trainer.total_epochs=2", f"trainer.output_dir={out}", "trainer.save_freq=1",
        "reward.components.aesthetic=0.0", "reward.kwargs.vit_scalar.num_frames=2",
        "eval.sanity_gates.enable=false"]))
    header, rows = _rows(out)
    assert len(rows) == 2
    assert all(_finite(header, r, ("loss", "reward_mean", "grad_norm")) for r in rows)
    assert float(rows[0][header.index("grad_norm")]) > 0
    meta = json.loads((out / "checkpoint-final" / "checkpoint_meta.json").read_text())
    assert meta["family"] == "cosmos" and meta["next_epoch"] == 2
    # every periodic checkpoint carries one middle-frame sample per evaluation prompt (here the
    # first four training prompts, the held-out file of the config does not exist); the final one none
    for name in ("checkpoint-1", "checkpoint-2"):
        frames = sorted(p.name for p in (out / name / "eval_samples").glob("*.png"))
        assert len(frames) == 4 and all(f.startswith(f"prompt_{i}_score_") for i, f in enumerate(frames))
    assert not (out / "checkpoint-final" / "eval_samples").exists()
    payload = torch.load(out / "checkpoint-final" / "checkpoint.pt", map_location="cpu", weights_only=False)
    trained = payload["model"]["trainable_modules"]
    assert trained and all(any("lora" in k for k in sd) for sd in trained.values())


@pytest.mark.timeout(600)
def test_nextstep_continuous_token_recipe_trains_on_cpu(tmp_path):
    out = tmp_path / "nextstep"
    _train(load_config("experiment/nextstep_1_ocr_grpo", overrides=TINY_VIT_REWARD + [
        "model.random_init=true", "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
        "model.arch.ffn_dim=128", "model.arch.vocab_size=128", "model.arch.token_dim=16",
        "model.arch.head_hidden=32", "model.arch.head_layers=2", "+model.arch.token_patch=2",
        "+model.arch.vae_base=8", "+model.arch.vae_mults=[1,2]", "+model.arch.vae_blocks=1",
        "model.dtype=float32", "model.lora.rank=4", "model.lora.alpha=8",
        "sampling.image_size=16", "sampling.image_token_num=4", "sampling.num_flow_steps=3",
        "rollout.n_samples_per_prompt=2", "rollout.rollout_batch_size=2", "rollout.max_text_length=8",
        "trainer.total_epochs=2", f"trainer.output_dir={out}", "trainer.save_freq=0", "actor.bf16=false",
        "reward.components.ocr=0.0", "reward.kwargs.vit_scalar.num_frames=1"]))
    header, rows = _rows(out)
    assert len(rows) == 2 and "r_vit_scalar" in header
    assert all(_finite(header, r, ("loss", "reward_mean", "grad_norm", "approx_kl")) for r in rows)
    assert float(rows[0][header.index("grad_norm")]) > 0
    assert float(rows[0][header.index("group_size")]) == 2
    perf = [json.loads(line) for line in (out / "perf.jsonl").read_text().splitlines()]
    assert len(perf) == 2 and all(p["samples"] == 4 for p in perf)
    assert (out / "checkpoint-final" / "checkpoint.pt").exists()


@pytest.mark.timeout(600)
def test_wan_diffusion_dpo_recipe_trains_on_cpu(tmp_path):
    out = tmp_path / "dpo"
    _train(load_config("experiment/wan_2_1_1_3b_shape_dpo", overrides=TINY_VIDEO_ARCH + [
        "model.dtype=float32", "sampling.num_steps=4", "trainer.max_train_steps=3",
        f"trainer.output_dir={out}", "data.synthetic.num_pairs=4"]))
    header, rows = _rows(out)
    assert header[:4] == ["step", "loss", "raw_model_loss", "raw_ref_loss"]
    assert [r[0] for r in rows] == ["1", "2", "3"]
    assert all(_finite(header, r, ("loss", "model_diff", "ref_diff", "grad_norm")) for r in rows)
    # the adapters start at zero, so policy and frozen reference agree on the first step and the
    # preference loss is exactly log 2
    first = rows[0]
    assert float(first[header.index("loss")]) == pytest.approx(math.log(2.0), abs=1e-5)
    assert float(first[header.index("model_diff")]) == pytest.approx(float(first[header.index("ref_diff")]), abs=1e-6)
    assert float(first[header.index("grad_norm")]) > 0
    assert (out / "checkpoint-final" / "checkpoint.pt").exists()


COSMOS_TINY = TINY_VIDEO_ARCH + TINY_VIT_REWARD + [
    "model.random_init=true", "+model.dtype=float32", "model.lora.rank=4", "model.lora.alpha=8",
    "sampling.num_steps=3", "rollout.n=2", "rollout.rollout_batch_size=1", "rollout.sample_batch_size=2",
    "trainer.total_epochs=1", "trainer.save_freq=0", "reward.components.aesthetic=0.0",
    "reward.kwargs.vit_scalar.num_frames=2"]


@pytest.mark.timeout(600)
def test_cosmos_sanity_gates_adapter_export_and_eval_only_comparison(tmp_path):
    out = tmp_path / "cosmos"
    # epoch 0 replays its own rollout: ratio 1, nothing clipped, so the default gates let it pass
    _train(load_config("experiment/cosmos_predict2_2b_grpo", overrides=COSMOS_TINY + [
        f"trainer.output_dir={out}", "eval.sanity_gates.enable=true"]))
    export = out / "checkpoint-final" / "lora_weights"
    assert (export / "adapter_model.safetensors").exists()
    config = json.loads((export / "adapter_config.json").read_text())
    assert config["peft_type"] == "LORA" and config["r"] == 4 and config["lora_alpha"] == 8.0
    assert any(name.endswith("self_attn.qkv") for name in config["target_modules"])

    # a gate that cannot be met stops the run after epoch 0 and says which metric tripped it
    with pytest.raises(RuntimeError, match="epoch-0 sanity gate: approx_kl"):
        _train(load_config("experiment/cosmos_predict2_2b_grpo", overrides=COSMOS_TINY + [
            f"trainer.output_dir={tmp_path / 'gated'}", "eval.sanity_gates.enable=true",
            "eval.sanity_gates.approx_kl_threshold=-1.0"]))

    # eval-only needs an adapter to evaluate
    prompts = tmp_path / "eval_prompts.txt"
    prompts.write_text("a fox\na boat\n")
    eval_overrides = COSMOS_TINY + [f"trainer.output_dir={out}", "eval.eval_only=true",
                                    f"eval.prompts_file={prompts}", "eval.seeds=2"]
    with pytest.raises(ValueError, match="model.lora.path"):
        _train(load_config("experiment/cosmos_predict2_2b_grpo", overrides=eval_overrides))

    _train(load_config("experiment/cosmos_predict2_2b_grpo",
                       overrides=eval_overrides + [f"model.lora.path={export}"]))
    rows = list(csv.DictReader((out / "eval_only" / "eval_results.csv").open()))
    assert [(r["prompt"], r["seed"]) for r in rows] == [("a fox", "0"), ("a fox", "1"), ("a boat", "0"), ("a boat", "1")]
    assert all(abs(float(r["lora_score"]) - float(r["base_score"]) - float(r["delta"])) < 2e-4 for r in rows)
    frames = sorted(p.name for p in (out / "eval_only").glob("*.png"))
    assert len(frames) == 8 and sum(n.startswith("lora_prompt_") for n in frames) == 4
    # the base pass really ran without the adapter: the trained adapter moves the reward a little
    hist = (out / "eval_only" / "eval_results.csv").read_text()
    assert hist.count("\n") == 5
    # no metrics row was added: nothing was trained
    assert len((out / "metrics.csv").read_text().splitlines()) == 2


@pytest.mark.timeout(600)
def test_sd3_ocr_recipe_with_an_engine_named_in_the_config(tmp_path):
    """The OCR reward reads generated images through whatever engine ``reward.kwargs.ocr.engine``
    names (none ships offline).  The rollout runs on the in-process worker of the Ray-style
    backend, which holds its own build of the policy: the first replay must still reproduce the
    rollout's log-probabilities exactly, so nothing is clipped and the KL estimate is zero."""
    from tests.rewards import ocr_engines

    ocr_engines.CALLS.clear()
    out = tmp_path / "ocr"
    _train(load_config("experiment/sd3_5_ocr_grpo", overrides=TINY_VIT_REWARD[3:] + [
        "model.random_init=true", "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
        "model.arch.context_dim=32", "model.arch.pooled_dim=32", "model.arch.in_channels=4", "+model.dtype=float32",
        "model.lora.rank=4", "model.lora.alpha=8", "sampling.height=32", "sampling.width=32",
        "sampling.max_sequence_length=8", "sampling.num_steps=3", "actor.bf16=false", "rollout.n=2",
        "rollout.rollout_batch_size=2", "rollout.sample_batch_size=2", "trainer.total_epochs=1",
        "trainer.save_freq=0", f"trainer.output_dir={out}",
        "reward.kwargs.ocr.engine=tests.rewards.ocr_engines:reads_amber"]))
    header, rows = _rows(out)
    assert header[-1] == "r_ocr" and len(rows) == 1
    row = dict(zip(header, rows[0]))
    assert float(row["clip_fraction"]) == 0.0 and float(row["approx_kl"]) < 1e-9
    assert 0.0 <= float(row["r_ocr"]) <= 1.0 and float(row["reward_mean"]) == pytest.approx(float(row["r_ocr"]), abs=1e-4)
    # one frame per generated image went through the engine: 2 prompts x 2 samples, 32 x 32 RGB
    assert len(ocr_engines.CALLS) == 4 and set(ocr_engines.CALLS) == {(32, 32, 3)}


@pytest.mark.timeout(600)
def test_wan_multi_reward_recipe_mixes_its_components(tmp_path):
    out = tmp_path / "multi"
    _train(load_config("experiment/wan_2_1_1_3b_multi_reward_grpo", overrides=TINY_VIDEO_ARCH + [
        "model.random_init=true", "model.dtype=float32", "model.lora.rank=4", "model.lora.alpha=8",
        "model.arch.in_channels=4", "sampling.num_steps=3", "rollout.n=2", "rollout.rollout_batch_size=2",
        "rollout.sample_batch_size=2", "trainer.total_epochs=1", "trainer.save_freq=0",
        f"trainer.output_dir={out}", "reward.kwargs.aesthetic.model_name=random:vit_tiny",
        "reward.kwargs.clipscore.model_name=random:vit_tiny", "data.manifest=synthetic:8:0",
        "distributed.rollout.gpus_per_worker=0"]))
    header, rows = _rows(out)
    # the zero-weight OCR slot of the config is dropped; the other two are logged one column each
    assert header[-2:] == ["r_aesthetic", "r_clipscore"]
    row = dict(zip(header, rows[0]))
    mixed = 0.5 * float(row["r_aesthetic"]) + 0.5 * float(row["r_clipscore"])
    assert float(row["reward_mean"]) == pytest.approx(mixed, abs=2e-4)
    assert float(row["clip_fraction"]) == 0.0 and float(row["grad_norm"]) > 0


@pytest.mark.timeout(600)
def test_janus_ocr_recipe_runs_through_its_own_entry_point(tmp_path):
    from tests.rewards import ocr_engines

    ocr_engines.CALLS.clear()
    out = tmp_path / "janus_ocr"
    cfg = load_config("experiment/janus_pro_1b_ocr_grpo", overrides=[
        "model.random_init=true", "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
        "model.arch.ffn_dim=128", "model.arch.vocab_size=128", "model.arch.image_vocab_size=96",
        "model.arch.codebook_dim=8", "+model.arch.vq_base=16", "+model.arch.vq_mults=[1,2]",
        "+model.arch.vq_blocks=1", "model.dtype=float32", "model.lora.rank=4", "model.lora.alpha=8",
        "model.int4_decode=false", "sampling.image_token_num=9", "sampling.image_size=32",
        "rollout.n_samples_per_prompt=2", "rollout.rollout_batch_size=2", "rollout.max_text_length=8",
        "actor.bf16=false", "trainer.total_epochs=1", "trainer.save_freq=0", f"trainer.output_dir={out}",
        "reward.kwargs.ocr.engine=tests.rewards.ocr_engines:reads_amber", "data.manifest=synthetic:8:0",
        "distributed.rollout.gpus_per_worker=0"])
    assert cfg.trainer.entrypoint.endswith(":train_janus_pro_ocr_grpo")
    _train(cfg)
    header, rows = _rows(out)
    row = dict(zip(header, rows[0]))
    assert header[-1] == "r_ocr" and float(row["clip_fraction"]) == 0.0 and float(row["approx_kl"]) < 1e-9
    assert len(ocr_engines.CALLS) == 4
    assert (out / "checkpoint-final" / "lora_weights" / "adapter_model.safetensors").exists()


@pytest.mark.timeout(600)
def test_wan_dpo_recipe_on_a_local_dataset_in_the_pickapic_schema(tmp_path):
    """The pixel path of the DPO recipe: a parquet directory with the Pick-a-Pic columns
    (``jpg_0``, ``jpg_1``, ``label_0``, ``caption``) is read through ``datasets``, ties are dropped,
    images are resized / cropped / normalised, encoded by the frozen encoder and trained on."""
    datasets = pytest.importorskip("datasets")
    pytest.importorskip("torchvision")
    import io

    import numpy as np
    from PIL import Image

    from visionrl_b200.trainers.pickapic import load_pickapic

    rng = np.random.default_rng(0)

    def jpg():
        buf = io.BytesIO()
        Image.fromarray(rng.integers(0, 255, (40, 48, 3), dtype=np.uint8)).save(buf, format="JPEG")
        return buf.getvalue()

    root = tmp_path / "pairs"
    root.mkdir()
    datasets.Dataset.from_dict({"jpg_0": [jpg() for _ in range(6)], "jpg_1": [jpg() for _ in range(6)],
                                "label_0": [1, 0, 0.5, 1, 0, 1],
                                "caption": [f"caption {i}" for i in range(6)]}).to_parquet(str(root / "train.parquet"))
    pairs = load_pickapic(dataset_name=str(root), resolution=32, no_hflip=True)
    assert len(pairs) == 5                                                # the tie is gone
    item = pairs[1]                                                       # label_0 == 0: the second image won
    assert item["pixel_values"].shape == (6, 32, 32) and item["caption"] == "caption 1"
    assert float(item["pixel_values"].min()) >= -1.0 and float(item["pixel_values"].max()) <= 1.0

    out = tmp_path / "dpo_pixels"
    _train(load_config("experiment/wan_2_1_1_3b_dpo", overrides=[
        o for o in TINY_VIDEO_ARCH if "num_frames" not in o] + [
        "model.random_init=true", "model.dtype=float32", "model.lora.rank=4", "model.lora.alpha=8",
        "actor.mixed_precision=no", "sampling.num_steps=4", "trainer.max_train_steps=3",
        "trainer.checkpointing_steps=2", "trainer.log_interval=1", f"trainer.output_dir={out}",
        f"data.dataset_name={root}", "data.dataloader_num_workers=0"]))
    header, rows = _rows(out)
    assert [r[0] for r in rows] == ["1", "2", "3"]
    assert all(_finite(header, r, ("loss", "raw_model_loss", "grad_norm")) for r in rows)
    assert float(rows[0][header.index("loss")]) == pytest.approx(math.log(2.0), abs=1e-5)
    assert sorted(p.name for p in out.glob("checkpoint-*")) == ["checkpoint-2", "checkpoint-final"]
