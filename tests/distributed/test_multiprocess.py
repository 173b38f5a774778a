"""Multi-rank behaviour: gloo ranks on CPU (always), NCCL + in-kernel NVLink paths on >= 2 GPUs."""

import socket

import pytest
import torch
import torch.multiprocessing as mp

from tests.distributed import _workers


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(fn, world, *args, timeout=240):
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=fn, args=(r, world, port, *args, out)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    for p in procs:
        if p.is_alive():
            p.kill()
            raise AssertionError("worker timed out")
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    return out.get(timeout=10)


def test_sharded_adamw_gloo_world2():
    res = _run(_workers.sharded_adamw_matches_single, 2, "gloo", "nccl")
    assert res["err"] < 1e-5 and res["same"]
    assert res["state_keys"] == [0, 1, 2, 3]


def test_ulysses_attention_gloo_world2():
    res = _run(_workers.ulysses_attention_matches_dense, 2, "gloo", False)
    assert res["fwd"] and res["bwd"]


@pytest.mark.parametrize("checkpointing", [True, False])
def test_fsdp_gloo_world2_matches_replicated(checkpointing):
    res = _run(_workers.fsdp_training_matches_replicated, 2, "gloo", "nccl", 1, checkpointing)
    assert res["shapes_ok"] and res["err"] < 2e-4 and res["fwd_err"] < 1e-3, res
    assert res["handles"] > 0 and res["buckets"] > 0
    assert res["opt_entries"] == res["params"]
    rep = res["report"]
    assert rep["param_shard_bytes"] * 2 == rep["full_param_bytes"]
    # the rollout replica is republished after every optimiser step and serves no-grad forwards
    assert res["replica_used"] and res["broadcasts"] == 3
    assert rep["rollout_replica_bytes"] == rep["full_param_bytes"]


def test_hsdp_gloo_world4_matches_replicated():
    res = _run(_workers.fsdp_training_matches_replicated, 4, "gloo", "nccl", 2, True)
    assert res["shapes_ok"] and res["err"] < 2e-4 and res["fwd_err"] < 1e-3, res
    rep = res["report"]
    assert rep["param_shard_bytes"] * 2 == rep["full_param_bytes"]      # sharded over 2 of the 4 ranks


@pytest.mark.timeout(600)
@pytest.mark.parametrize("world,sp", [(2, 2), (2, 1), (4, 2)])
def test_wan_recipe_on_cpu_ranks_sharded_with_and_without_sequence_parallelism(tmp_path, world, sp):
    """Public entry point on gloo ranks: DP=1 x SP=2, DP=2 x SP=1 and DP=2 x SP=2, block weights sharded
    over all ranks; train one epoch, checkpoint (rank 0 writes, every rank joins the gathers), resume for
    another.  The first replay reproduces the rollout on every mesh: nothing is clipped."""
    import math

    res = _run(_workers.wan_recipe_runs_sharded_and_sequence_parallel, world, sp, str(tmp_path / f"run_sp{sp}"),
               _free_port(), timeout=500)
    rows, perf = res["rows"], res["perf"]
    assert rows[0][0] == "epoch" and [r[0] for r in rows[1:]] == ["0", "1"]     # one epoch, then one more after resume
    assert all(math.isfinite(float(v)) for r in rows[1:] for v in r[1:10])
    assert len(perf) == 2 and all(p["n_ranks"] == world and p["step_ms"] > 0 for p in perf)
    assert perf[0]["samples"] == 2 * max(1, world // sp)             # group of 2 per prompt, one prompt per DP rank
    first = dict(zip(rows[0], rows[1]))
    assert float(first["clip_fraction"]) == 0.0 and float(first["approx_kl"]) < 1e-9


TINY_JANUS = [
    "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2", "model.arch.ffn_dim=128",
    "model.arch.vocab_size=128", "model.arch.image_vocab_size=96", "model.arch.codebook_dim=8",
    "+model.arch.vq_base=16", "+model.arch.vq_mults=[1,2]", "+model.arch.vq_blocks=1", "model.dtype=float32",
    "model.lora.rank=4", "model.lora.alpha=8", "model.int4_decode=false", "sampling.image_token_num=9",
    "sampling.image_size=32", "rollout.n_samples_per_prompt=4", "rollout.rollout_batch_size=2",
    "rollout.max_text_length=8", "reward.kwargs.vit_scalar.preset=vit_tiny", "actor.bf16=false",
]


TINY_COSMOS = [
    "model.random_init=true", "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
    "model.arch.ffn_dim=128", "model.arch.text_dim=32", "model.arch.freq_dim=32", "+model.dtype=float32",
    "model.lora.rank=4", "model.lora.alpha=8", "sampling.num_frames=5", "sampling.height=32", "sampling.width=32",
    "sampling.max_sequence_length=8", "sampling.num_steps=3", "actor.bf16=false", "rollout.n=2",
    "rollout.rollout_batch_size=2", "rollout.sample_batch_size=2", "reward.components.aesthetic=0.0",
    "reward.components.vit_scalar=1.0", "reward.kwargs.vit_scalar.preset=vit_tiny", "reward.kwargs.vit_scalar.seed=0",
    "reward.kwargs.vit_scalar.num_frames=2", "data.manifest=synthetic:8:0", "distributed.rollout.gpus_per_worker=0",
]
TINY_NEXTSTEP = [
    "model.random_init=true", "model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
    "model.arch.ffn_dim=128", "model.arch.vocab_size=128", "model.arch.token_dim=16", "model.arch.head_hidden=32",
    "model.arch.head_layers=2", "+model.arch.token_patch=2", "+model.arch.vae_base=8", "+model.arch.vae_mults=[1,2]",
    "+model.arch.vae_blocks=1", "model.dtype=float32", "model.lora.rank=4", "model.lora.alpha=8",
    "sampling.image_size=16", "sampling.image_token_num=4", "sampling.num_flow_steps=3",
    "rollout.n_samples_per_prompt=2", "rollout.rollout_batch_size=2", "rollout.max_text_length=8", "actor.bf16=false",
    "reward.components.ocr=0.0", "reward.components.vit_scalar=1.0", "reward.kwargs.vit_scalar.preset=vit_tiny",
    "reward.kwargs.vit_scalar.seed=0", "reward.kwargs.vit_scalar.num_frames=1", "data.manifest=synthetic:8:0",
    "distributed.rollout.gpus_per_worker=0",
]


@pytest.mark.timeout(600)
@pytest.mark.parametrize("experiment,overrides,samples,epochs", [
    ("experiment/tiny_dit_grpo", ["sampling.num_steps=3", "rollout.n=2", "rollout.rollout_batch_size=2",
                                  "rollout.sample_batch_size=2", "distributed.param_sharding=full"], 4, ["0", "1"]),
    ("experiment/janus_pro_1b_shape_grpo", TINY_JANUS, 8, ["0", "1"]),
    ("experiment/cosmos_predict2_2b_grpo", TINY_COSMOS, 4, ["0", "1"]),
    ("experiment/nextstep_1_ocr_grpo", TINY_NEXTSTEP, 4, ["1", "2"]),        # this recipe counts steps from 1
])
def test_recipes_train_checkpoint_and_resume_on_two_data_parallel_cpu_ranks(tmp_path, experiment, overrides, samples,
                                                                            epochs):
    import math

    res = _run(_workers.recipe_runs_on_cpu_ranks, 2, experiment, overrides, str(tmp_path / "run"), _free_port(),
               timeout=500)
    rows, perf = res["rows"], res["perf"]
    assert [r[0] for r in rows[1:]] == epochs
    assert all(math.isfinite(float(v)) for r in rows[1:] for v in r[1:6])
    assert [p["n_ranks"] for p in perf] == [2, 2] and perf[0]["samples"] == samples


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("collectives", ["nccl", "fused"])
def test_fsdp_gpu_matches_replicated(collectives):
    world = min(torch.cuda.device_count(), 4)
    res = _run(_workers.fsdp_training_matches_replicated, world, "nccl", collectives, 1, True)
    assert res["shapes_ok"] and res["err"] < 6e-2 and res["fwd_err"] < 0.25, res
    assert res["handles"] > 0 and res["buckets"] > 0
    assert (res["fused_gathers"] > 0) == (collectives == "fused")


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("collectives", ["nccl", "fused"])
def test_sharded_adamw_gpu(collectives):
    world = min(torch.cuda.device_count(), 4)
    res = _run(_workers.sharded_adamw_matches_single, world, "nccl", collectives)
    assert res["err"] < 2e-2 and res["same"]


@pytest.mark.gpu
@pytest.mark.multigpu
@pytest.mark.parametrize("use_kernels", [False, True])
def test_ulysses_attention_gpu(use_kernels):
    world = 2
    res = _run(_workers.ulysses_attention_matches_dense, world, "nccl", use_kernels)
    assert res["fwd"] and res["bwd"]
    assert (res["launches"] > 0) == use_kernels
    assert res["fused_layers"] == (5 if use_kernels else 0)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_weight_broadcast_versions_and_bounded_wait():
    world = min(torch.cuda.device_count(), 4)
    res = _run(_workers.weight_broadcast_and_timeout, world)
    assert res["ok"] and res["timed_out"]


@pytest.mark.gpu
@pytest.mark.multigpu
def test_allgather_fused_gemm_matches_library():
    world = min(torch.cuda.device_count(), 4)
    res = _run(_workers.allgather_gemm_matches_library, world)
    assert res["ok"], res["detail"]


@pytest.mark.timeout(600)
def test_recipe_restarts_in_place_from_the_latest_checkpoint_after_a_rank_raises(tmp_path):
    res = _run(_workers.recipe_restarts_in_place_after_a_rank_raises, 2, str(tmp_path / "run"), _free_port(),
               timeout=500)
    assert res["restarts"] == 1 and res["attempts"] == [0, 1]
    # epochs 0 and 1 ran before the failure, epoch 2 after the restart; nothing ran twice
    assert [r[0] for r in res["rows"][1:]] == ["0", "1", "2"]
    assert res["checkpoints"] == ["checkpoint-1", "checkpoint-2", "checkpoint-3", "checkpoint-final"]
    assert res["resume_configs"] == 1


@pytest.mark.timeout(600)
def test_preference_recipe_trains_and_resumes_on_two_cpu_ranks(tmp_path):
    import math

    overrides = ["model.arch.num_layers=2", "model.arch.hidden_size=64", "model.arch.num_heads=2",
                 "model.arch.ffn_dim=128", "model.arch.text_dim=32", "model.arch.freq_dim=32", "model.dtype=float32",
                 "sampling.num_frames=5", "sampling.height=32", "sampling.width=32", "sampling.max_sequence_length=8",
                 "sampling.num_steps=4", "actor.bf16=false", "data.synthetic.num_pairs=8"]
    res = _run(_workers.dpo_recipe_runs_on_cpu_ranks, 2, overrides, str(tmp_path / "run"), _free_port(), timeout=500)
    header, rows = res["rows"][0], res["rows"][1:]
    # three steps, then the resumed run picks up the latest checkpoint and adds steps four and five
    assert [r[0] for r in rows] == ["1", "2", "3", "4", "5"]
    assert res["checkpoints"] == ["checkpoint-2", "checkpoint-4", "checkpoint-final"]
    assert float(rows[0][header.index("loss")]) == pytest.approx(math.log(2.0), abs=1e-5)
    # the learning rate is scaled by the number of ranks (actor.scale_lr)
    assert float(rows[0][header.index("lr")]) == pytest.approx(2.0e-8)
    assert all(math.isfinite(float(r[header.index("grad_norm")])) for r in rows)
