"""Recovery after a rank failed: the latest-checkpoint search behind ``trainer.resume_from=auto``,
the host-side fault plan, the restart decision, and two whole jobs under the real launcher on CPU
ranks — one restarted in place by the surviving processes, one whose processes the launcher
replaces.  Every failure is raised on the host before a step launches anything."""

import json
import os
import socket
import subprocess
import sys

import pytest
import torch

from visionrl_b200.config.loader import load_config
from visionrl_b200.parallel import liveness
from visionrl_b200.scripts import elastic
from visionrl_b200.trainers import checkpointing as ck

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _checkpoint(root, name, next_epoch, *, payload=True, meta=True):
    d = root / name
    d.mkdir(parents=True)
    if payload:
        torch.save({"schema_version": ck.CHECKPOINT_SCHEMA_VERSION, "family": "sd3_5", "trainer": {}, "model": {},
                    "progress": {"next_epoch": next_epoch}, "rng": {}}, d / ck.TRAINING_CHECKPOINT_NAME)
    if meta:
        (d / ck.CHECKPOINT_META_NAME).write_text(json.dumps({"next_epoch": next_epoch, "family": "sd3_5"}))
    return d


def test_latest_checkpoint_is_the_complete_one_that_is_furthest_along(tmp_path):
    assert ck.latest_checkpoint(tmp_path / "absent") is None
    assert ck.latest_checkpoint(tmp_path) is None
    _checkpoint(tmp_path, "checkpoint-1", 1)
    second = _checkpoint(tmp_path, "checkpoint-2", 2)
    _checkpoint(tmp_path, "checkpoint-3", 3, meta=False)             # interrupted before its meta file
    _checkpoint(tmp_path, "checkpoint-4", 4, payload=False)          # meta without payload
    (tmp_path / "checkpoint-5").mkdir()
    (tmp_path / "checkpoint-5" / ck.CHECKPOINT_META_NAME).write_text("not json")
    (tmp_path / "metrics.csv").write_text("epoch\n")
    assert ck.latest_checkpoint(tmp_path) == second
    final = _checkpoint(tmp_path, "checkpoint-final", 2)             # same progress, written later
    os.utime(final / ck.TRAINING_CHECKPOINT_NAME, (2e9, 2e9))
    assert ck.latest_checkpoint(tmp_path) == final


def test_auto_resume_starts_fresh_without_a_checkpoint_and_picks_the_latest_with_one(tmp_path):
    def cfg():
        return load_config("experiment/tiny_dit_grpo", overrides=[f"trainer.output_dir={tmp_path}",
                                                                    "trainer.resume_from=auto"])

    assert ck.load_training_checkpoint_from_config(cfg()) is None
    _checkpoint(tmp_path, "checkpoint-1", 1)
    _checkpoint(tmp_path, "checkpoint-2", 2)
    found = ck.load_training_checkpoint_from_config(cfg())
    assert found is not None and found.checkpoint_dir.name == "checkpoint-2"


def test_a_checkpoint_payload_is_never_seen_half_written(tmp_path, monkeypatch):
    seen = {}
    real = os.replace

    def spy(src, dst):
        seen["partial_existed"] = os.path.exists(src) and not os.path.exists(dst)
        real(src, dst)

    monkeypatch.setattr(ck.os, "replace", spy)

    class _Trainer:
        def state_dict(self):
            return {"step": 3}

    bundle = type("B", (), {"trainable_modules": {"m": torch.nn.Linear(2, 2)}, "metadata": {"family": "sd3_5"}})()
    ck.save_training_checkpoint(tmp_path / "checkpoint-1", trainer=_Trainer(), bundle=bundle, family="sd3_5",
                                progress={"completed_epoch": 1, "next_epoch": 1})
    assert seen["partial_existed"]
    assert sorted(p.name for p in (tmp_path / "checkpoint-1").iterdir()) == [ck.TRAINING_CHECKPOINT_NAME,
                                                                            ck.CHECKPOINT_META_NAME]
    assert ck.latest_checkpoint(tmp_path) == tmp_path / "checkpoint-1"


def test_fault_plan_fires_on_its_rank_step_and_attempt_only(monkeypatch):
    monkeypatch.delenv("VRL_FAULT_INJECT", raising=False)
    monkeypatch.delenv("VRL_RESTART_ATTEMPT", raising=False)
    monkeypatch.delenv("TORCHELASTIC_RESTART_COUNT", raising=False)
    liveness.maybe_inject_fault(1, 2)                                  # no plan: nothing happens
    monkeypatch.setenv("VRL_FAULT_INJECT", "rank=1, step=2")
    liveness.maybe_inject_fault(0, 2)
    liveness.maybe_inject_fault(1, 1)
    with pytest.raises(liveness.InjectedFault, match="rank 1 at step 2"):
        liveness.maybe_inject_fault(1, 2)
    monkeypatch.setenv("VRL_RESTART_ATTEMPT", "1")                     # the restarted run is left alone
    liveness.maybe_inject_fault(1, 2)
    monkeypatch.delenv("VRL_RESTART_ATTEMPT")
    monkeypatch.setenv("TORCHELASTIC_RESTART_COUNT", "1")              # and so are relaunched workers
    liveness.maybe_inject_fault(1, 2)
    monkeypatch.setenv("VRL_FAULT_INJECT", "rank=1,step=2,attempt=1")
    with pytest.raises(liveness.InjectedFault):
        liveness.maybe_inject_fault(1, 2)
    monkeypatch.setenv("VRL_FAULT_INJECT", "rank=one")
    with pytest.raises(ValueError, match="VRL_FAULT_INJECT"):
        liveness.maybe_inject_fault(1, 2)


def test_each_start_of_a_job_has_its_own_liveness_keys(monkeypatch):
    monkeypatch.delenv("VRL_RESTART_ATTEMPT", raising=False)
    monkeypatch.delenv("TORCHELASTIC_RESTART_COUNT", raising=False)
    first = liveness.incarnation()
    monkeypatch.setenv("VRL_RESTART_ATTEMPT", "1")
    second = liveness.incarnation()
    monkeypatch.setenv("TORCHELASTIC_RESTART_COUNT", "2")
    third = liveness.incarnation()
    assert len({first, second, third}) == 3


def test_restart_decision_and_rendezvous_ports():
    assert elastic.restartable(RuntimeError("peer gone"), group_was_formed=True)
    assert elastic.restartable(liveness.RankFailure(1, "silent"), group_was_formed=True)
    assert not elastic.restartable(RuntimeError("bad config"), group_was_formed=False)
    assert not elastic.restartable(FileNotFoundError("manifest"), group_was_formed=True)
    assert not elastic.restartable(KeyboardInterrupt(), group_was_formed=True)
    assert [elastic.rendezvous_port(k, None, 29500) for k in range(3)] == [29500, 29501, 29502]
    assert elastic.rendezvous_port(1, [4000, 4100], 29500) == 4100
    with pytest.raises(ValueError, match="only 2"):
        elastic.rendezvous_port(2, [4000, 4100], 29500)
    with pytest.raises(ValueError, match="max_restarts"):
        elastic.run_with_restarts("experiment/tiny_dit_grpo", max_restarts=-1)


def test_a_failure_before_any_group_exists_is_not_retried(tmp_path, monkeypatch):
    monkeypatch.delenv("WORLD_SIZE", raising=False)
    calls = []
    with pytest.raises(Exception):
        elastic.run_with_restarts("experiment/does_not_exist", max_restarts=3, before_attempt=calls.append)
    assert calls == [0]


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(tmp_path, module, launcher_args, extra, overrides=()):
    out = tmp_path / "run"
    env = dict(os.environ, VRL_FAULT_INJECT="rank=1,step=2", PYTHONPATH=ROOT)
    for name in ("RANK", "WORLD_SIZE", "LOCAL_RANK", "MASTER_PORT", "VRL_RESTART_ATTEMPT", "TORCHELASTIC_RESTART_COUNT"):
        env.pop(name, None)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), *launcher_args, "-m", module,
           *extra, "--config", "experiment/tiny_dit_grpo", "sampling.num_steps=3", "rollout.n=2",
           "rollout.rollout_batch_size=2", "rollout.sample_batch_size=2", f"trainer.output_dir={out}",
           "trainer.total_epochs=3", "trainer.save_freq=1", "distributed.backend=native",
           "distributed.collectives=nccl", "distributed.timeout_s=15", *overrides]
    done = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=500)
    return out, done


def _assert_three_epochs_once_each(out, done):
    assert done.returncode == 0, done.stderr[-3000:]
    assert "injected failure on rank 1 at step 2" in done.stderr
    rows = (out / "metrics.csv").read_text().splitlines()
    assert [r.split(",")[0] for r in rows[1:]] == ["0", "1", "2"]
    assert sorted(p.name for p in out.glob("checkpoint-*")) == ["checkpoint-1", "checkpoint-2", "checkpoint-3",
                                                               "checkpoint-final"]
    assert len(list(out.glob("resume_config_*.yaml"))) == 1


@pytest.mark.timeout(600)
def test_job_under_the_launcher_restarts_in_place_after_a_rank_raises(tmp_path):
    out, done = _launch(tmp_path, "visionrl_b200.scripts.elastic", [], ["--max-restarts", "1"])
    _assert_three_epochs_once_each(out, done)
    assert "finished after 1 restart" in done.stderr


@pytest.mark.timeout(600)
def test_workers_replaced_by_the_launcher_resume_from_the_latest_checkpoint(tmp_path):
    out, done = _launch(tmp_path, "visionrl_b200.scripts.train", ["--max-restarts", "1"], [],
                        ["trainer.resume_from=auto"])
    _assert_three_epochs_once_each(out, done)
