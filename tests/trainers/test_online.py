"""OnlineTrainer on a one-parameter model with fake collector / evaluator / algorithm / syncer.

Mirrors the behaviours the reference pins in ``tests/trainers/test_online.py``: weights are
pushed before the first collect and again after the step, plain prompts are collected in one call
and trained one group at a time, ``PromptExample`` fields travel as collect keyword arguments,
metrics propagate, optimizer and EMA state survive a checkpoint round trip.
"""

import asyncio
from dataclasses import dataclass

import pytest
import torch
from torch import nn

from visionrl_b200.algorithms.base import Algorithm
from visionrl_b200.algorithms.types import TrainStepMetrics
from visionrl_b200.rollouts.batch import RolloutBatch
from visionrl_b200.rollouts.evaluators.types import SignalBatch
from visionrl_b200.trainers.data import PromptExample
from visionrl_b200.trainers.online import OnlineTrainer, split_batch_by_group
from visionrl_b200.trainers.types import EMAConfig, TrainerConfig
from visionrl_b200.trainers.weight_sync import WeightSyncer


@dataclass
class _AlgoConfig:
    init_kl_coef: float = 0.0


class _FakeAlgorithm(Algorithm):
    def __init__(self):
        self.config = _AlgoConfig()
        self.advantage_inputs = []
        self._last_policy_loss_tensor = None
        self._last_kl_term_tensor = None

    def compute_advantages_from_tensors(self, rewards, group_ids):
        self.advantage_inputs.append((rewards.clone(), group_ids.clone()))
        return rewards - rewards.mean()

    def compute_signal_loss(self, signals, advantages, old_log_probs):
        loss = -(signals.log_prob * advantages).mean()
        self._last_policy_loss_tensor = loss
        return loss, TrainStepMetrics(loss=float(loss.detach()), policy_loss=float(loss.detach()),
                                      approx_kl=0.25, clip_fraction=0.5)


class _FakeCollector:
    def __init__(self, events, timesteps=2):
        self.events = events
        self.calls = []
        self.timesteps = timesteps

    async def collect(self, prompts, group_size, **kwargs):
        self.events.append("collect")
        self.calls.append((list(prompts), group_size, kwargs))
        b = len(prompts) * group_size
        obs = torch.arange(b, dtype=torch.float32).view(b, 1, 1).repeat(1, self.timesteps, 1) / 10
        group_ids = torch.arange(len(prompts)).repeat_interleave(group_size)
        return RolloutBatch(observations=obs, actions=obs + 1, rewards=torch.arange(b, dtype=torch.float32),
                            dones=torch.ones(b), group_ids=group_ids,
                            extras={"log_probs": torch.zeros(b, self.timesteps)}, context={},
                            prompts=[p for p in prompts for _ in range(group_size)])


class _FakeEvaluator:
    def __init__(self):
        self.batch_sizes = []

    def evaluate(self, model, batch, timestep_idx, ref_model=None, signal_request=None):
        self.batch_sizes.append(batch.observations.shape[0])
        x = batch.observations[:, timestep_idx].to(next(model.parameters()).dtype)
        return SignalBatch(log_prob=model(x).squeeze(-1))


class _RecordingSyncer(WeightSyncer):
    def __init__(self, events):
        self.events, self.pushed = events, []

    async def push(self, state_dict):
        self.events.append("push")
        self.pushed.append({k: v.clone() for k, v in state_dict.items()})

    async def pull(self):
        return self.pushed[-1]


def _trainer(events=None, ema=False, prompts=None, **cfg_kwargs):
    events = events if events is not None else []
    torch.manual_seed(0)
    model = nn.Linear(1, 1)
    cfg = TrainerConfig(n=2, rollout_batch_size=4, bf16=False, ema=EMAConfig(enable=ema, decay=0.9),
                        **cfg_kwargs)
    collector, evaluator, algo = _FakeCollector(events), _FakeEvaluator(), _FakeAlgorithm()
    syncer = _RecordingSyncer(events)
    trainer = OnlineTrainer(algo, collector, evaluator, model, weight_syncer=syncer, config=cfg,
                            prompts=prompts or ["a", "b", "c", "d"], device="cpu")
    return trainer, collector, evaluator, algo, syncer, events


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


def test_push_before_first_collect_and_after_step():
    trainer, *_, syncer, events = _trainer()
    _run(trainer.step())
    assert events[0] == "push" and events[1] == "collect" and events[-1] == "push"
    assert events.count("push") == 2
    assert not torch.equal(syncer.pushed[0]["weight"], syncer.pushed[1]["weight"])


def test_plain_prompts_one_collect_then_training_per_group():
    trainer, collector, evaluator, *_ = _trainer()
    metrics = _run(trainer.step())
    assert len(collector.calls) == 1 and collector.calls[0][0] == ["a", "b", "c", "d"]
    assert collector.calls[0][1] == 2
    # 4 groups x 2 timesteps, every evaluate call sees one group of two samples
    assert evaluator.batch_sizes == [2] * 8
    assert metrics.approx_kl == pytest.approx(0.25) and metrics.clip_fraction == pytest.approx(0.5)
    assert trainer.state.step == 1 and trainer.state.global_step >= 1


def test_prompt_example_fields_travel_as_collect_kwargs():
    examples = [PromptExample(prompt="p0", target_text="HELLO", task_type="ocr", metadata={"k": 1}),
                PromptExample(prompt="p1", target_text="WORLD", references=["r"])]
    trainer, collector, *_ = _trainer(prompts=examples)
    _run(trainer.step())
    assert len(collector.calls) == 2
    (p0, n0, kw0), (p1, n1, kw1) = collector.calls
    assert p0 == ["p0"] and n0 == 2 and kw0["target_text"] == "HELLO" and kw0["task_type"] == "ocr"
    assert kw0["sample_metadata"] == {"k": 1}
    assert p1 == ["p1"] and kw1["references"] == ["r"]


def test_advantages_use_only_the_current_step():
    trainer, _, _, algo, *_ = _trainer()
    _run(trainer.step())
    _run(trainer.step())
    sizes = [r.numel() for r, _ in algo.advantage_inputs]
    assert sizes and all(s == sizes[0] for s in sizes)          # nothing accumulates across steps
    _, gids = algo.advantage_inputs[-1]
    assert sorted(set(gids.tolist())) == [0, 1, 2, 3]


def test_diagnostic_tensors_cleared_after_backward():
    trainer, _, _, algo, *_ = _trainer()
    _run(trainer.step())
    assert algo._last_policy_loss_tensor is None and algo._last_kl_term_tensor is None


def test_split_batch_by_group_preserves_rows():
    collector = _FakeCollector([])
    batch = _run(collector.collect(["a", "b", "c"], 2))
    parts = split_batch_by_group(batch)
    assert [p.rewards.tolist() for p in parts] == [[0.0, 1.0], [2.0, 3.0], [4.0, 5.0]]
    assert [p.prompts for p in parts] == [["a", "a"], ["b", "b"], ["c", "c"]]


def test_optimizer_and_ema_resume_round_trip():
    trainer, *_ = _trainer(ema=True)
    _run(trainer.step())
    state = trainer.state_dict()
    assert {"step", "global_step", "total_reward", "total_loss", "optimizer", "ema"} <= set(state)
    fresh, *_ = _trainer(ema=True)
    fresh._rollout_weights_initialized = True
    fresh.load_state_dict(state)
    assert fresh.state.step == trainer.state.step
    assert fresh._rollout_weights_initialized is False          # forces a re-push before collecting
    a = fresh._optimizer.state_dict()["state"]
    b = trainer._optimizer.state_dict()["state"]
    assert a.keys() == b.keys()
    for k in a:
        for name in ("exp_avg", "exp_avg_sq"):
            assert torch.allclose(a[k][name], b[k][name])
    ema_a, ema_b = fresh._ema.state_dict(), trainer._ema.state_dict()
    assert ema_a["decay"] == ema_b["decay"]
    for x, y in zip(ema_a["ema_parameters"], ema_b["ema_parameters"]):
        assert torch.equal(x, y)


def test_ema_state_rejected_when_ema_disabled():
    trainer, *_ = _trainer(ema=True)
    _run(trainer.step())
    state = trainer.state_dict()
    plain, *_ = _trainer(ema=False)
    with pytest.raises(ValueError):
        plain.load_state_dict(state)
    plain.load_state_dict(state, strict=False)                  # tolerated when not strict


def test_zero_advantage_samples_are_filtered_when_a_stat_tracker_is_attached():
    class _Tracker:
        def update(self, prompts, rewards):
            adv = torch.ones(len(prompts))
            adv[::2] = 0.0                      # first sample of every group of two
            return adv.numpy()

        def get_stats(self):
            return 2.0, 4

        def clear(self):
            return None

    trainer, _, evaluator, *_ = _trainer()
    trainer.stat_tracker = _Tracker()
    metrics = _run(trainer.step())
    assert evaluator.batch_sizes == [1] * 8          # one surviving sample per group
    assert metrics.group_size == pytest.approx(2.0) and metrics.trained_prompt_num == 4
