"""Reward combination and OCR scoring (reference expectations: ``tests/rewards/test_multi.py:32-52``,
``test_composite.py``, ``test_ocr.py:90-141``)."""

import asyncio

import pytest
import torch

from visionrl_b200.algorithms.types import Rollout, Trajectory
from visionrl_b200.rewards import CompositeReward, MultiReward, RewardFunction, get_reward, register_reward
from visionrl_b200.rewards.ocr import OCRReward, _edit_distance, _normalize_ocr_text
from visionrl_b200.rewards.remote import RemoteReward


def _run(coro):
    return asyncio.new_event_loop().run_until_complete(coro)


def _rollout(output=None, prompt="p", **meta):
    return Rollout(request=None, trajectory=Trajectory(prompt=prompt, seed=0, steps=[], output=output),
                   metadata=meta)


class _Const(RewardFunction):
    def __init__(self, value, device="cpu"):
        self.value = value

    async def score(self, rollout):
        return self.value


def test_multi_reward_accumulates_component_history_until_reset():
    multi = MultiReward([("a", 1.0, _Const(0.2)), ("b", 2.0, _Const(0.5))])
    assert _run(multi.score(_rollout())) == pytest.approx(1.2)
    assert _run(multi.score_batch([_rollout(), _rollout()])) == pytest.approx([1.2, 1.2])
    assert multi.last_components == {"a": [0.2, 0.2, 0.2], "b": [0.5, 0.5, 0.5]}
    assert multi.component_means() == pytest.approx({"a": 0.2, "b": 0.5})
    multi.reset_components()
    assert multi.last_components == {}
    _run(multi.score(_rollout()))
    assert multi.last_components == {"a": [0.2], "b": [0.5]}


def test_registry_round_trip_and_from_dict():
    class _Mine(_Const):
        def __init__(self, device="cpu", value=0.75):
            super().__init__(value)

    register_reward("mine_for_test", _Mine)
    assert get_reward("mine_for_test") is _Mine
    multi = MultiReward.from_dict({"mine_for_test": 2.0}, device="cpu",
                                  reward_kwargs={"mine_for_test": {"value": 0.5}})
    assert _run(multi.score(_rollout())) == pytest.approx(1.0)
    with pytest.raises((KeyError, ValueError)):
        get_reward("definitely_not_registered")
    for name in ("aesthetic", "clipscore", "pickscore", "ocr"):
        assert issubclass(get_reward(name), RewardFunction)


def test_composite_is_a_weighted_sum():
    comp = CompositeReward([(0.5, _Const(1.0)), (2.0, _Const(0.25))])
    assert _run(comp.score(_rollout())) == pytest.approx(1.0)
    assert _run(comp.score_batch([_rollout(), _rollout()])) == pytest.approx([1.0, 1.0])


def test_default_score_batch_is_sequential_score():
    assert _run(_Const(0.3).score_batch([_rollout()] * 3)) == pytest.approx([0.3] * 3)


# ------------------------------------------------------------------------------------- OCR
def test_levenshtein_and_normalisation():
    assert _edit_distance("kitten", "sitting") == 3
    assert _edit_distance("", "abc") == 3 and _edit_distance("abc", "abc") == 0
    assert _normalize_ocr_text(" He llo") == "hello"


def test_image_substring_gets_full_credit():
    reward = OCRReward(device="cpu", engine=lambda frame: "xx HELLO world yy")
    image = torch.rand(3, 16, 16)
    assert _run(reward.score(_rollout(image, target_text="Hello World"))) == 1.0
    assert _run(reward.score(_rollout(image))) == 0.0                      # no target -> 0


def test_video_uses_edit_distance_on_every_fourth_frame():
    seen = []

    def engine(frame):
        seen.append(frame.shape)
        return "hellp" if len(seen) == 1 else "zzzzz"

    reward = OCRReward(device="cpu", engine=engine)
    video = torch.rand(3, 9, 8, 8)                                         # [C, T, H, W]
    value = _run(reward.score(_rollout(video, target_text="hello")))
    assert len(seen) == 3 and seen[0] == (8, 8, 3)                         # frames 0, 4, 8
    assert 0.0 < value < 1.0 and value == pytest.approx(0.8)               # mean over frames with reward > 0


def test_debug_dump_writes_best_frame(tmp_path):
    reward = OCRReward(device="cpu", debug_dir=str(tmp_path), engine=lambda frame: "hello")
    _run(reward.score(_rollout(torch.rand(3, 8, 8), target_text="hello")))
    assert len(list(tmp_path.glob("*.txt"))) == 1


# ---------------------------------------------------------------------------------- remote
def test_remote_reward_payload_and_score(monkeypatch):
    reward = RemoteReward("http://127.0.0.1:9/score", reward_name="aesthetic")
    rollout = _rollout(prompt="a cat", foo=1)
    payload = reward._payload(rollout)
    assert payload["prompt"] == "a cat" and payload["reward"] == "aesthetic" and payload["metadata"] == {"foo": 1}

    async def fake_post(body):
        return {"score": 0.4, "scores": [0.4, 0.6]}

    monkeypatch.setattr(reward, "_post", fake_post)
    assert _run(reward.score(rollout)) == pytest.approx(0.4)
    assert _run(reward.score_batch([rollout, rollout])) == pytest.approx([0.4, 0.6])


def test_aesthetic_head_weights_are_resolved_from_path_env_or_assets(tmp_path, monkeypatch):
    import torch

    from visionrl_b200.rewards.aesthetic import AestheticMLP, AestheticReward, resolve_mlp_weights

    monkeypatch.delenv("VRL_AESTHETIC_MLP", raising=False)
    assert resolve_mlp_weights(None) is None                      # nothing shipped: stand-in is used
    with pytest.raises(FileNotFoundError):
        resolve_mlp_weights(str(tmp_path / "missing.pth"))
    head = AestheticMLP(768)
    with torch.no_grad():
        for p in head.parameters():
            p.fill_(0.01)
    path = tmp_path / "head.pth"
    torch.save(head.state_dict(), path)
    assert resolve_mlp_weights(str(path)) == path
    monkeypatch.setenv("VRL_AESTHETIC_MLP", str(path))
    assert resolve_mlp_weights(None) == path
    reward = AestheticReward(device="cpu", model_name="vit_tiny", random_init=False)
    try:
        reward._ensure_loaded()
    except Exception:      # noqa: BLE001 - the image tower needs weights that are not available offline
        return
    assert torch.allclose(reward._mlp.layers[0].weight, torch.full_like(reward._mlp.layers[0].weight, 0.01))


def test_reward_constructors_take_the_reference_argument_order(tmp_path):
    """Positional calls written against the reference keep working: ``(device, dtype, model_name)``
    for the aesthetic and preference scorers, ``(device, model_name)`` for CLIP-score,
    ``(url, timeout)`` for the remote one, ``(device, debug_dir)`` for OCR."""
    from visionrl_b200.rewards.aesthetic import AestheticReward
    from visionrl_b200.rewards.clip import CLIPScoreReward
    from visionrl_b200.rewards.ocr import OCRReward
    from visionrl_b200.rewards.pickscore import PickScoreReward
    from visionrl_b200.rewards.remote import RemoteReward
    from visionrl_b200.rewards.vision_tower import tower_dtype

    aesthetic = AestheticReward("cpu", "float32", "random:vit_tiny")
    assert (aesthetic._device, aesthetic._dtype, aesthetic.model_name) == ("cpu", "float32", "random:vit_tiny")
    clip = CLIPScoreReward("cpu", "random:vit_tiny")
    assert clip.model_name == "random:vit_tiny" and clip._dtype is None
    pick = PickScoreReward("cpu", "bfloat16", "some/processor", "random:vit_tiny")
    assert (pick._dtype, pick.processor_name, pick.model_name) == ("bfloat16", "some/processor", "random:vit_tiny")
    assert RemoteReward("http://x/score", 5.0).timeout_s == 5.0 and RemoteReward("http://x/score").timeout_s == 60.0
    ocr = OCRReward("cpu", str(tmp_path / "dbg"))
    assert ocr._debug_dir == tmp_path / "dbg" and ocr._debug_dir.is_dir()
    # the dtype string is honoured by the tower that gets built
    score = aesthetic.score_tensor_batch(torch.rand(1, 3, 32, 32), ["p"]) if hasattr(aesthetic, "score_tensor_batch") else None
    assert aesthetic._tower is None or aesthetic._tower.proj.weight.dtype == torch.float32
    del score
    assert tower_dtype("bf16", torch.device("cpu")) == torch.bfloat16
    assert tower_dtype(None, torch.device("cpu")) == torch.float32
    with pytest.raises(ValueError):
        tower_dtype("int8", torch.device("cpu"))
