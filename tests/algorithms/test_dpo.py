"""Diffusion-DPO loss against an inline statement of the formula."""

import math

import pytest
import torch
import torch.nn.functional as F

from vrl.algorithms.dpo import diffusion_dpo_loss, diffusion_sft_loss


def _inline(model_pred, ref_pred, target, beta):
    dims = tuple(range(1, model_pred.ndim))
    ml = ((model_pred - target) ** 2).mean(dims)
    rl = ((ref_pred - target) ** 2).mean(dims)
    b = ml.shape[0] // 2
    inside = -0.5 * beta * ((ml[:b] - ml[b:]) - (rl[:b] - rl[b:]))
    return -F.logsigmoid(inside).mean(), (inside > 0).float().mean()


@pytest.mark.parametrize("shape", [(6, 4, 8, 8), (4, 4, 3, 8, 8)])
def test_parity_with_inline_formula(shape):
    torch.manual_seed(0)
    mp, rp, tg = (torch.randn(shape) for _ in range(3))
    out = diffusion_dpo_loss(mp, rp, tg, beta=3.0)
    loss, acc = _inline(mp, rp, tg, 3.0)
    assert torch.allclose(out["loss"], loss) and torch.allclose(out["implicit_acc"], acc)
    assert set(out) == {"loss", "raw_model_loss", "raw_ref_loss", "model_diff", "ref_diff",
                        "implicit_acc"}


def test_policy_equals_reference_gives_log2():
    p, t = torch.randn(4, 3, 5, 5), torch.randn(4, 3, 5, 5)
    out = diffusion_dpo_loss(p, p.clone(), t, beta=5000.0)
    assert out["loss"].item() == pytest.approx(math.log(2.0), rel=1e-6)
    assert out["implicit_acc"].item() == 0.0


def test_bad_inputs_raise():
    with pytest.raises(ValueError, match="2\\*B"):
        diffusion_dpo_loss(torch.zeros(3, 2), torch.zeros(3, 2), torch.zeros(3, 2), 1.0)
    with pytest.raises(ValueError, match="shape mismatch"):
        diffusion_dpo_loss(torch.zeros(2, 2), torch.zeros(2, 3), torch.zeros(2, 2), 1.0)


def test_sft_loss_is_mse():
    a, b = torch.randn(3, 4), torch.randn(3, 4)
    assert torch.allclose(diffusion_sft_loss(a, b), F.mse_loss(a, b))
