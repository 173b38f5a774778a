"""One fixed set of calls into the algorithm layer (losses, advantages, the flow-matching SDE / CPS
step with sampling, replay and the deterministic path, KL terms, the per-prompt statistics tracker,
OCR text distances, the K-repeat sampler), with seeded inputs.  ``compute()`` returns every result
as a tensor under a readable key; ``tests/golden/algorithm_outputs.pt`` holds the values the
reference implementation's own functions give for exactly these calls."""

import inspect
import math  # noqa: F401

import numpy as np
import torch


class _Schedule:
    """Shifted flow-matching grid with the three members the SDE step reads."""

    def __init__(self, steps: int, shift: float = 3.0, train_steps: int = 1000):
        sigma = torch.linspace(1.0, 1.0 / train_steps, steps, dtype=torch.float64)
        sigma = shift * sigma / (1 + (shift - 1) * sigma)
        self.timesteps = (sigma * train_steps).to(torch.float32)
        self.sigmas = torch.cat([sigma, sigma.new_zeros(1)]).to(torch.float32)

    def index_for_timestep(self, timestep) -> int:
        return int(torch.argmin((self.timesteps - float(timestep)).abs()).item())


def compute() -> dict:
    res = {}
    g = torch.Generator().manual_seed(0)
    R = lambda *s: torch.randn(*s, generator=g)  # noqa: E731
    import sys  # noqa: F401
    g = torch.Generator().manual_seed(0)
    R = lambda *s: torch.randn(*s, generator=g)

    # --- DPO
    from vrl.algorithms.dpo import diffusion_dpo_loss, diffusion_sft_loss
    for name, shape in (("img", (6, 4, 8, 8)), ("vid", (4, 4, 3, 8, 8))):
        pred, ref, tgt = R(*shape), R(*shape), R(*shape)
        st = diffusion_dpo_loss(pred, ref, tgt, 2500.0)
        st = st if isinstance(st, dict) else st.__dict__
        for k, v in st.items():
            if torch.is_tensor(v): res[f"dpo/{name}/{k}"] = v.detach().float()
        res[f"sft/{name}"] = diffusion_sft_loss(pred[: shape[0] // 2], tgt[: shape[0] // 2]).detach()

    # --- GRPO advantages + loss
    from vrl.algorithms.grpo import GRPO, GRPOConfig
    from vrl.rollouts.evaluators import SignalBatch
    for gs in (False, True):
        algo = GRPO(GRPOConfig(global_std=gs, adv_clip_max=1.5))
        rewards = R(12)
        groups = torch.tensor([0, 0, 0, 0, 1, 1, 1, 1, 2, 2, 2, 2])
        res[f"grpo/adv/{gs}"] = algo.compute_advantages_from_tensors(rewards, groups)
    same = torch.ones(4)
    res["grpo/adv/zero_std"] = GRPO(GRPOConfig()).compute_advantages_from_tensors(same, torch.zeros(4, dtype=torch.long))
    import inspect
    fields = set(inspect.signature(SignalBatch).parameters)
    def sig(**kw):
        return SignalBatch(**{k: v for k, v in kw.items() if k in fields})
    for kl in (0.0, 0.02):
        for use_dt in (False, True):
            algo = GRPO(GRPOConfig(eps_clip=0.2, init_kl_coef=kl, flow_kl_use_dt=use_dt))
            new_lp, old_lp, adv = R(8), R(8), R(8)
            mean, ref_mean = R(8, 4, 6, 6), R(8, 4, 6, 6)
            std = torch.rand(8, 1, 1, 1, generator=g) + 0.1
            dt = -(torch.rand(8, 1, 1, 1, generator=g) + 0.1)
            s = sig(log_prob=new_lp, prev_sample_mean=mean, ref_prev_sample_mean=ref_mean if kl > 0 else None, std_dev_t=std, dt=dt, ref_log_prob=R(8) if kl > 0 else None, aux={}, dist_family="flow_matching")
            loss, m = algo.compute_signal_loss(s, adv, old_lp)
            res[f"grpo/loss/{kl}/{use_dt}"] = loss.detach()
            for k in ("policy_loss", "kl_penalty", "clip_fraction", "approx_kl"):
                res[f"grpo/loss/{kl}/{use_dt}/{k}"] = torch.tensor(float(getattr(m, k)))

    # --- TokenGRPO
    from vrl.algorithms.grpo_token import TokenGRPO, TokenGRPOConfig
    for est in ("k1", "k3"):
        for kl in (0.0, 0.05):
            algo = TokenGRPO(TokenGRPOConfig(eps_clip=0.2, init_kl_coef=kl, kl_estimator=est))
            new_lp, old_lp, ref_lp, adv = R(4, 9) * 0.3, R(4, 9) * 0.3, R(4, 9) * 0.3, R(4)
            mask = (torch.rand(4, 9, generator=g) > 0.3).float()
            s = sig(log_prob=new_lp, ref_log_prob=ref_lp if kl > 0 else None, aux={"token_mask": mask}, prev_sample_mean=None, ref_prev_sample_mean=None, std_dev_t=None, dt=None, dist_family="categorical")
            loss, m = algo.compute_signal_loss(s, adv, old_lp)
            res[f"tgrpo/{est}/{kl}"] = loss.detach()
            for k in ("policy_loss", "kl_penalty", "clip_fraction", "approx_kl"):
                res[f"tgrpo/{est}/{kl}/{k}"] = torch.tensor(float(getattr(m, k)))

    # --- stat tracker
    from vrl.algorithms.stat_tracking import PerPromptStatTracker
    for gs in (False, True):
        tr = PerPromptStatTracker(global_std=gs)
        prompts = ["a", "a", "b", "b", "b", "c"]
        r1 = np.array([1.0, 2.0, 0.5, 0.7, 0.9, 3.0])
        r2 = np.array([0.0, 1.0, 0.1, 0.2, 0.3, 2.0])
        res[f"stat/{gs}/1"] = torch.tensor(tr.update(prompts, r1))
        res[f"stat/{gs}/2"] = torch.tensor(tr.update(prompts, r2))
        res[f"stat/{gs}/stats"] = torch.tensor([float(x) for x in tr.get_stats()])

    # --- flow-matching SDE step
    from vrl.algorithms.flow_matching import sde_step_with_logprob, compute_kl_divergence
    for sde_type in ("sde", "cps"):
        for nl in (0.7, 1.0):
            sch = _Schedule(10)
            x, v = R(3, 4, 6, 6), R(3, 4, 6, 6)
            t = sch.timesteps[[2, 2, 5]]
            gen = torch.Generator().manual_seed(5)
            out_ = sde_step_with_logprob(sch, v, t, x, generator=gen, noise_level=nl, sde_type=sde_type, return_dt=True)
            for k in ("prev_sample", "log_prob", "prev_sample_mean", "std_dev_t", "dt"):
                val = getattr(out_, k, None)
                if torch.is_tensor(val): res[f"sde/{sde_type}/{nl}/{k}"] = val.detach().float().reshape(-1)
            # replay with the recorded next sample
            rep = sde_step_with_logprob(sch, v, t, x, prev_sample=out_.prev_sample, noise_level=nl, sde_type=sde_type)
            res[f"sde/{sde_type}/{nl}/replay_lp"] = rep.log_prob.detach().float()
            det = sde_step_with_logprob(sch, v, t, x, deterministic=True, noise_level=nl, sde_type=sde_type)
            res[f"sde/{sde_type}/{nl}/det"] = det.prev_sample.detach().float().reshape(-1)
    res["kl/plain"] = compute_kl_divergence(R(3, 4, 5), R(3, 4, 5), torch.rand(3, 1, 1, generator=g) + 0.2)
    res["kl/dt"] = compute_kl_divergence(R(3, 4, 5), R(3, 4, 5), torch.rand(3, 1, 1, generator=g) + 0.2, dt=torch.rand(3, 1, 1, generator=g) + 0.2)

    # --- OCR helpers
    from vrl.rewards import ocr as O
    for a, b in (("Hello, World!", "hello world"), ("kitten", "sitting"), ("", "abc"), ("  A  b ", "ab"), ("Open-Late!!", "open late")):
        res[f"ocr/{a}|{b}"] = torch.tensor([float(O._edit_distance(O._normalize_ocr_text(a), O._normalize_ocr_text(b))),
                                            float(O._normalized_edit_distance(O._normalize_text(a), O._normalize_text(b))),
                                            float(len(O._normalize_ocr_text(a))), float(len(O._normalize_text(a)))])
        res[f"ocrfrag/{a}"] = torch.tensor([float(ord(c)) for c in O._safe_filename_fragment(a)] or [0.0])

    # --- K-repeat sampler
    from vrl.trainers.data import DistributedKRepeatSampler
    class DS:
        def __len__(self): return 37
    for rank in (0, 1):
        smp = DistributedKRepeatSampler(DS(), batch_size=6, k=3, num_replicas=2, rank=rank, seed=7)
        it = iter(smp)
        smp.set_epoch(2) if hasattr(smp, "set_epoch") else None
        res[f"sampler/{rank}"] = torch.tensor([list(next(it)) for _ in range(2)])
    return res
