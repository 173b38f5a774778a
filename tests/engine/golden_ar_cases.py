"""The autoregressive side of the rollout path with seeded inputs: request parsing and the chunk
helpers (prompt-major expansion, chunk validation and seed offsets, padding two token batches to one
length), the discrete and the continuous packer on hand-made output batches, and both token
evaluators on stub policies (log-probabilities, the adapter-off reference, masks).  ``compute()``
flattens everything into named tensors; ``tests/golden/ar_path_outputs.pt`` holds what the
reference's own helpers, packers and evaluators give."""

import asyncio
import contextlib

import torch
from torch import nn
from vrl.engine.core.types import GenerationRequest, OutputBatch, GenerationMetrics
from vrl.engine.core.worker import GenerationIdFactory
from vrl.engine.microbatching import MicroBatchPlan
from vrl.engine.ar import (align_pair, chunk_seed_offset, expand_prompt_major_prompts, ordered_chunks, parse_ar_generation_spec,
                           require_rows, validate_chunk, ARTokenScheduler, ActiveSequence, ARSequenceKey)
from vrl.rollouts.packers.base import RolloutPackContext
from vrl.rollouts.packers.ar_discrete import ARDiscreteRolloutPacker
from vrl.rollouts.packers.ar_continuous import ARContinuousRolloutPacker
from vrl.rollouts.evaluators.ar import TokenLogProbEvaluator, ContinuousTokenLogProbEvaluator
from vrl.rollouts.evaluators import SignalRequest
def flat(res, prefix, obj, depth=0):
    if torch.is_tensor(obj): res[prefix] = obj.detach().float().clone()
    elif isinstance(obj, dict):
        for k, v in sorted(obj.items(), key=lambda kv: str(kv[0])): flat(res, f"{prefix}.{k}", v, depth + 1)
    elif isinstance(obj, bool) or isinstance(obj, (int, float)): res[prefix] = torch.tensor(float(obj))
    elif isinstance(obj, str): res[prefix] = torch.tensor([float(ord(c)) for c in obj] or [0.0])
    elif isinstance(obj, (list, tuple)) and depth < 4:
        for i, v in enumerate(obj): flat(res, f"{prefix}[{i}]", v, depth + 1)
    elif hasattr(obj, "__dataclass_fields__") and depth < 4:
        for k in obj.__dataclass_fields__: flat(res, f"{prefix}.{k}", getattr(obj, k), depth + 1)

def compute() -> dict:
    res = {}
    g = torch.Generator().manual_seed(0)
    req = GenerationRequest(request_id="r", family="janus_pro", task="ar_t2i", prompts=["p0", "p1", "p2"], samples_per_prompt=3,
                            sampling={"cfg_weight": 5.0, "temperature": 0.9, "image_token_num": 9, "image_size": 32, "seed": 11, "max_text_length": 8, "sample_batch_size": 2})
    specs = GenerationIdFactory().build_sample_specs(req)
    flat(res, "spec", parse_ar_generation_spec(req, default_image_token_num=16, default_image_size=64, default_max_text_length=12)
         if "default_image_token_num" in parse_ar_generation_spec.__code__.co_varnames else parse_ar_generation_spec(req))
    flat(res, "expand", expand_prompt_major_prompts(req))
    for i, (ps, ss, sc) in enumerate(((0, 0, 2), (0, 2, 1), (2, 1, 2))):
        ch = MicroBatchPlan(prompt_index=ps, prompt=req.prompts[ps], sample_start=ss, sample_count=sc)
        validate_chunk(req, ch)
        res[f"seedoff{i}"] = torch.tensor(float(chunk_seed_offset(req, ch)))
    for bad in ((5, 0, 1), (0, 2, 2), (0, 0, 0)):
        try:
            validate_chunk(req, MicroBatchPlan(prompt_index=bad[0], prompt="x", sample_start=bad[1], sample_count=bad[2]))
            res[f"bad{bad}"] = torch.tensor(0.0)
        except Exception as e: res[f"bad{bad}"] = torch.tensor(1.0)
    a, am = torch.randint(0, 9, (2, 5), generator=g), torch.ones(2, 5, dtype=torch.long)
    b, bm = torch.randint(0, 9, (2, 3), generator=g), torch.ones(2, 3, dtype=torch.long)
    try:
        flat(res, "align", align_pair(a, am, b, bm, pad_id=0) if "pad_id" in align_pair.__code__.co_varnames else align_pair(a, am, b, bm))
    except TypeError as e:
        res["align_sig"] = torch.tensor([float(len(align_pair.__code__.co_varnames))])
    # token scheduler
    try:
        sch = ARTokenScheduler(max_batch_size=3) if "max_batch_size" in ARTokenScheduler.__init__.__code__.co_varnames else ARTokenScheduler()
        res["sched_ok"] = torch.tensor(1.0)
    except Exception as e:
        res["sched_ok"] = torch.tensor(0.0)
    # packers
    B, L = 4, 6
    o_extra = {"token_ids": torch.randint(0, 50, (B, L), generator=g), "token_log_probs": -torch.rand(B, L, generator=g), "token_mask": torch.ones(B, L),
               "prompt_input_ids": torch.randint(0, 50, (B, 5), generator=g), "prompt_attention_mask": torch.ones(B, 5, dtype=torch.long),
               "uncond_input_ids": torch.randint(0, 50, (B, 5), generator=g), "uncond_attention_mask": torch.ones(B, 5, dtype=torch.long), "context": {"cfg_weight": 5.0, "temperature": 1.0}}
    r2 = GenerationRequest(request_id="r2", family="janus_pro", task="ar_t2i", prompts=["p0", "p1"], samples_per_prompt=2, sampling={})
    sp2 = GenerationIdFactory().build_sample_specs(r2)
    ob = OutputBatch(request_id="r2", family="janus_pro", task="ar_t2i", prompts=["p0", "p1"], sample_specs=sp2, output=torch.rand(B, 3, 8, 8, generator=g), extra=o_extra)
    loop = asyncio.new_event_loop()
    ctx = RolloutPackContext(metadata={}, device=torch.device("cpu"), kl_reward=0.0, rescale_to_unit=True)
    pk = ARDiscreteRolloutPacker()
    flat(res, "disc.reward_outputs", pk.reward_outputs(ob, ctx))
    flat(res, "disc.reward_prompts", pk.reward_prompts(ob, ctx))
    batch = loop.run_until_complete(pk.pack(ob, torch.arange(4.0), ctx))
    flat(res, "disc.batch", {"obs": batch.observations, "act": batch.actions, "rew": batch.rewards, "done": batch.dones.float(), "gid": batch.group_ids.float(), "extras": batch.extras, "ctx": batch.context, "videos": batch.videos, "prompts": batch.prompts})
    class TokPolicy(nn.Module):
        def __init__(self):
            super().__init__()
            torch.manual_seed(1)
            self.emb = nn.Embedding(50, 50)
            self.adapter = True
        def replay_forward(self, batch, timestep_idx=0):
            ids = batch.actions
            logits = self.emb(ids) * (1.0 if self.adapter else 0.5)
            return {"logits": logits, "target_tokens": ids, "log_probs": None}
        @contextlib.contextmanager
        def disable_adapter(self):
            self.adapter = False
            try: yield
            finally: self.adapter = True
        has_adapters = True
        uses_lora = True
    pol = TokPolicy()
    for need_ref in (False, True):
        try:
            s = TokenLogProbEvaluator().evaluate(pol, batch, 0, ref_model=None, signal_request=SignalRequest(need_ref=need_ref))
            flat(res, f"tok.sig{need_ref}", s)
        except Exception as e:
            res[f"tok.err{need_ref}"] = torch.tensor([float(ord(c)) for c in type(e).__name__])
    # continuous packer / evaluator
    D = 4
    c_extra = {"tokens": torch.randn(B, L, D, generator=g), "log_probs": -torch.rand(B, L, generator=g), "saved_noise": torch.randn(B, L, D, generator=g), "token_mask": torch.ones(B, L),
               "prompt_input_ids": o_extra["prompt_input_ids"], "prompt_attention_mask": o_extra["prompt_attention_mask"], "uncond_input_ids": o_extra["uncond_input_ids"],
               "uncond_attention_mask": o_extra["uncond_attention_mask"], "images_for_reward": torch.rand(B, 3, 8, 8, generator=g), "context": {"cfg_scale": 4.5, "num_flow_steps": 3, "noise_level": 1.0}}
    ob2 = OutputBatch(request_id="r2", family="nextstep_1", task="ar_t2i", prompts=["p0", "p1"], sample_specs=sp2, output=torch.rand(B, 3, 8, 8, generator=g) * 2 - 1, extra=c_extra)
    pk2 = ARContinuousRolloutPacker()
    flat(res, "cont.reward_outputs", pk2.reward_outputs(ob2, ctx))
    batch2 = loop.run_until_complete(pk2.pack(ob2, torch.arange(4.0), ctx))
    flat(res, "cont.batch", {"obs": batch2.observations, "act": batch2.actions, "rew": batch2.rewards, "gid": batch2.group_ids.float(), "extras": batch2.extras, "ctx": batch2.context, "videos": batch2.videos})
    class ContPolicy(nn.Module):
        def __init__(self):
            super().__init__()
            self.w = nn.Parameter(torch.tensor(0.3))
            self.adapter = True
        def replay_forward(self, batch, timestep_idx=0):
            lp = -(batch.actions.float() ** 2).sum(-1) * (self.w if self.adapter else self.w.detach() * 0.5)
            return {"log_probs": lp, "target_tokens": batch.actions}
        @contextlib.contextmanager
        def disable_adapter(self):
            self.adapter = False
            try: yield
            finally: self.adapter = True
        has_adapters = True
        uses_lora = True
    cp = ContPolicy()
    for need_ref in (False, True):
        try:
            s = ContinuousTokenLogProbEvaluator().evaluate(cp, batch2, 0, ref_model=None, signal_request=SignalRequest(need_ref=need_ref))
            flat(res, f"cont.sig{need_ref}", s)
        except Exception as e:
            res[f"cont.err{need_ref}"] = torch.tensor([float(ord(c)) for c in type(e).__name__])
    return res
