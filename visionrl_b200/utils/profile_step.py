"""Kernel-time breakdown of one training step of any online recipe.

``python -m visionrl_b200.utils.profile_step [--config experiment/sd3_5_shape_grpo] [--prompts 1]
[--torch-baseline] [--rows 40] [key=value ...]`` lets the recipe named by the config build its trainer
exactly as a training run would, runs one warm-up step, then records one step (rollout, reward,
replay, backward, optimizer) with the PyTorch profiler and prints the CUDA kernels sorted by device
time; kernels replayed from a CUDA graph (the autoregressive decode step) are listed like any other.
The reference reaches the same information through ``torch.profiler`` hooks in its trainer loop
(``vrl/trainers/online.py``); here it is a stand-alone tool so that a profile never perturbs a timed run.
"""

from __future__ import annotations

import argparse
import asyncio
import inspect

import torch


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(prog="visionrl_b200.utils.profile_step")
    parser.add_argument("--config", default="experiment/sd3_5_shape_grpo")
    parser.add_argument("--prompts", type=int, default=1, help="prompt groups per step (rollout_batch_size)")
    parser.add_argument("--torch-baseline", action="store_true", help="switch every custom kernel off")
    parser.add_argument("--rows", type=int, default=40)
    parser.add_argument("overrides", nargs="*", help="extra key=value config overrides")
    args = parser.parse_args(argv)
    if not torch.cuda.is_available():
        print("profile_step needs a CUDA device")
        return 1

    from torch.profiler import ProfilerActivity, profile

    from visionrl_b200.config.loader import load_config
    from visionrl_b200.ops import _ext
    from visionrl_b200.scripts.common import capture_trainer
    from visionrl_b200.scripts.train import run_config

    if args.torch_baseline:
        _ext.set_kernels_enabled(False)
    cfg = load_config(args.config, overrides=[f"rollout.rollout_batch_size={args.prompts}",
                                              "trainer.output_dir=/tmp/vrl_profile_step",
                                              "distributed.destroy_on_exit=false", *args.overrides])
    loop = asyncio.new_event_loop()
    with capture_trainer() as box:
        outcome = run_config(cfg)
        if inspect.isawaitable(outcome):
            loop.run_until_complete(outcome)
    trainer = box["trainer"]
    prompts = list(box["examples"])[:args.prompts]
    loop.run_until_complete(trainer.step(prompts))                      # warm-up: allocator, autotuned paths
    torch.cuda.synchronize()
    with profile(activities=[ProfilerActivity.CUDA, ProfilerActivity.CPU]) as prof:
        loop.run_until_complete(trainer.step(prompts))
        torch.cuda.synchronize()
    print(prof.key_averages().table(sort_by="self_cuda_time_total", row_limit=args.rows,
                                    max_name_column_width=64))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
