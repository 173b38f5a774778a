"""Headline benchmark: GRPO samples/sec (rollout + train) of the SD3.5-medium-shape MMDiT.

    python bench.py --gpus N --steps K --warmup W [--impl native|torch_baseline|reference]

Workload: 24 joint blocks, hidden 1536, 24 heads, 16x64x64 latents (1024 image tokens), 154 x 4096
context + 2048 pooled (synthetic, seeded), 10 SDE steps with CFG 4.5, 8 prompts x group 8 = 64
samples per step in total (strong scaling: the global batch is fixed, rank r takes prompts
r, r+N, ...), ViT-L/14 scalar reward on the 512x512 image from a 16-channel VAE decoder,
full-parameter bf16 training with the flat sharded AdamW.  Every step runs rollout, reward,
advantages, the per-timestep replay forward/backward and the optimiser update.

Two timings, both through ``OnlineTrainer.step`` (the call a training run makes):
  * ``value``  — K steps between CUDA events, conditioning already resident on the device;
  * ``e2e``    — K steps in which the step's prompt conditioning is copied from pinned host
                 memory and the step's metrics are read back to the host.
Every rank times on its device; the slowest rank defines the result.  The step's working set
(4 GB of weights plus activations) is far larger than the 126 MB L2, so no explicit flush is used.
"""

from __future__ import annotations

import argparse
import asyncio
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "GRPO samples/sec (rollout+train, device-timed, max over ranks)"

# The named benchmark workloads.  `--config` picks one; the default is the headline one.
CONFIGS = {
    "sd3_5": {
        "experiment": "experiment/sd3_5_shape_grpo",
        "model": "SD3.5-medium-shape MMDiT (24 blocks, hidden 1536, 24 heads, 1024+154 tokens)",
        "seq_len": 1024 + 154, "prompts": 8, "group": 8,
        "extra": {"sde_steps": 10, "cfg": 4.5, "train_timesteps": 9,
                  "reward": "ViT-L/14 scalar head on VAE-decoded 512x512"},
    },
    "wan_1_3b": {
        "experiment": "experiment/wan_2_1_1_3b_shape_grpo",
        "model": "Wan-2.1-1.3B-shape video DiT (30 blocks, dim 1536, 12 heads, FFN 8960, 14040 tokens)",
        "seq_len": 14040, "prompts": 2, "group": 8,
        "extra": {"sde_steps": 16, "cfg": 5.0, "reward": "ViT-L/14 scalar head on 4 frames",
                  "mesh": "dp = N / sp, Ulysses sp = min(4, N)"},
    },
    "wan_14b": {
        "experiment": "experiment/wan_2_1_14b_shape_grpo",
        "model": "Wan-2.1-14B-shape video DiT (40 blocks, dim 5120, 40 heads, FFN 13824, 32760 tokens)",
        "seq_len": 32760, "prompts": 1, "group": 4,
        "extra": {"sde_steps": 16, "cfg": 5.0, "reward": "ViT-L/14 scalar head on 4 frames",
                  "mesh": "Ulysses sp = N"},
    },
    "janus": {
        "experiment": "experiment/janus_pro_1b_shape_grpo",
        "model": "Janus-Pro-1B-shape LLaMA decoder (24 layers, hidden 2048, 16 heads, 576 image tokens)",
        "seq_len": 64 + 576, "prompts": 1, "group": 16,
        "extra": {"cfg": 5.0, "decode": "int4 weight-only KV-cache decode",
                  "reward": "ViT-B/16 scalar head on the VQ-decoded image"},
    },
}
MODEL = CONFIGS["sd3_5"]["model"]


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu_index = gpu_index
        self.rows: list[list[str]] = []
        self._proc = None
        self._thread = None

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "200", "-i", str(self.gpu_index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return

        def pump():
            for line in self._proc.stdout:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) >= 9:
                    self.rows.append(parts)

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> dict:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        sm, sm_max, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                sm_max.append(float(r[2]))
            except ValueError:
                continue
            for name, flag in zip(names, r[5:9]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(sm_max) if sm_max else None, "reasons": sorted(reasons),
                "samples": len(sm)}


def reference_arm() -> None:
    """The reference installs offline only with --no-deps; its training path cannot run here."""
    print(json.dumps({
        "impl": "reference",
        "unavailable": "reference stock path needs ray + diffusers + peft + omegaconf and HF "
                       "checkpoints (none installed, no network); it defines no model in-tree",
    }))


def run(args) -> None:
    import inspect

    import torch
    import torch.distributed as dist

    from visionrl_b200.config.loader import load_config
    from visionrl_b200.ops import _ext
    from visionrl_b200.scripts.common import capture_trainer
    from visionrl_b200.scripts.train import run_config

    spec = CONFIGS[args.config]
    if args.prompts is None:
        args.prompts = spec["prompts"]
    if args.group is None:
        args.group = spec["group"]
    baseline = args.impl in ("torch_baseline", "torch_compile_baseline")
    if baseline:
        _ext.set_kernels_enabled(False)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torchrun")
    overrides = [
        f"distributed.collectives={'nccl' if baseline else args.collectives}",
        f"distributed.param_sharding={args.sharding}",
        f"distributed.rollout_replica={'true' if args.rollout_replica else 'false'}",
        "distributed.destroy_on_exit=false",
        "trainer.output_dir=/tmp/vrl_bench", f"rollout.rollout_batch_size={args.prompts}",
    ]
    if args.config == "janus":
        overrides += [f"rollout.n_samples_per_prompt={args.group}"]
    else:
        overrides += [f"rollout.n={args.group}"]
    if args.config == "sd3_5":
        overrides += [f"rollout.sample_batch_size={args.group}"]
    if args.config == "wan_1_3b":
        overrides += [f"distributed.mesh.sp={min(4, args.gpus)}"]
    if args.config == "wan_14b":
        overrides += [f"distributed.mesh.sp={args.gpus}"]
    overrides += list(args.override)
    cfg = load_config(spec["experiment"], overrides=overrides)
    loop = asyncio.new_event_loop()
    # the recipe named by the config builds everything (model, collector, runtime, trainer) exactly
    # as a training run would, then hands the trainer over instead of entering its epoch loop
    with capture_trainer() as box:
        outcome = run_config(cfg)
        if inspect.isawaitable(outcome):
            loop.run_until_complete(outcome)
    trainer, examples = box["trainer"], box["examples"]
    gen = torch.Generator().manual_seed(box["ctx"].trainer_config.seed)
    prompts = [examples[i] for i in torch.randperm(len(examples), generator=gen)[:args.prompts].tolist()]
    rank = dist.get_rank() if dist.is_initialized() else 0
    device = trainer.device
    policy = trainer.model
    if args.impl == "torch_compile_baseline":
        # what the reference's stock diffusion path does to its transformer (comparison arm only)
        policy.transformer = torch.compile(policy.transformer, mode="default", dynamic=False)
    text = getattr(getattr(policy, "backend_handle", None), "text", None)
    if text is None or not hasattr(text, "drop_device_cache"):
        text = _NoHostConditioning()
    samples_per_step = args.prompts * args.group

    def barrier():
        if dist.is_initialized():
            dist.barrier()
        torch.cuda.synchronize()

    async def one_step():
        return await trainer.step(prompts)

    for _ in range(args.warmup):
        loop.run_until_complete(one_step())
    ext_status = [int(v) for v in _ext.load().kernel_status_all()] if not baseline else []
    if any(ext_status):
        raise RuntimeError(f"kernel status words {ext_status} (gemm, attention, int4) during warm-up")
    runtime = getattr(policy, "param_runtime", None)
    sharded = runtime is not None and runtime.active

    def timed(clear_device_cache: bool):
        barrier()
        launches0 = _ext.launch_count
        text.reset_transfer_stats()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        wall0 = time.perf_counter()
        start.record()
        d2h = 0
        for _ in range(args.steps):
            if clear_device_cache:
                text.drop_device_cache()
            m = loop.run_until_complete(one_step())
            d2h += trainer.last_d2h_bytes
        end.record()
        barrier()
        wall = time.perf_counter() - wall0
        ms = start.elapsed_time(end)
        return ms, wall, _ext.launch_count - launches0, text.h2d_bytes, d2h, m

    sampler = ClockSampler(torch.cuda.current_device())
    sampler.start()
    dev_ms, _, launches, _, _, metrics = timed(clear_device_cache=False)
    clocks = sampler.stop()
    e2e_ms, e2e_wall, _, h2d, d2h, _ = timed(clear_device_cache=True)

    def max_over_ranks(value: float) -> float:
        t = torch.tensor([value], device=device, dtype=torch.float64)
        if dist.is_initialized():
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    phases = None
    if args.phases:
        # one more step, outside both timed regions, with a device synchronisation around every
        # phase: where the step's time goes (the synchronisations make it slower than a timed step)
        was = trainer.config.profile
        trainer.config.profile = True
        try:
            barrier()
            pm = loop.run_until_complete(one_step())
        finally:
            trainer.config.profile = was
        phases = {k: round(max_over_ranks(float(v)) * 1e3, 1) for k, v in sorted(pm.phase_times.items())}

    dev_ms = max_over_ranks(dev_ms)
    e2e_s = max_over_ranks(max(e2e_ms / 1e3, e2e_wall))
    launches = int(max_over_ranks(float(launches)))
    value = samples_per_step * args.steps / (dev_ms / 1e3)
    e2e_value = samples_per_step * args.steps / e2e_s
    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 4), "unit": "samples/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(dev_ms / args.steps, 3), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": args.impl,
            "config": {
                "name": args.config, "model": spec["model"], "global_batch": samples_per_step,
                "seq_len": spec["seq_len"],
                "parallelism": ("single" if args.gpus == 1 else f"fsdp{runtime.world}" if sharded
                                else f"dp{args.gpus}+sharded-optimizer"),
                "prompts": args.prompts, "group_size": args.group, **spec["extra"],
                "l2_policy": "working set (GBs of weights + activations) exceeds the 126 MB L2",
                "collectives": "nccl" if baseline else args.collectives,
                "attention": "library SDPA" if baseline else _attention_impl(),
            },
            "clocks": clocks,
            "e2e": ({"value": round(e2e_value, 4), "unit": "samples/s",
                     "h2d_bytes_per_step": int(h2d // max(args.steps, 1)),
                     "d2h_bytes_per_step": int(d2h // max(args.steps, 1))}
                    if not isinstance(text, _NoHostConditioning) else None),
            "gpu_launches": launches,
            "sharding": ({**runtime.memory_report(), "fused_gathers": runtime.fused_gathers,
                          "gathers": runtime.gathers, "standalone_gathers": runtime.standalone_gathers,
                          "gather_ahead_launches": runtime.prefetches, "buckets_reduced": runtime.buckets_reduced,
                          "weight_broadcasts": runtime.broadcasts}
                         if sharded else None),
            "phases_ms": phases,
            "last_metrics": {"loss": metrics.loss, "reward_mean": metrics.reward_mean,
                             "grad_norm": metrics.grad_norm},
        }
        print(json.dumps(line))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


class _NoHostConditioning:
    """Stand-in for families whose prompt conditioning is not staged through pinned host memory
    (no end-to-end figure is reported for them)."""

    h2d_bytes = 0

    def reset_transfer_stats(self) -> None:
        return None

    def drop_device_cache(self) -> None:
        return None


def _attention_impl() -> str:
    from visionrl_b200.ops import attention as A

    return ("own tcgen05 forward + backward" if A.backward_impl() == "own"
            else "own tcgen05 forward (no-grad calls), library SDPA under autograd")


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=2)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="native",
                        choices=["native", "torch_baseline", "torch_compile_baseline", "reference"],
                        help="native: this repository's kernels; torch_baseline: the same models in "
                             "eager PyTorch (cuBLAS + SDPA + NCCL); torch_compile_baseline: that, with "
                             "the transformer under torch.compile as the reference's stock path has "
                             "it; reference: the unmodified reference package")
    parser.add_argument("--config", default="sd3_5", choices=sorted(CONFIGS),
                        help="which named workload to run (default: the headline one)")
    parser.add_argument("--collectives", default="fused", choices=["fused", "nccl"])
    parser.add_argument("--sharding", default="full", choices=["full", "optimizer_only"],
                        help="full: block weights, gradients and optimiser state sharded over the "
                             "ranks (FSDP); optimizer_only: replicated bf16 weights")
    parser.add_argument("--no-rollout-replica", dest="rollout_replica", action="store_false",
                        help="rollouts gather the sharded weights like training does instead of "
                             "reading a full per-rank replica kept current by the P2P broadcast")
    parser.add_argument("--phases", action="store_true",
                        help="after the timed regions, run one synchronised step and report the time "
                             "of each phase (collect, evaluate, backward, optimiser, ...)")
    parser.add_argument("--prompts", type=int, default=None, help="default: the config's own")
    parser.add_argument("--group", type=int, default=None, help="default: the config's own")
    parser.add_argument("--override", action="append", default=[],
                        help="extra config override, e.g. model.arch.num_layers=4")
    args = parser.parse_args()
    if args.warmup < 3:
        print("note: fewer than 3 warm-up steps; the number is not a valid headline", file=sys.stderr)
    if args.impl == "reference":
        reference_arm()
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    run(args)


if __name__ == "__main__":
    main()
