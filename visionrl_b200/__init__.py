"""visionrl_b200 — Blackwell-native RL post-training for visual generative models.

The package keeps the public surface of the reference project (importable as
``vrl.*`` through the alias package next to this one) and adds three
B200-specific layers:

* ``visionrl_b200.ops``      — hand-written sm_100a kernels and their PyTorch oracles
* ``visionrl_b200.parallel`` — process mesh, symmetric memory, sharded-parameter
  runtime, Ulysses sequence parallelism and device-side weight broadcast
* ``visionrl_b200.models.nn``— native model definitions built from shape specs
"""

__version__ = "0.1.0"
