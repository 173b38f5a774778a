"""Rollout runtime selection and launch inputs."""

from visionrl_b200.rollouts.runtime.backend import (
    DRIVER_CUDA_OWNERSHIP_ERROR, ReleasableRayRolloutBackend, build_rollout_backend_from_cfg,
    validate_rollout_backend_config,
)
from visionrl_b200.rollouts.runtime.config import RolloutBackendConfig
from visionrl_b200.rollouts.runtime.launch_inputs import (
    RolloutRuntimeInputs, build_rollout_runtime_inputs,
)

__all__ = ["DRIVER_CUDA_OWNERSHIP_ERROR", "ReleasableRayRolloutBackend", "RolloutBackendConfig",
           "RolloutRuntimeInputs", "build_rollout_backend_from_cfg",
           "build_rollout_runtime_inputs", "validate_rollout_backend_config"]
