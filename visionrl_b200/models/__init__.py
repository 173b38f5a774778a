"""Model contracts, registries and native model families."""

from visionrl_b200.models.diffusion import DiffusionPolicy, VideoGenerationRequest
from visionrl_b200.models.registry import list_models, register_model, resolve_model

__all__ = ["DiffusionPolicy", "VideoGenerationRequest", "list_models", "register_model",
           "resolve_model"]
