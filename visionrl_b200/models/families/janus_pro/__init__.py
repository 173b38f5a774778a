"""janus_pro model family."""
from visionrl_b200.models.families.janus_pro.policy import (
    JanusProConfig, JanusProPolicy, image_token_logits_from_hidden,
)

__all__ = ["JanusProConfig", "JanusProPolicy", "image_token_logits_from_hidden"]
