"""Reward assets (weights are loaded from user-provided paths)."""
