"""Rollout workers, planner, executor and runtime."""
