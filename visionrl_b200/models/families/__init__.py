"""Native model families (policy, executor, builder per family)."""
