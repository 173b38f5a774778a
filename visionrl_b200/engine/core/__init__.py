"""Engine core: payload types, executor protocols, registry, worker and runtime."""
