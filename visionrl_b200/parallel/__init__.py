"""Process mesh, symmetric memory, sharded parameters, sequence parallelism, weight broadcast."""
