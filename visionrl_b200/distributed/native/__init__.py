"""Native torch.distributed backend."""
