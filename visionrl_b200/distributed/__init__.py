"""Distributed backends: ``native`` (torch.distributed ranks, one per GPU) and the
``ray`` facade that keeps the reference's launcher / worker / executor names."""
