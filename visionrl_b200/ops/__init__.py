"""Hot operators: sm_100a kernels with PyTorch fp32 oracles of the same math."""
