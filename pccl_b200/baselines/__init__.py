"""Library baselines (PyTorch + NCCL + cuBLAS) that the framework's numbers are measured against on the same GPUs."""
