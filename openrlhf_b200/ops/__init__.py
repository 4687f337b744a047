"""Operator layer: every hot op has a CUDA kernel (sm_100a) and a plain PyTorch restatement used on CPU by tests."""
