"""Blackwell-native CausalLM training framework (PyTorch + sm_100a CUDA kernels + NCCL/NVLink)."""

__version__ = "0.1.0"
