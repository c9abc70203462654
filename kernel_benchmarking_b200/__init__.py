"""Fused RMSNorm -> Linear for NVIDIA B200 (sm_100a): hand-written CUDA behind a C ABI.

`rmsnorm_linear(x, gamma, W, eps) -> y` keeps the call surface of the kernels that
dungwoong/kernel-benchmarking profiles (demo/rmsnorm_linear.py).  There is no CPU
or PyTorch fallback: the compiled library must be present.
"""
from .host import HostRMSNormLinear  # noqa: F401
from .ops import (check_status, gemm_nt, lora_linear, quantize_rows_e4m3, rmsnorm_linear, rmsnorm_swiglu,  # noqa: F401
                  row_stats)

__all__ = ["rmsnorm_linear", "quantize_rows_e4m3", "check_status", "HostRMSNormLinear", "gemm_nt", "rmsnorm_swiglu",
           "row_stats", "lora_linear"]
