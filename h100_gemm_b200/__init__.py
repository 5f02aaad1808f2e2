"""B200 (sm_100a) dense bf16 GEMM, C = A * B^T, behind a C ABI (include/b200_gemm.h).

The package holds the CUDA sources (``csrc/``), the in-tree build (``build.py``), a ctypes
binding of the C ABI (``api.py``), the benchmark template and the tuner that mirror the
reference's matmul_h100.cu.jinja / gemm_tuner.py (``bench/``, ``tuner/``).
There is no CPU or library fallback: importing ``api`` without the built shared object, or
calling it without a CUDA device, raises.
"""
from .api import (GemmConfig, GemmError, default_config, device_status, gemm, gemm_batched,
                  gemm_fixed_scratch, gemm_host, heuristic_config, library, reference_gpu_gemm, run_kernel, tuning_add,
                  tuning_clear, tuning_load, tuning_size, workspace_bytes)

__all__ = ["GemmConfig", "GemmError", "default_config", "device_status", "gemm", "gemm_batched",
           "gemm_fixed_scratch", "gemm_host", "heuristic_config", "library", "reference_gpu_gemm", "run_kernel", "tuning_add",
           "tuning_clear", "tuning_load", "tuning_size", "workspace_bytes"]
