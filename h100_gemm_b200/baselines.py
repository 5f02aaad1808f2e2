"""ctypes binding of the vendor-library baselines (libb200gemm_baselines.so): cuBLAS cublasGemmEx
and cuBLASLt, bf16 with fp32 compute, on the same K-major operands as the GEMM under test.
Reported baselines only (the comparison harnesses of matmul_h100_optimal.cu:63-84,
cublas_ref/spmm_test.cu and cublaslt_matmul.cu); never on the product path."""
from __future__ import annotations

import ctypes
from pathlib import Path

_PATH = Path(__file__).resolve().parent / "lib" / "libb200gemm_baselines.so"
_lib = None


def library() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not _PATH.exists():
            raise RuntimeError(f"{_PATH} is missing: run `python -m h100_gemm_b200.build`")
        import torch  # noqa: F401  (makes the CUDA libraries torch ships resolvable first)
        lib = ctypes.CDLL(str(_PATH))
        vp, ci = ctypes.c_void_p, ctypes.c_int
        lib.b200_baseline_cublas_gemm_bf16.argtypes = [ci, ci, ci, vp, vp, vp, ci, vp]
        lib.b200_baseline_cublas_gemm_bf16.restype = ci
        lib.b200_baseline_cublaslt_gemm_bf16.argtypes = [ci, ci, ci, vp, vp, vp, vp]
        lib.b200_baseline_cublaslt_gemm_bf16.restype = ci
        lib.b200_baseline_last_status.restype = ci
        _lib = lib
    return _lib


def _run(fn, a, b, out, *extra):
    import torch
    M, K = a.shape
    N = b.shape[0]
    stream = torch.cuda.current_stream().cuda_stream or None
    if fn(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(), *extra, stream) != 0:
        raise RuntimeError(f"baseline call failed (cuBLAS status {library().b200_baseline_last_status()})")
    return out


def cublas_gemm(a, b, out=None, c_col_major: bool = False):
    """C = a @ b^T via cublasGemmEx; `out` is [M,N], or [N,M] when c_col_major."""
    import torch
    if out is None:
        shape = (b.shape[0], a.shape[0]) if c_col_major else (a.shape[0], b.shape[0])
        out = torch.empty(shape, dtype=torch.bfloat16, device=a.device)
    return _run(library().b200_baseline_cublas_gemm_bf16, a, b, out, 1 if c_col_major else 0)


def cublaslt_gemm(a, b, out=None):
    """C[M,N] = a @ b^T via cublasLtMatmul (heuristic top-1, 32 MiB workspace)."""
    import torch
    if out is None:
        out = torch.empty((a.shape[0], b.shape[0]), dtype=torch.bfloat16, device=a.device)
    return _run(library().b200_baseline_cublaslt_gemm_bf16, a, b, out)
