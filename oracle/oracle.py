"""TEST INFRASTRUCTURE — NOT A PRODUCT PATH.

ctypes access to the CPU oracle (oracle/cpu_gemm.c, a restatement of reference.h:5-46) and,
when it has been built from a checkout of the reference, to the real reference oracle
(oracle/_ref/libref_gemm.so, built by oracle/Makefile from reference.h where it lies).
Only tests, the smoke check and the benchmark's CPU-baseline leg import this module.

All matrices are numpy uint16 arrays holding bf16 bit patterns: A is [M,K], B is [N,K], both
K-contiguous; C = A * B^T is [M,N] row-major.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_DIR = Path(__file__).resolve().parent
_ORACLE_SO = _DIR / "liboracle_gemm.so"
_REF_SO = _DIR / "_ref" / "libref_gemm.so"
_oracle = None
_ref = None


def _load_oracle() -> ctypes.CDLL:
    global _oracle
    if _oracle is None:
        if not _ORACLE_SO.exists():
            subprocess.run(["make", "-C", str(_DIR), "all"], check=True, capture_output=True)
        lib = ctypes.CDLL(str(_ORACLE_SO))
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.oracle_cpu_gemm_bf16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf]
        lib.oracle_cpu_gemm_bf16.restype = None
        lib.oracle_cpu_gemm_bf16_rows.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf, ci, ci]
        lib.oracle_cpu_gemm_bf16_rows.restype = None
        lib.oracle_cpu_gemm_bf16_sampled_rows.argtypes = [ci, ci, vp, vp, vp, cf, cf, vp, ci]
        lib.oracle_cpu_gemm_bf16_sampled_rows.restype = None
        lib.oracle_cpu_gemm_f16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf]
        lib.oracle_cpu_gemm_f16.restype = None
        lib.oracle_f32_to_bf16.argtypes = [cf]
        lib.oracle_f32_to_bf16.restype = ctypes.c_uint16
        _oracle = lib
    return _oracle


def have_reference() -> bool:
    return _REF_SO.exists()


def _load_ref() -> ctypes.CDLL:
    global _ref
    if _ref is None:
        lib = ctypes.CDLL(str(_REF_SO))
        vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
        lib.ref_cpu_gemm_bf16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf]
        lib.ref_cpu_gemm_bf16.restype = None
        if hasattr(lib, "ref_cpu_gemm_f16"):
            lib.ref_cpu_gemm_f16.argtypes = [ci, ci, ci, vp, vp, vp, cf, cf]
            lib.ref_cpu_gemm_f16.restype = None
        _ref = lib
    return _ref


def set_threads(n: int) -> None:
    """OpenMP threads for the oracle and, when built, the reference library."""
    lib = _load_oracle()
    lib.oracle_set_threads.argtypes = [ctypes.c_int]
    lib.oracle_set_threads(int(n))
    if have_reference():
        ref = _load_ref()
        if hasattr(ref, "ref_set_threads"):
            ref.ref_set_threads.argtypes = [ctypes.c_int]
            ref.ref_set_threads(int(n))


def _check(a: np.ndarray, b: np.ndarray):
    assert a.dtype == np.uint16 and b.dtype == np.uint16
    assert a.ndim == 2 and b.ndim == 2 and a.shape[1] == b.shape[1]
    return np.ascontiguousarray(a), np.ascontiguousarray(b)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (NaN -> 0x7FFF), as cuda_bf16.h does."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (u & 0x7FFFFFFF) > 0x7F800000
    r = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)
    r[nan] = 0x7FFF
    return r


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def cpu_gemm(a: np.ndarray, b: np.ndarray, alpha: float = 1.0, beta: float = 0.0) -> np.ndarray:
    """The oracle: reference.h:5-46 semantics, bit patterns in, bit patterns out."""
    a, b = _check(a, b)
    M, K = a.shape
    N = b.shape[0]
    c = np.empty((M, N), dtype=np.uint16)
    _load_oracle().oracle_cpu_gemm_bf16(M, N, K, a.ctypes.data, b.ctypes.data, c.ctypes.data, alpha, beta)
    return c


def cpu_gemm_rows(a: np.ndarray, b: np.ndarray, rows, alpha: float = 1.0, beta: float = 0.0) -> np.ndarray:
    """Oracle result for the selected rows of C only: returns [len(rows), N]."""
    a, b = _check(a, b)
    rows = np.ascontiguousarray(rows, dtype=np.int32)
    N, K = b.shape
    c = np.empty((len(rows), N), dtype=np.uint16)
    _load_oracle().oracle_cpu_gemm_bf16_sampled_rows(N, K, a.ctypes.data, b.ctypes.data, c.ctypes.data,
                                                     alpha, beta, rows.ctypes.data, len(rows))
    return c


def reference_cpu_gemm(a: np.ndarray, b: np.ndarray, alpha: float = 1.0, beta: float = 0.0) -> np.ndarray:
    """The reference's own reference_cpu_gemm (needs oracle/_ref, see oracle/Makefile)."""
    a, b = _check(a, b)
    M, K = a.shape
    N = b.shape[0]
    c = np.empty((M, N), dtype=np.uint16)
    _load_ref().ref_cpu_gemm_bf16(M, N, K, a.ctypes.data, b.ctypes.data, c.ctypes.data, alpha, beta)
    return c


def f32_to_f16_bits(x: np.ndarray) -> np.ndarray:
    """fp32 -> IEEE half bit patterns (numpy's conversion is round-to-nearest-even)."""
    return np.ascontiguousarray(x, dtype=np.float32).astype(np.float16).view(np.uint16)


def f16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def cpu_gemm_f16(a: np.ndarray, b: np.ndarray, alpha: float = 1.0, beta: float = 0.0) -> np.ndarray:
    """The oracle for fp16 inputs/outputs (reference_cpu_gemm<half_t,half_t,half_t,float>)."""
    a, b = _check(a, b)
    M, K = a.shape
    N = b.shape[0]
    c = np.empty((M, N), dtype=np.uint16)
    _load_oracle().oracle_cpu_gemm_f16(M, N, K, a.ctypes.data, b.ctypes.data, c.ctypes.data, alpha, beta)
    return c


def reference_cpu_gemm_f16(a: np.ndarray, b: np.ndarray, alpha: float = 1.0, beta: float = 0.0) -> np.ndarray:
    a, b = _check(a, b)
    M, K = a.shape
    N = b.shape[0]
    c = np.empty((M, N), dtype=np.uint16)
    _load_ref().ref_cpu_gemm_f16(M, N, K, a.ctypes.data, b.ctypes.data, c.ctypes.data, alpha, beta)
    return c


def norm_relative_error(c_bits: np.ndarray, ref_bits: np.ndarray, a_bits: np.ndarray, b_bits: np.ndarray,
                        f16: bool = False) -> float:
    """max_ij |C_ij - R_ij| / (||A_i||_2 * ||B_j||_2): the acceptance metric (bound 1e-2)."""
    widen = f16_bits_to_f32 if f16 else bf16_bits_to_f32
    a = widen(a_bits).astype(np.float64)
    b = widen(b_bits).astype(np.float64)
    na = np.sqrt((a * a).sum(axis=1))
    nb = np.sqrt((b * b).sum(axis=1))
    denom = np.outer(na, nb)
    denom[denom == 0] = 1.0
    d = np.abs(widen(c_bits).astype(np.float64) - widen(ref_bits).astype(np.float64))
    return float((d / denom).max())
