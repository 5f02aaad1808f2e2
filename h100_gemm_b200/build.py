"""Builds the native pieces in-tree with nvcc/gcc (no JIT cache, no pip install).

  python -m h100_gemm_b200.build            # libb200gemm.so (+ baselines, oracle)

The CUDA sources are compiled for sm_100a only, with
``-gencode arch=compute_100a,code=sm_100a``: the plain ``-arch=sm_100a`` spelling the reference
uses for Hopper (Makefile:2, gemm_tuner.py:46) also emits a non-"a" PTX target for which ptxas
rejects tcgen05 and setmaxnreg.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
REPO_DIR = PKG_DIR.parent
CSRC = PKG_DIR / "csrc"
LIB_DIR = PKG_DIR / "lib"
LIB_PATH = LIB_DIR / "libb200gemm.so"
BASELINES_PATH = LIB_DIR / "libb200gemm_baselines.so"

NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_COMMON = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC", "-shared"]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found; the CUDA library cannot be built")
    return exe


def _newer(target: Path, sources) -> bool:
    if not target.exists():
        return False
    t = target.stat().st_mtime
    return all(Path(s).stat().st_mtime <= t for s in sources)


def _run(cmd, cwd=None) -> None:
    proc = subprocess.run(cmd, cwd=cwd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError(f"build failed: {' '.join(map(str, cmd))}\n{proc.stdout}\n{proc.stderr}")


def kernel_sources():
    return sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("sm100/*.cuh")) +
                  [REPO_DIR / "include" / "b200_gemm.h"])


def build_library(force: bool = False, verbose: bool = False) -> Path:
    """nvcc -> h100_gemm_b200/lib/libb200gemm.so (the C ABI of include/b200_gemm.h)."""
    LIB_DIR.mkdir(exist_ok=True)
    srcs = kernel_sources()
    if not force and _newer(LIB_PATH, srcs):
        return LIB_PATH
    cmd = [_nvcc(), *NVCC_COMMON, *NVCC_ARCH, "-o", str(LIB_PATH), str(CSRC / "launcher.cu")]
    if verbose:
        cmd += ["-Xptxas", "-v"]
    _run(cmd)
    return LIB_PATH


def build_baselines(force: bool = False) -> Path:
    """cuBLAS / cuBLASLt comparison entry points, kept out of the main library."""
    LIB_DIR.mkdir(exist_ok=True)
    src = CSRC / "baselines" / "cublas_baselines.cu"
    if not src.exists():
        return BASELINES_PATH
    if not force and _newer(BASELINES_PATH, [src]):
        return BASELINES_PATH
    _run([_nvcc(), *NVCC_COMMON, *NVCC_ARCH, "-o", str(BASELINES_PATH), str(src),
          "-lcublas", "-lcublasLt"])
    return BASELINES_PATH


def build_host_shim(force: bool = False) -> Path:
    """g++ -> lib/libb200gemm_hostshim.so: scheduler/descriptor arithmetic for CPU-only tests."""
    LIB_DIR.mkdir(exist_ok=True)
    out = LIB_DIR / "libb200gemm_hostshim.so"
    srcs = [CSRC / "host_shim.cpp", CSRC / "sm100" / "desc.cuh", CSRC / "sm100" / "scheduler.cuh"]
    if not force and _newer(out, srcs):
        return out
    _run(["/usr/bin/g++", "-std=c++17", "-O2", "-x", "c++", "-shared", "-fPIC", "-o", str(out),
          str(CSRC / "host_shim.cpp")])
    return out


def build_oracle() -> None:
    """The CPU checker used by tests and the benchmark's CPU leg (never by the library)."""
    oracle_dir = REPO_DIR / "oracle"
    _run(["make", "-C", str(oracle_dir), "all"])
    # A checkout of the reference project: where B200_REFERENCE_DIR points, else a directory named
    # "reference" beside this repository. Without one only the restatement is built.
    reference = Path(os.environ.get("B200_REFERENCE_DIR") or REPO_DIR.parent / "reference")
    if (reference / "reference.h").exists():
        _run(["make", "-C", str(oracle_dir), "ref", f"REFERENCE={reference}"])


def build_all(force: bool = False) -> None:
    build_library(force=force)
    build_baselines(force=force)
    build_host_shim(force=force)
    build_oracle()


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(LIB_PATH)
