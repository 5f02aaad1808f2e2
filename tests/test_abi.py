"""The C-ABI library loads on a machine without a GPU and exports what include/b200_gemm.h declares.
No compute entry point is called here."""
import ctypes
import re
from pathlib import Path

import pytest

from h100_gemm_b200 import api, build

REPO = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def lib():
    build.build_library()
    return api.library()


def declared_functions():
    text = (REPO / "include" / "b200_gemm.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_functions()
    for want in ("b200_gemm_bf16", "b200_gemm_batched_bf16", "b200_gemm_workspace_bytes", "b200_run_kernel",
                 "b200_gemm_bf16_host", "b200_reference_gpu_gemm_bf16", "b200_gemm_last_device_status",
                 "b200_gemm_strerror"):
        assert want in names


def test_library_exports_every_declared_symbol(lib):
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} is declared in include/b200_gemm.h but not exported"


def test_library_does_not_link_cublas_or_libcuda(lib):
    # The product library carries its own kernels only; vendor GEMMs live in the separate
    # baselines library, and libcuda is reached through the runtime's driver entry points.
    import subprocess
    needed = subprocess.run(["readelf", "-d", str(build.LIB_PATH)], capture_output=True, text=True).stdout
    needed = [line for line in needed.splitlines() if "NEEDED" in line]
    assert needed and not any("cublas" in n or "libcuda" in n or "nccl" in n for n in needed)


def test_strerror(lib):
    assert lib.b200_gemm_strerror(0) == b"success"
    assert b"workspace" in lib.b200_gemm_strerror(4)
    assert b"unknown" in lib.b200_gemm_strerror(12345)


def test_workspace_sizes(lib):
    C = api.GemmConfig
    # data-parallel, aligned: nothing
    assert api.workspace_bytes(1, 8192, 8192, 8192, C()) == 0
    # K not a multiple of 8: re-pitched copies of A and B at pitch 5560
    assert api.workspace_bytes(1, 1000, 3000, 5555, C()) >= (1000 + 3000) * 5560 * 2
    # split-K: split_k * tiles fp32 tiles
    cfg = C(block_n=128, cluster_m=1, sched=1, split_k=4)
    assert api.workspace_bytes(1, 128, 1024, 4096, cfg) == 4 * 8 * 128 * 128 * 4
    # stream-K: one slot per worker plus 16 flag words each. 148 SMs are assumed without a device;
    # 224 tiles are streamed by 140 of them (8 tiles per 5 workers: few tiles are cut)
    cfg = C(block_n=128, cluster_m=1, sched=2)
    assert api.workspace_bytes(1, 64, 28672, 8192, cfg) == 140 * 128 * 128 * 4 + 140 * 128
    # 37 tiles on 148 workers: every tile is cut in four, all workers are used
    assert api.workspace_bytes(1, 64, 37 * 128, 8192, cfg) == 148 * 128 * 128 * 4 + 148 * 128
    # invalid sizes / unsupported configurations need nothing and report nothing
    assert api.workspace_bytes(1, 0, 10, 10, None) == 0
    assert api.workspace_bytes(1, 128, 128, 128, C(block_n=100)) == 0


def test_default_config(lib):
    c = api.default_config(1, 8192, 8192, 8192)
    assert (c.block_m, c.block_n, c.block_k, c.cluster_m, c.cluster_n) == (256, 256, 64, 2, 1)
    assert c.stages >= 3
    # decode shape: the 16 rows ride the MMA's N (16 x 128 tiles), K split evenly over the SMs
    s = api.default_config(1, 16, 28672, 8192)
    assert (s.block_m, s.block_n, s.sched, s.cluster_m) == (16, 128, 2, 1)
    assert s.stages == 9                                          # the shipped table's measured entry
    assert api.heuristic_config(1, 16, 28672, 8192).stages == 0  # the heuristic leaves it to "as many as fit"
    assert api.default_config(1, 33, 28672, 8192).block_m == 64
    assert api.default_config(1, 16, 8192, 8192).sched == 0      # up to one wave of tiles: whole tiles
    # 65..128 rows keep 128-row tiles with a short A stage: whole 224-column tiles while they fit one
    # wave, stream-K over 128-column tiles beyond
    t = api.default_config(1, 90, 28672, 8192)
    assert (t.block_m, t.block_n, t.sched, t.cluster_m, t.epilogue) == (128, 224, 0, 1, 2)
    t = api.default_config(1, 90, 256 * 200, 8192)
    assert (t.block_m, t.block_n, t.sched, t.cluster_m) == (128, 128, 2, 1)
    # nearly 128 rows and no more 224-column tiles than SMs: one whole 128 x 224 tile per SM, stored from
    # registers; 256-column tiles when only those fit one wave
    t = api.default_config(1, 128, 28672, 8192)
    assert (t.block_m, t.block_n, t.sched, t.cluster_m, t.epilogue) == (128, 224, 0, 1, 2)
    t = api.default_config(1, 128, 256 * 140, 8192)
    assert (t.block_m, t.block_n, t.sched, t.cluster_m, t.epilogue) == (128, 256, 0, 1, 1)
    t = api.default_config(1, 128, 256 * 200, 8192)
    assert (t.block_m, t.block_n, t.sched) == (128, 128, 2)
    # few-rows stream-K workspace: one 128 x 16 fp32 slot and 16 flag words per SM
    assert api.workspace_bytes(1, 16, 28672, 8192, None) == 140 * 128 * 16 * 4 + 140 * 128
    with pytest.raises(api.GemmError):
        api.default_config(1, 0, 1, 1)


def test_python_binding_refuses_cpu_tensors(lib):
    import torch
    a = torch.zeros(4, 8, dtype=torch.bfloat16)
    with pytest.raises(api.GemmError):
        api.gemm(a, a)
