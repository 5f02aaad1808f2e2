"""Out-of-bounds-store detection for every way the epilogue writes C.

C sits in the middle of a larger device buffer filled with a sentinel bit pattern; after the call
the sentinel words before and after C must be untouched, and C itself must equal the CPU oracle
bit for bit (integer-valued inputs), which also catches a store that lands in the wrong place
inside C. The shapes have tails in M and N, so the last tiles of every row and column band are
partly outside the matrix. The reference guards the same spot with per-element predicates
(matmul_h100.cu.jinja:689-698) and asserts on its tensor-map extents (tma.cuh:95-148).
"""
import numpy as np
import pytest

import util
from oracle import oracle

pytestmark = pytest.mark.gpu

GUARD = 8192          # sentinel elements on each side of C (a multiple of 8: C stays 16-byte aligned)
SENTINEL = 0x7FC5     # a NaN pattern no result can take (results here are small integers)


def _cases():
    from h100_gemm_b200.api import GemmConfig as C
    tails = (300, 520, 264)        # N % 8 == 0: TMA / vector / staged stores are eligible
    odd_n = (300, 517, 264)        # N % 8 != 0: rows of C are not 16-byte aligned -> 2-byte stores
    few = (40, 1000, 520)          # few rows: operands swapped inside, transposed stores
    return [
        ("tma-pair-128x256", C(block_m=128, block_n=256, cluster_m=2, epilogue=1), tails),
        ("tma-single-128x64", C(block_m=128, block_n=64, cluster_m=1, epilogue=1), tails),
        ("tma-drained-256x256-pair", C(block_m=256, block_n=256, cluster_m=2, epilogue=1), (700, 776, 328)),
        ("tma-drained-256x256-single", C(block_m=256, block_n=256, cluster_m=1, epilogue=1), (700, 776, 328)),
        ("vector-128x256", C(block_m=128, block_n=256, cluster_m=2, epilogue=2), tails),
        ("vector-256x256", C(block_m=256, block_n=256, cluster_m=2, epilogue=2), (700, 776, 328)),
        ("staged-128x192", C(block_m=128, block_n=192, cluster_m=1, epilogue=3), tails),
        ("staged-256x256", C(block_m=256, block_n=256, cluster_m=2, epilogue=3), (700, 776, 328)),
        # 224-column tiles end in half a chunk: three TMA boxes and 32 columns from registers.
        # 520 = 224 + 224 + 72 (the last tile's half chunk lies beyond N), 424 = 224 + 192 + 8 (eight
        # live columns in the half chunk), 517: 2-byte stores
        ("tma-128x224", C(block_m=128, block_n=224, cluster_m=1, epilogue=1), tails),
        ("tma-128x224-partial-half-chunk", C(block_m=128, block_n=224, cluster_m=1, epilogue=1), (300, 424, 264)),
        ("vector-128x224", C(block_m=128, block_n=224, cluster_m=1, epilogue=2), (100, 1120, 264)),
        ("scalar-odd-n-128x224", C(block_m=128, block_n=224, cluster_m=1), (300, 445, 264)),
        ("default-128-rows-decode", None, (128, 2240, 520)),
        ("scalar-odd-n", C(block_m=128, block_n=128, cluster_m=1), odd_n),
        ("scalar-odd-n-256x256", C(block_m=256, block_n=256, cluster_m=2), (700, 773, 328)),
        ("few-rows-16", C(block_m=16, block_n=128, cluster_m=1), few),
        ("few-rows-64-pair", C(block_m=64, block_n=128, cluster_m=2, swap_ab=1), few),
        ("few-rows-32-two-subtiles", C(block_m=32, block_n=256, cluster_m=1, swap_ab=1), few),
        ("few-rows-128-pair-two-subtiles", C(block_m=128, block_n=256, cluster_m=2, swap_ab=1), (100, 1000, 520)),
        ("stream-k-finisher-tma", C(block_m=128, block_n=256, cluster_m=2, sched=2, epilogue=1), tails),
        ("stream-k-finisher-vector", C(block_m=128, block_n=128, cluster_m=1, sched=2, epilogue=2), (100, 1000, 2056)),
        ("stream-k-finisher-few-rows", C(block_m=32, block_n=128, cluster_m=1, sched=2), (24, 1000, 2056)),
        ("split-k-fixup", C(block_m=128, block_n=128, cluster_m=1, sched=1, split_k=3), tails),
        ("hybrid", C(block_m=128, block_n=64, cluster_m=1, sched=3), tails),
        ("column-major", C(block_m=128, block_n=128, cluster_m=1, c_col_major=1), tails),
        ("default", None, tails),
        ("default-few-rows", None, few),
    ]


@pytest.mark.parametrize("name,cfg,shape", _cases(), ids=[c[0] for c in _cases()])
def test_stores_stay_inside_c(name, cfg, shape):
    import torch
    import h100_gemm_b200 as g
    M, N, K = shape
    a_bits, b_bits = util.integer_bits((M, K), 3), util.integer_bits((N, K), 4)
    a, b = util.to_device(a_bits), util.to_device(b_bits)
    col_major = cfg is not None and cfg.c_col_major
    buf = torch.full((GUARD + M * N + GUARD,), SENTINEL, dtype=torch.int16,
                     device="cuda").view(torch.bfloat16)
    out = buf[GUARD:GUARD + M * N].view((N, M) if col_major else (M, N))
    g.gemm(a, b, out=out, cfg=cfg)
    rc, words = g.device_status()
    assert rc == 0, f"device status {words}"
    raw = buf.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.all(raw[:GUARD] == SENTINEL), f"{name}: store before C at {np.flatnonzero(raw[:GUARD] != SENTINEL)[:4]}"
    assert np.all(raw[GUARD + M * N:] == SENTINEL), \
        f"{name}: store after C at {np.flatnonzero(raw[GUARD + M * N:] != SENTINEL)[:4]}"
    got = raw[GUARD:GUARD + M * N].reshape((N, M) if col_major else (M, N))
    want = oracle.cpu_gemm(a_bits, b_bits)
    assert np.array_equal(got.T if col_major else got, want)


def test_fixed_scratch_and_batched_stores_stay_inside_c():
    import torch
    import h100_gemm_b200 as g
    # the entry point that keeps its partial tiles in the library's own array
    M, N, K = 100, 1000, 2056
    a_bits, b_bits = util.integer_bits((M, K), 5), util.integer_bits((N, K), 6)
    buf = torch.full((GUARD + M * N + GUARD,), SENTINEL, dtype=torch.int16, device="cuda").view(torch.bfloat16)
    g.gemm_fixed_scratch(util.to_device(a_bits), util.to_device(b_bits), out=buf[GUARD:GUARD + M * N].view(M, N))
    assert g.device_status()[0] == 0
    raw = buf.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.all(raw[:GUARD] == SENTINEL) and np.all(raw[GUARD + M * N:] == SENTINEL)
    assert np.array_equal(raw[GUARD:GUARD + M * N].reshape(M, N), oracle.cpu_gemm(a_bits, b_bits))
    # batched: three problems back to back, tails in M and N
    batch, M, N, K = 3, 200, 264, 136
    a_bits, b_bits = util.integer_bits((batch, M, K), 7), util.integer_bits((batch, N, K), 8)
    buf = torch.full((GUARD + batch * M * N + GUARD,), SENTINEL, dtype=torch.int16, device="cuda").view(torch.bfloat16)
    g.gemm_batched(util.to_device(a_bits), util.to_device(b_bits), out=buf[GUARD:GUARD + batch * M * N].view(batch, M, N))
    assert g.device_status()[0] == 0
    raw = buf.view(torch.int16).cpu().numpy().view(np.uint16)
    assert np.all(raw[:GUARD] == SENTINEL) and np.all(raw[GUARD + batch * M * N:] == SENTINEL)
    for i in range(batch):
        assert np.array_equal(raw[GUARD + i * M * N:GUARD + (i + 1) * M * N].reshape(M, N),
                              oracle.cpu_gemm(a_bits[i], b_bits[i]))
