"""The fixed-scratch GEMM entry point (b200_gemm_bf16_fixed_scratch), for hosts that cannot give the
library device memory: a serving loop whose device memory plan is frozen at start-up (cudaMalloc
on the hot path is banned there because it synchronises the device and can fail late), or a
plug-in interface that passes operands only.

Called through the C ABI and compared with the existing entry point (b200_gemm_bf16 with a
caller-supplied workspace), twice in a row so that the second call runs on the scratch contents
the first one left behind. This file sorts last on purpose: it must pass in a fresh process and
after every other test has run.
"""
import ctypes

import numpy as np
import pytest

import util
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max |dC| / (|A_i| |B_j|), the bound the other GPU tests use


def _both(lib, api, torch, M, N, K, seed, alpha=1.0, beta=0.0):
    a_bits = util.normal_bits((M, K), seed)
    b_bits = util.normal_bits((N, K), seed + 1, 0.02)
    a, b = util.to_device(a_bits), util.to_device(b_bits)
    # existing entry point: default configuration, workspace from the caller
    ws_bytes = lib.b200_gemm_workspace_bytes(1, M, N, K, None)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    assert lib.b200_gemm_bf16(M, N, K, a.data_ptr(), b.data_ptr(), ref.data_ptr(), alpha, beta, None, ws.data_ptr(),
                              ws_bytes, None) == api.STATUS_OK
    # new entry point: operands and output only
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    assert lib.b200_gemm_bf16_fixed_scratch(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(), alpha, beta,
                                            None) == api.STATUS_OK
    torch.cuda.synchronize()
    words = (ctypes.c_uint * 4)()
    assert lib.b200_gemm_last_device_status(ctypes.byref(words)) == api.STATUS_OK, list(words)
    return a_bits, b_bits, util.to_bits(out), util.to_bits(ref)


def test_fixed_scratch_matches_workspace_entry_point_twice_in_a_row():
    import torch
    from h100_gemm_b200 import api
    lib = api.library()
    # two different shapes back to back: the second call finds the first call's partial tiles and
    # flag words in the shared array
    for (M, N, K, seed, alpha, beta) in ((48, 4096, 2048, 1, 1.0, 0.0), (128, 3008, 4096, 7, 0.5, 0.25)):
        a_bits, b_bits, got, want = _both(lib, api, torch, M, N, K, seed, alpha, beta)
        assert oracle.norm_relative_error(got, want, a_bits, b_bits) <= TOL
        assert np.array_equal(got, want)  # same kernel, same schedule: the two agree exactly
    # and the same shape twice
    for _ in range(2):
        a_bits, b_bits, got, want = _both(lib, api, torch, 16, 28672, 8192, 3)
        assert oracle.norm_relative_error(got, want, a_bits, b_bits) <= TOL
        assert np.array_equal(got, want)


def test_fixed_scratch_rejects_what_it_cannot_hold():
    import torch
    from h100_gemm_b200 import api
    lib = api.library()
    a = torch.zeros(256, 1024, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(512, 1024, dtype=torch.bfloat16, device="cuda")
    c = torch.zeros(256, 512, dtype=torch.bfloat16, device="cuda")
    # more rows than the few-rows path handles
    assert lib.b200_gemm_bf16_fixed_scratch(256, 512, 1024, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, 0.0,
                                            None) == api.STATUS_STATIC_SCRATCH
    # K that would need re-pitched operand copies
    assert lib.b200_gemm_bf16_fixed_scratch(64, 512, 1001, a.data_ptr(), b.data_ptr(), c.data_ptr(), 1.0, 0.0,
                                            None) == api.STATUS_STATIC_SCRATCH
    assert b"fixed scratch" in lib.b200_gemm_strerror(api.STATUS_STATIC_SCRATCH)
    assert lib.b200_gemm_bf16_fixed_scratch(64, 512, 1024, None, b.data_ptr(), c.data_ptr(), 1.0, 0.0,
                                            None) == api.STATUS_INVALID_ARG
