"""The fixed-scratch GEMM entry point (b200_gemm_bf16_fixed_scratch), for hosts that cannot give the
library device memory: a serving loop whose device memory plan is frozen at start-up (cudaMalloc
on the hot path is banned there because it synchronises the device and can fail late), or a
plug-in interface that passes operands only.

Called through the C ABI and checked against the CPU oracle and against the existing entry point
(b200_gemm_bf16 with the same configuration and a caller-supplied workspace), twice in a row so
that the second call runs on the scratch contents the first one left behind; a second test checks
that calls leave the amount of free device memory unchanged. This file sorts last on purpose: it
must pass in a fresh process and after every other test has run.
"""
import ctypes

import numpy as np
import pytest

import util
from oracle import oracle

pytestmark = pytest.mark.gpu
TOL = 1e-2  # max |dC| / (|A_i| |B_j|), the bound the other GPU tests use


def _operands(M, N, K, seed, integer):
    if integer:
        a_bits, b_bits = util.integer_bits((M, K), seed), util.integer_bits((N, K), seed + 1)
    else:
        a_bits, b_bits = util.normal_bits((M, K), seed), util.normal_bits((N, K), seed + 1, 0.02)
    return a_bits, b_bits, util.to_device(a_bits), util.to_device(b_bits)


def _status_ok(lib, api):
    words = (ctypes.c_uint * 4)()
    assert lib.b200_gemm_last_device_status(ctypes.byref(words)) == api.STATUS_OK, list(words)


def _fixed_scratch(lib, api, torch, a, b, M, N, K, alpha, beta, out=None):
    """The entry point under test: operands and output only, through the C ABI."""
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    out.fill_(float("nan"))
    assert lib.b200_gemm_bf16_fixed_scratch(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(), alpha, beta,
                                            None) == api.STATUS_OK
    torch.cuda.synchronize()
    _status_ok(lib, api)
    return out


def _workspace_entry_point(lib, api, torch, a, b, M, N, K, alpha, beta):
    """The existing entry point with the SAME configuration the fixed-scratch call uses (its own
    pinned few-rows plan, which ignores the tuning table) and a caller-supplied workspace."""
    cfg = api._Cfg()
    assert lib.b200_gemm_fixed_scratch_cfg(M, N, K, ctypes.byref(cfg)) == api.STATUS_OK
    ws_bytes = lib.b200_gemm_workspace_bytes(1, M, N, K, ctypes.byref(cfg))
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device="cuda")
    ref = torch.empty(M, N, dtype=torch.bfloat16, device="cuda")
    assert lib.b200_gemm_bf16(M, N, K, a.data_ptr(), b.data_ptr(), ref.data_ptr(), alpha, beta, ctypes.byref(cfg),
                              ws.data_ptr(), ws_bytes, None) == api.STATUS_OK
    torch.cuda.synchronize()
    _status_ok(lib, api)
    return ref


def test_fixed_scratch_matches_the_oracle_and_the_workspace_entry_point_twice_in_a_row():
    import torch
    from h100_gemm_b200 import api
    lib = api.library()
    # Different shapes back to back: each call finds the previous call's partial tiles and flag
    # words in the shared array. Integer-valued operands must match the CPU oracle bit for bit
    # (alpha and beta included), normal ones within the tolerance of the other GPU tests.
    for (M, N, K, seed, alpha, beta, integer) in ((48, 4096, 2048, 1, 1.0, 0.0, True),
                                                  (128, 3008, 4096, 7, 0.5, 0.25, True),
                                                  (100, 5000, 1024, 9, 1.0, 0.0, False),
                                                  (16, 28672, 8192, 3, 1.0, 0.0, False)):
        a_bits, b_bits, a, b = _operands(M, N, K, seed, integer)
        want = oracle.cpu_gemm(a_bits, b_bits, alpha, beta)
        other = util.to_bits(_workspace_entry_point(lib, api, torch, a, b, M, N, K, alpha, beta))
        for _ in range(2):  # and the same shape twice
            got = util.to_bits(_fixed_scratch(lib, api, torch, a, b, M, N, K, alpha, beta))
            if integer:
                assert np.array_equal(got, want)
            else:
                assert oracle.norm_relative_error(got, want, a_bits, b_bits) <= TOL
            assert np.array_equal(got, other)  # same kernel, same schedule: the two agree exactly


def test_fixed_scratch_allocates_no_device_memory():
    """What the entry point is for: after its first call on the device, free device memory (as
    cudaMemGetInfo reports it) is the same before and after any number of calls."""
    import torch
    from h100_gemm_b200 import api
    lib = api.library()
    M, N, K = 64, 8192, 4096
    a_bits, b_bits, a, b = _operands(M, N, K, 11, True)
    out = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    _fixed_scratch(lib, api, torch, a, b, M, N, K, 1.0, 0.0, out)  # first call: one-time set-up
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(5):
        assert lib.b200_gemm_bf16_fixed_scratch(M, N, K, a.data_ptr(), b.data_ptr(), out.data_ptr(), 1.0, 0.0,
                                                None) == api.STATUS_OK
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    _status_ok(lib, api)
    assert np.array_equal(util.to_bits(out), oracle.cpu_gemm(a_bits, b_bits))


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
