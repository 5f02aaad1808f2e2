"""The CPU oracle (oracle/cpu_gemm.c) against the reference's own oracle.

The reference holds no golden vectors or unit tests (its checks are self-checks inside benchmark
mains, matmul_h100.cu.jinja:1043-1058), so parity is pinned two ways:
  * tests/golden/*.npz — outputs of the real reference_cpu_gemm (reference.h:5-46), produced by
    tests/golden/make_golden.py;
  * a bit-for-bit diff against oracle/_ref (reference.h compiled in place) when it is present.
"""
import hashlib
from pathlib import Path

import numpy as np
import pytest

import util
from oracle import oracle

GOLDEN = Path(__file__).resolve().parent / "golden"
SMALL = sorted(p for p in GOLDEN.glob("*.npz") if p.name != "config1_1024.npz" and not p.name.startswith("f16_"))
F16 = sorted(GOLDEN.glob("f16_*.npz"))


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


@pytest.mark.parametrize("path", SMALL, ids=lambda p: p.stem)
def test_oracle_matches_golden(path):
    g = np.load(path)
    c = oracle.cpu_gemm(g["a"], g["b"], float(g["alpha"]), float(g["beta"]))
    assert np.array_equal(c, g["c"])


@pytest.mark.parametrize("path", F16, ids=lambda p: p.stem)
def test_fp16_oracle_matches_golden(path):
    """reference_cpu_gemm<half_t,half_t,half_t,float>, the reference template's instantiation."""
    g = np.load(path)
    assert np.array_equal(oracle.cpu_gemm_f16(g["a"], g["b"], float(g["alpha"]), float(g["beta"])), g["c"])


@pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref not built (needs the reference checkout)")
def test_fp16_oracle_matches_reference_build():
    rng = np.random.Generator(np.random.Philox(5))
    for (M, N, K) in ((1, 1, 1), (65, 33, 129), (128, 200, 555)):
        a = oracle.f32_to_f16_bits(rng.standard_normal((M, K)).astype(np.float32))
        b = oracle.f32_to_f16_bits((rng.standard_normal((N, K)) * 0.02).astype(np.float32))  # reaches subnormals
        assert np.array_equal(oracle.cpu_gemm_f16(a, b), oracle.reference_cpu_gemm_f16(a, b))
        assert np.array_equal(oracle.cpu_gemm_f16(a, b, 300.0, -2.0), oracle.reference_cpu_gemm_f16(a, b, 300.0, -2.0))


def test_fp16_conversions_match_numpy():
    lib = oracle._load_oracle()
    import ctypes
    lib.oracle_f32_to_f16.argtypes = [ctypes.c_float]
    lib.oracle_f32_to_f16.restype = ctypes.c_uint16
    lib.oracle_f16_to_f32.argtypes = [ctypes.c_uint16]
    lib.oracle_f16_to_f32.restype = ctypes.c_float
    rng = np.random.Generator(np.random.Philox(6))
    x = np.concatenate([rng.standard_normal(3000).astype(np.float32) * s for s in (1e-8, 1e-5, 1e-3, 1, 100, 30000)]
                       + [np.array([0, -0.0, 65504, 65519.99, 65520, 1e9, np.inf, 5.96e-8, 2.98e-8, 2.9e-8, 3.1e-8],
                                   dtype=np.float32)])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = np.array([lib.oracle_f32_to_f16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(got, want)
    for h in (0x0001, 0x03FF, 0x0400, 0x3C00, 0x7BFF, 0x7C00, 0x8001, 0xFBFF):
        assert lib.oracle_f16_to_f32(h) == float(np.array([h], dtype=np.uint16).view(np.float16)[0])


def test_oracle_matches_golden_config1():
    """BASELINE configuration 1: M=N=K=1024, uniform[-1,1] from seed 0, bit-exact."""
    g = np.load(GOLDEN / "config1_1024.npz")
    a = util.uniform_bits((1024, 1024), 0)
    b = util.uniform_bits((1024, 1024), 1)
    assert sha(a) == str(g["sha_a"]) and sha(b) == str(g["sha_b"]), "input generator drifted"
    c = oracle.cpu_gemm(a, b)
    assert sha(c) == str(g["sha_c"])
    assert np.array_equal(c[g["rows"]], g["c_rows"])
    assert np.array_equal(oracle.cpu_gemm_rows(a, b, g["rows"]), g["c_rows"])


@pytest.mark.skipif(not oracle.have_reference(), reason="oracle/_ref not built (needs the reference checkout)")
@pytest.mark.parametrize("shape", [(1, 1, 1), (3, 5, 7), (64, 64, 32), (65, 129, 33), (200, 100, 555),
                                   (128, 1000, 64), (256, 256, 2048)])
def test_oracle_matches_reference_build(shape):
    M, N, K = shape
    a = util.normal_bits((M, K), 7)
    b = util.normal_bits((N, K), 8, 0.02)
    assert np.array_equal(oracle.cpu_gemm(a, b), oracle.reference_cpu_gemm(a, b))
    assert np.array_equal(oracle.cpu_gemm(a, b, 1.5, -0.75), oracle.reference_cpu_gemm(a, b, 1.5, -0.75))


def test_oracle_close_to_float64():
    """Sanity against exact dot products: error bounded by bf16 output rounding + fp32 sums."""
    M, N, K = 70, 90, 300
    a = util.uniform_bits((M, K), 3)
    b = util.uniform_bits((N, K), 4)
    exact = oracle.bf16_bits_to_f32(a).astype(np.float64) @ oracle.bf16_bits_to_f32(b).astype(np.float64).T
    got = oracle.bf16_bits_to_f32(oracle.cpu_gemm(a, b)).astype(np.float64)
    assert np.abs(got - exact).max() <= np.abs(exact).max() * 2.0 ** -8 + 1e-3


def test_integer_inputs_are_exact():
    """The reference harness's fill (common.h:283-289): sums are integers below 2^24, so any
    summation order gives the same fp32 value and the bf16 result is order-independent."""
    M, N, K = 40, 50, 512
    a = util.integer_bits((M, K), 5)
    b = util.integer_bits((N, K), 6)
    exact = oracle.bf16_bits_to_f32(a).astype(np.int64) @ oracle.bf16_bits_to_f32(b).astype(np.int64).T
    assert np.array_equal(oracle.cpu_gemm(a, b), oracle.f32_to_bf16_bits(exact.astype(np.float32)))


def test_scalar_beta_rule():
    """reference.h:40 adds beta as a scalar (not beta*C): C = (bf16)(acc*alpha + beta)."""
    a = util.uniform_bits((8, 16), 9)
    b = util.uniform_bits((8, 16), 10)
    acc = oracle.bf16_bits_to_f32(a).astype(np.float64) @ oracle.bf16_bits_to_f32(b).astype(np.float64).T
    got = oracle.bf16_bits_to_f32(oracle.cpu_gemm(a, b, 2.0, 3.0))
    assert np.abs(got - (acc * 2.0 + 3.0)).max() < 0.05


def test_bf16_rounding_helpers():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 0.0, np.inf, np.nan, 3.4e38], dtype=np.float32)
    bits = oracle.f32_to_bf16_bits(x)
    lib_bits = np.array([oracle._load_oracle().oracle_f32_to_bf16(float(v)) for v in x], dtype=np.uint16)
    assert np.array_equal(bits, lib_bits)
    assert bits[0] == 0x3F80 and bits[1] == 0x3F80 and bits[2] == 0x3F82  # ties to even, both ways
    assert bits[5] == 0x7F80 and bits[6] == 0x7FFF and bits[7] == 0x7F80   # inf, NaN, overflow to inf


def test_norm_relative_error_metric():
    a = util.uniform_bits((4, 8), 1)
    b = util.uniform_bits((5, 8), 2)
    c = oracle.cpu_gemm(a, b)
    assert oracle.norm_relative_error(c, c, a, b) == 0.0
    d = c.copy()
    d[0, 0] ^= 0x0040
    assert oracle.norm_relative_error(d, c, a, b) > 0.0
