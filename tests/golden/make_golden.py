"""Generates tests/golden/*.npz from the REAL reference oracle.

Run in a container that has a checkout of the reference (its location is the REFERENCE variable of oracle/Makefile):

    make -C oracle ref            # builds oracle/_ref/libref_gemm.so from reference.h, in place
    python tests/golden/make_golden.py

Every fixture stores the inputs (bf16 bit patterns) and the output of the reference's own
reference_cpu_gemm<bf16,bf16,bf16,float> (reference.h:5-46), so the fixtures pin parity on
machines where the reference is not present. The 1024^3 configuration stores a SHA-256 of C and
64 sampled rows instead of the full 2 MB matrix; its inputs are regenerated from the seed and
guarded by their own SHA-256.
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))
sys.path.insert(0, str(HERE.parent))

from oracle import oracle  # noqa: E402
import util  # noqa: E402

SMALL_CASES = [
    # name, M, N, K, generator, alpha, beta
    ("uniform_100x70x45", 100, 70, 45, "uniform", 1.0, 0.0),
    ("uniform_64x64x64", 64, 64, 64, "uniform", 1.0, 0.0),
    ("uniform_130x257x333", 130, 257, 333, "uniform", 1.0, 0.0),
    ("integer_96x160x200", 96, 160, 200, "integer", 1.0, 0.0),
    ("normal_17x129x1000", 17, 129, 1000, "normal", 1.0, 0.0),
    ("alphabeta_65x63x77", 65, 63, 77, "uniform", 0.5, 0.25),
    ("k1_33x31x1", 33, 31, 1, "uniform", 1.0, 0.0),
    ("row_1x300x257", 1, 300, 257, "uniform", 1.0, 0.0),
]


def gen(kind, shape, seed):
    if kind == "uniform":
        return util.uniform_bits(shape, seed)
    if kind == "integer":
        return util.integer_bits(shape, seed)
    return util.normal_bits(shape, seed)


F16_CASES = [
    # fp16 fixtures: the data type of the reference's template path (reference_cpu_gemm<half_t,...>)
    ("f16_uniform_70x90x300", 70, 90, 300, "uniform", 1.0, 0.0),
    ("f16_integer_64x96x256", 64, 96, 256, "integer", 1.0, 0.0),
    ("f16_alphabeta_33x47x129", 33, 47, 129, "uniform", 0.5, 0.25),
]


def gen_f16(kind, shape, seed):
    rng = np.random.Generator(np.random.Philox(seed))
    x = rng.integers(-5, 5, size=shape) if kind == "integer" else rng.uniform(-1.0, 1.0, size=shape)
    return oracle.f32_to_f16_bits(x.astype(np.float32))


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def main():
    assert oracle.have_reference(), "build oracle/_ref first (make -C oracle ref)"
    for i, (name, M, N, K, kind, alpha, beta) in enumerate(SMALL_CASES):
        a = gen(kind, (M, K), 100 + 2 * i)
        b = gen(kind, (N, K), 101 + 2 * i)
        c = oracle.reference_cpu_gemm(a, b, alpha, beta)
        np.savez_compressed(HERE / f"{name}.npz", a=a, b=b, c=c, alpha=np.float32(alpha), beta=np.float32(beta))
        print(name, c.shape)
    for i, (name, M, N, K, kind, alpha, beta) in enumerate(F16_CASES):
        a = gen_f16(kind, (M, K), 300 + 2 * i)
        b = gen_f16(kind, (N, K), 301 + 2 * i)
        c = oracle.reference_cpu_gemm_f16(a, b, alpha, beta)
        np.savez_compressed(HERE / f"{name}.npz", a=a, b=b, c=c, alpha=np.float32(alpha), beta=np.float32(beta))
        print(name, c.shape)
    # Configuration 1: M=N=K=1024, uniform[-1,1], seed 0 (A) and 1 (B).
    a = util.uniform_bits((1024, 1024), 0)
    b = util.uniform_bits((1024, 1024), 1)
    c = oracle.reference_cpu_gemm(a, b)
    rows = np.arange(0, 1024, 16, dtype=np.int32)
    np.savez_compressed(HERE / "config1_1024.npz", rows=rows, c_rows=c[rows], sha_a=sha(a), sha_b=sha(b), sha_c=sha(c))
    print("config1_1024", sha(c))


if __name__ == "__main__":
    main()
