"""GPU parity tests: the CUDA path, called through the C ABI (h100_gemm_b200.api -> libb200gemm.so),
against the CPU oracle (oracle/cpu_gemm.c, pinned to reference.h:5-46) on the same seeded inputs.

Tolerances (floating point, accumulation order differs between the tensor cores and the oracle):
  * general inputs:  max_ij |C - C_oracle| / (||A_i||_2 ||B_j||_2) <= 1e-2   (the acceptance bound)
  * integer-valued inputs (the reference harness's own fill, common.h:283-289): every partial sum
    is an integer below 2^24, so results must agree BIT FOR BIT in any summation order.
"""
import numpy as np
import pytest

import util
from oracle import oracle

pytestmark = pytest.mark.gpu

TOL = 1e-2
GOLDEN = __import__("pathlib").Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module")
def g():
    import torch
    assert torch.cuda.is_available()
    import h100_gemm_b200 as lib
    lib.library()  # raises if the CUDA library has not been built: there is no fallback
    return lib


def cfgs():
    from h100_gemm_b200.api import GemmConfig as C
    out = []
    for cm in (1, 2):
        for bn in (64, 128, 192, 256):
            out.append(C(block_n=bn, cluster_m=cm))
    for cm in (1, 2):
        for bn in (128, 256):
            out.append(C(block_m=256, block_n=bn, cluster_m=cm))  # two A sub-tiles per CTA
    out.append(C(block_n=256, cluster_m=2, epilogue=2))                # vector-store epilogue
    out.append(C(block_m=256, block_n=256, cluster_m=2, epilogue=2))
    out.append(C(block_n=64, cluster_m=1, epilogue=2))
    out.append(C(block_n=256, cluster_m=2, epilogue=3))                # staged coalesced stores
    out.append(C(block_m=256, block_n=256, cluster_m=2, epilogue=3))
    out.append(C(block_n=192, cluster_m=1, epilogue=3))
    for bm in (16, 32, 64):                                            # few-rows plan: operands swapped inside
        out.append(C(block_m=bm, block_n=128, cluster_m=1))
    return out


def cfg_id(c):
    return "auto" if c is None else f"bm{c.block_m}-bn{c.block_n}-cm{c.cluster_m}-e{c.epilogue}-st{c.stages}-s{c.sched}k{c.split_k}-r{c.raster}g{c.group}"


def run(g, a_bits, b_bits, cfg=None, alpha=1.0, beta=0.0):
    out = g.gemm(util.to_device(a_bits), util.to_device(b_bits), cfg=cfg, alpha=alpha, beta=beta)
    rc, words = g.device_status()
    assert rc == 0, f"device status {words}"
    return util.to_bits(out)


def assert_close(c, ref, a, b, rows=None):
    a_used = a if rows is None else a[rows]
    err = oracle.norm_relative_error(c, ref, a_used, b)
    assert err <= TOL, f"norm-relative error {err:.3e} > {TOL}"


# ------------------------------------------------------------------------------------------------
# Configuration 1: M=N=K=1024, uniform[-1,1] seed 0 — full matrix against the oracle and the
# golden rows produced by the reference's own reference_cpu_gemm.
# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def config1():
    a = util.uniform_bits((1024, 1024), 0)
    b = util.uniform_bits((1024, 1024), 1)
    return a, b, oracle.cpu_gemm(a, b)


@pytest.mark.parametrize("cfg", [None] + cfgs(), ids=cfg_id)
def test_config1_full_matrix(g, config1, cfg):
    a, b, ref = config1
    c = run(g, a, b, cfg)
    assert_close(c, ref, a, b)
    gold = np.load(GOLDEN / "config1_1024.npz")
    assert_close(c[gold["rows"]], gold["c_rows"], a, b, rows=gold["rows"])
    # bf16 output: at most one unit in the last place away from the oracle almost everywhere
    diff = np.abs(oracle.bf16_bits_to_f32(c) - oracle.bf16_bits_to_f32(ref))
    assert np.mean(diff > 0) < 0.2


@pytest.mark.parametrize("path", sorted(p for p in GOLDEN.glob("*.npz")
                                        if p.name != "config1_1024.npz" and not p.name.startswith("f16_")),
                         ids=lambda p: p.stem)
def test_golden_fixtures(g, path):
    """Small, ragged shapes (K=1, a single row, tails in every dimension, alpha/beta)."""
    gold = np.load(path)
    a, b, ref = gold["a"], gold["b"], gold["c"]
    for cfg in (None, cfgs()[1], cfgs()[7]):
        c = run(g, a, b, cfg, float(gold["alpha"]), float(gold["beta"]))
        if path.stem.startswith("integer"):
            assert np.array_equal(c, ref)
        else:
            assert_close(c, ref, a, b)


@pytest.mark.parametrize("epilogue", [0, 1, 2])
def test_224_column_tiles(g, config1, epilogue):
    """The 128 x 224 tile (three 64-column chunks through the store path in use, the last 32 columns
    from registers): configuration 1, every golden fixture (bf16 and fp16, alpha/beta), tails in M, N
    and K with integer-valued inputs at three ring depths, and a batch."""
    from h100_gemm_b200.api import GemmConfig as C
    cfg = C(block_m=128, block_n=224, cluster_m=1, sched=0, epilogue=epilogue)
    a, b, ref = config1
    assert_close(run(g, a, b, cfg), ref, a, b)
    for path in sorted(GOLDEN.glob("*.npz")):
        if path.name == "config1_1024.npz":
            continue
        gold = np.load(path)
        runner = run_f16 if path.name.startswith("f16_") else run
        c = runner(g, gold["a"], gold["b"], cfg, float(gold["alpha"]), float(gold["beta"]))
        if "integer" in path.stem:
            assert np.array_equal(c, gold["c"]), path.stem
        elif path.name.startswith("f16_"):
            assert oracle.norm_relative_error(c, gold["c"], gold["a"], gold["b"], f16=True) <= TOL, path.stem
        else:
            assert_close(c, gold["c"], gold["a"], gold["b"])
    for stages in (2, 3, 0):
        ai, bi = util.integer_bits((300, 1544), 7), util.integer_bits((1352, 1544), 8)
        cs = C(block_m=128, block_n=224, cluster_m=1, sched=0, epilogue=epilogue, stages=stages)
        assert np.array_equal(run(g, ai, bi, cs), oracle.cpu_gemm(ai, bi))
    ab, bb = util.integer_bits((3 * 200, 264), 9), util.integer_bits((3 * 456, 264), 10)
    out = g.gemm_batched(util.to_device(ab).view(3, 200, 264), util.to_device(bb).view(3, 456, 264), cfg=cfg)
    assert g.device_status()[0] == 0
    for i in range(3):
        assert np.array_equal(util.to_bits(out[i]), oracle.cpu_gemm(ab[i * 200:(i + 1) * 200], bb[i * 456:(i + 1) * 456]))


@pytest.mark.parametrize("cfg", cfgs(), ids=cfg_id)
@pytest.mark.parametrize("stages", [2, 3, 0])
def test_integer_inputs_bit_exact(g, cfg, stages):
    """Every kernel instantiation and ring depth, tails in M, N and K, bit for bit."""
    from dataclasses import replace
    M, N, K = 777, 1000, 1544
    a = util.integer_bits((M, K), 11)
    b = util.integer_bits((N, K), 12)
    ref = oracle.cpu_gemm(a, b)
    assert np.array_equal(run(g, a, b, replace(cfg, stages=stages)), ref)


# ------------------------------------------------------------------------------------------------
# Configuration 2: square sweep. Oracle on sampled rows; whole-matrix bit-exactness against the
# on-device SIMT GEMM on integer inputs; size-independent properties at full size.
# ------------------------------------------------------------------------------------------------
def device_inputs(M, N, K, seed, kind="uniform", sigma_b=1.0):
    import torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    if kind == "uniform":
        a = (torch.rand(M, K, device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
        b = (torch.rand(N, K, device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
    elif kind == "integer":
        a = torch.randint(-5, 5, (M, K), device="cuda", generator=gen).to(torch.bfloat16)
        b = torch.randint(-5, 5, (N, K), device="cuda", generator=gen).to(torch.bfloat16)
    else:
        a = torch.randn(M, K, device="cuda", generator=gen).to(torch.bfloat16)
        b = (torch.randn(N, K, device="cuda", generator=gen) * sigma_b).to(torch.bfloat16)
    return a, b


@pytest.mark.parametrize("n", [4096, 8192, 16384])
def test_square_sampled_rows(g, n):
    a, b = device_inputs(n, n, n, seed=n)
    c = g.gemm(a, b)
    assert g.device_status()[0] == 0
    rows = np.unique(np.concatenate([np.arange(0, n, n // 16), [n - 1, 127, 128, 255, 256]])).astype(np.int32)
    a_rows = util.to_bits(a[rows.tolist()])
    ref = oracle.cpu_gemm(a_rows, util.to_bits(b))
    assert_close(util.to_bits(c[rows.tolist()]), ref, a_rows, util.to_bits(b))


@pytest.mark.parametrize("n", [4096, 8192])
def test_square_integer_whole_matrix_vs_simt(g, n):
    import torch
    a, b = device_inputs(n, n, n, seed=5, kind="integer")
    c = g.gemm(a, b)
    ref = g.reference_gpu_gemm(a, b)
    assert g.device_status()[0] == 0
    assert torch.equal(c.view(torch.int16), ref.view(torch.int16))
    # and the SIMT cross-check itself against the oracle on a few rows
    rows = [0, 1000, n - 1]
    want = oracle.cpu_gemm(util.to_bits(a[rows]), util.to_bits(b))
    assert np.array_equal(util.to_bits(ref[rows]), want)


def test_properties_at_full_size(g):
    """8192^3: exact power-of-two scaling, row permutation, run-to-run determinism."""
    import torch
    n = 8192
    a, b = device_inputs(n, n, n, seed=9)
    c = g.gemm(a, b)
    c2 = g.gemm(a, b)
    assert torch.equal(c.view(torch.int16), c2.view(torch.int16))
    c_scaled = g.gemm(a * 2, b * 0.5)
    assert torch.equal(c.view(torch.int16), c_scaled.view(torch.int16))
    perm = torch.randperm(n, device="cuda", generator=torch.Generator(device="cuda").manual_seed(1))
    c_perm = g.gemm(a[perm].contiguous(), b)
    assert torch.equal(c[perm].view(torch.int16), c_perm.view(torch.int16))
    assert g.device_status()[0] == 0


# ------------------------------------------------------------------------------------------------
# Configuration 3: skinny decode shapes, A ~ N(0,1), B ~ N(0,0.02); stream-K (default) and split-K.
# ------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def skinny_b():
    import torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(33)
    b = (torch.randn(28672, 8192, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    return b, util.to_bits(b)


@pytest.mark.parametrize("m", [16, 32, 64, 128])
def test_skinny_decode(g, skinny_b, m):
    from h100_gemm_b200.api import GemmConfig as C
    b, b_bits = skinny_b
    a_bits = util.normal_bits((m, 8192), 40 + m)
    a = util.to_device(a_bits)
    ref = oracle.cpu_gemm(a_bits, b_bits)
    for cfg in (None, C(block_n=128, cluster_m=1, sched=1, split_k=4), C(block_n=64, cluster_m=1, sched=2),
                C(block_n=256, cluster_m=1, sched=0), C(block_n=224, cluster_m=1, sched=0, epilogue=1)):
        c = util.to_bits(g.gemm(a, b, cfg=cfg))
        assert g.device_status()[0] == 0
        assert_close(c, ref, a_bits, b_bits)


@pytest.mark.parametrize("cfg_kw", [dict(block_n=128, cluster_m=1, sched=1, split_k=3),
                                    dict(block_n=256, cluster_m=2, sched=1, split_k=5),
                                    dict(block_n=128, cluster_m=1, sched=2),
                                    dict(block_n=256, cluster_m=2, sched=2),
                                    dict(block_n=192, cluster_m=2, sched=2, max_ctas=20),
                                    dict(block_m=256, block_n=256, cluster_m=2, sched=2),
                                    dict(block_m=256, block_n=128, cluster_m=1, sched=1, split_k=2),
                                    dict(block_n=64, cluster_m=1, sched=3),
                                    dict(block_n=128, cluster_m=2, sched=3, max_ctas=16),
                                    dict(block_m=256, block_n=128, cluster_m=1, sched=3, max_ctas=5),
                                    dict(block_n=128, cluster_m=1, sched=4, max_ctas=20),
                                    dict(block_n=256, cluster_m=2, sched=4, max_ctas=10),
                                    dict(block_m=256, block_n=256, cluster_m=2, sched=4, max_ctas=6)])
def test_split_and_stream_k_integer_exact(g, cfg_kw):
    from h100_gemm_b200.api import GemmConfig as C
    M, N, K = 700, 900, 3000
    a = util.integer_bits((M, K), 21)
    b = util.integer_bits((N, K), 22)
    ref = oracle.cpu_gemm(a, b)
    c1 = run(g, a, b, C(**cfg_kw))
    assert np.array_equal(c1, ref)
    assert np.array_equal(run(g, a, b, C(**cfg_kw), alpha=0.5, beta=1.0), oracle.cpu_gemm(a, b, 0.5, 1.0))


# ------------------------------------------------------------------------------------------------
# Configuration 4: prefill shape, row-sharded. One GPU computes every shard; the concatenation
# must equal the unsharded product bit for bit (what the multi-GPU run relies on).
# ------------------------------------------------------------------------------------------------
def test_row_shards_concatenate_bit_exact(g):
    import torch
    M, N, K = 65536, 8192, 8192
    a, b = device_inputs(M, N, K, seed=4, kind="normal", sigma_b=0.02)
    full = g.gemm(a, b)
    rows = np.array([0, 8191, 8192, 30000, 65535], dtype=np.int32)
    a_rows = util.to_bits(a[rows.tolist()])
    b_bits = util.to_bits(b)
    assert_close(util.to_bits(full[rows.tolist()]), oracle.cpu_gemm(a_rows, b_bits), a_rows, b_bits)
    for world in (2, 8):
        shard = M // world
        parts = [g.gemm(a[r * shard:(r + 1) * shard], b) for r in range(world)]
        assert torch.equal(torch.cat(parts).view(torch.int16), full.view(torch.int16))
    assert g.device_status()[0] == 0


def test_fused_gather_epilogue_on_one_device(g):
    """b200_gemm_bf16_gather with every "rank's" copy of C on this device: each call must fill
    exactly its own row range in ALL copies — equal to the CPU oracle's rows within the tolerance
    (bit for bit with integer-valued operands), and the same bits as the plain GEMM — and leave
    the rest."""
    import torch
    from h100_gemm_b200 import api
    world, M, N, K = 3, 1024, 768, 512
    b_bits = util.normal_bits((N, K), 12, 0.05)
    shard_bits = [util.normal_bits((M, K), 13 + r) for r in range(world - 1)] + [util.integer_bits((M, K), 19)]
    b = util.to_device(b_bits)
    shards = [util.to_device(x) for x in shard_bits]
    refs = [oracle.cpu_gemm(x, b_bits) for x in shard_bits]
    int_b_bits = util.integer_bits((N, K), 20)
    int_ref = oracle.cpu_gemm(shard_bits[-1], int_b_bits)
    bufs = [api.DeviceBuffer(world * M * N * 2) for _ in range(world)]
    try:
        views = [buf.tensor((world * M, N)) for buf in bufs]
        for v in views:
            v.fill_(-7.0)
        for cfg in (None, api.GemmConfig(block_m=128, block_n=256, cluster_m=2, epilogue=1),
                    api.GemmConfig(block_m=256, block_n=256, cluster_m=2, epilogue=1)):
            for rank in range(world):
                api.gemm_gather(shards[rank], b, [buf.ptr for buf in bufs], rank, cfg=cfg)
                assert g.device_status()[0] == 0
                want = g.gemm(shards[rank], b)
                for v in views:
                    got = v[rank * M:(rank + 1) * M]
                    assert_close(util.to_bits(got), refs[rank], shard_bits[rank], b_bits)
                    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
                    later = v[(rank + 1) * M:]
                    if cfg is None and later.numel():
                        assert bool((later == -7.0).all())  # rows of ranks that have not run yet
        # integer-valued operands: every copy holds the oracle's bits
        api.gemm_gather(shards[-1], util.to_device(int_b_bits), [buf.ptr for buf in bufs], world - 1)
        assert g.device_status()[0] == 0
        for v in views:
            assert np.array_equal(util.to_bits(v[(world - 1) * M:]), int_ref)
        # the tracing build of the fused kernel: same bits, counters filled
        prof = torch.zeros(148 * 8, dtype=torch.int64, device="cuda")
        api.set_profile_buffer(prof)
        try:
            api.gemm_gather(shards[-1], util.to_device(int_b_bits), [buf.ptr for buf in bufs], world - 1)
        finally:
            api.set_profile_buffer(None)
        assert g.device_status()[0] == 0
        for v in views:
            assert np.array_equal(util.to_bits(v[(world - 1) * M:]), int_ref)
        counters = prof.view(148, 8).cpu().numpy()
        assert counters[:, api.PROFILE_SLOTS.index("tiles")].sum() > 0 and (counters[:, 0] >= 0).all()
        # a tile shape the fused epilogue is not built for is refused, not mis-executed
        with pytest.raises(api.GemmError) as e:
            api.gemm_gather(shards[0], b, [buf.ptr for buf in bufs], 0, cfg=api.GemmConfig(block_n=128, cluster_m=1))
        assert e.value.status == api.STATUS_UNSUPPORTED_CFG
    finally:
        for buf in bufs:
            buf.close()


@pytest.mark.parametrize("gather", [False, True])
def test_single_process_multi_gpu_handle(g, gather):
    """b200_mgemm_*: the row-sharded GEMM from one process. With one device visible the ranks share
    it (their kernels do not wait on one another); with more, rank p runs on device p. Every rank's
    rows — and, with the fused gather, every rank's full copy — must equal the CPU oracle bit for
    bit on integer-valued operands."""
    import torch
    from h100_gemm_b200 import api
    world, M, N, K = 2, 512, 768, 328
    ndev = torch.cuda.device_count()
    devices = [p % ndev for p in range(world)]
    b_bits = util.integer_bits((N, K), 31)
    a_bits = [util.integer_bits((M, K), 32 + p) for p in range(world)]
    want = np.concatenate([oracle.cpu_gemm(a, b_bits) for a in a_bits])
    mg = api.MultiGemm(world, M, N, K, gather=gather, devices=devices)
    try:
        for p in range(world):
            mg.a(p).copy_(util.to_device(a_bits[p]).to(f"cuda:{devices[p]}"))
            mg.b(p).copy_(util.to_device(b_bits).to(f"cuda:{devices[p]}"))
            mg.c(p).fill_(-3.0)
        torch.cuda.synchronize()
        for _ in range(2):
            mg.run()
            assert mg.sync() > 0.0
        for p in range(world):
            got = util.to_bits(mg.c(p))
            assert np.array_equal(got, want if gather else want[p * M:(p + 1) * M]), f"rank {p}"
    finally:
        mg.close()
    assert g.device_status()[0] == 0
    with pytest.raises(api.GemmError):
        api.MultiGemm(9, M, N, K)


# ------------------------------------------------------------------------------------------------
# Configuration 5: irregular shapes and the batched problem.
# ------------------------------------------------------------------------------------------------
DIMS = (1000, 3000, 5555)


@pytest.mark.parametrize("m", DIMS)
@pytest.mark.parametrize("n", DIMS)
@pytest.mark.parametrize("k", DIMS)
def test_irregular_shapes(g, m, n, k):
    a_bits = util.uniform_bits((m, k), m + k)
    b_bits = util.uniform_bits((n, k), n + k + 1)
    c = run(g, a_bits, b_bits)
    rows = np.array(sorted({0, 1, 127, 128, 255, 256, m // 2, m - 2, m - 1}), dtype=np.int32)
    assert_close(c[rows], oracle.cpu_gemm_rows(a_bits, b_bits, rows), a_bits, b_bits, rows=rows)


def test_irregular_integer_bit_exact(g):
    a = util.integer_bits((1000, 5555), 1)
    b = util.integer_bits((3000, 5555), 2)
    assert np.array_equal(run(g, a, b), oracle.cpu_gemm(a, b))
    a = util.integer_bits((5555, 1000), 3)
    b = util.integer_bits((5555, 1000), 4)
    assert np.array_equal(run(g, a, b), oracle.cpu_gemm(a, b))


def test_batched_32x2048x2048x512(g):
    import torch
    gen = torch.Generator(device="cuda")
    gen.manual_seed(77)
    a = (torch.rand(32, 2048, 512, device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
    b = (torch.rand(32, 2048, 512, device="cuda", generator=gen) * 2 - 1).to(torch.bfloat16)
    c = g.gemm_batched(a, b)
    assert g.device_status()[0] == 0
    for i in (0, 13, 31):
        ai, bi = util.to_bits(a[i]), util.to_bits(b[i])
        assert_close(util.to_bits(c[i]), oracle.cpu_gemm(ai, bi), ai, bi)
    # batches must not bleed into each other: integer inputs, ragged shape, bit-exact
    a = torch.randint(-5, 5, (5, 300, 520), device="cuda", generator=gen).to(torch.bfloat16)
    b = torch.randint(-5, 5, (5, 200, 520), device="cuda", generator=gen).to(torch.bfloat16)
    c = g.gemm_batched(a, b)
    for i in range(5):
        assert np.array_equal(util.to_bits(c[i]), oracle.cpu_gemm(util.to_bits(a[i]), util.to_bits(b[i])))


# ------------------------------------------------------------------------------------------------
# fp16: the data type of the reference's template path (b200_gemm_f16)
# ------------------------------------------------------------------------------------------------
def run_f16(g, a_bits, b_bits, cfg=None, alpha=1.0, beta=0.0):
    out = g.gemm(util.to_device_f16(a_bits), util.to_device_f16(b_bits), cfg=cfg, alpha=alpha, beta=beta)
    rc, words = g.device_status()
    assert rc == 0, f"device status {words}"
    return util.to_bits(out.view(__import__("torch").bfloat16))


@pytest.mark.parametrize("path", sorted(GOLDEN.glob("f16_*.npz")), ids=lambda p: p.stem)
def test_fp16_golden_fixtures(g, path):
    gold = np.load(path)
    a, b, ref = gold["a"], gold["b"], gold["c"]
    for cfg in (None, cfgs()[1], cfgs()[7], cfgs()[11]):
        c = run_f16(g, a, b, cfg, float(gold["alpha"]), float(gold["beta"]))
        if "integer" in path.stem:
            assert np.array_equal(c, ref)
        else:
            assert oracle.norm_relative_error(c, ref, a, b, f16=True) <= TOL


@pytest.mark.parametrize("cfg", [None] + cfgs()[:12:3] + cfgs()[-3:], ids=cfg_id)
def test_fp16_parity(g, cfg):
    from h100_gemm_b200.api import GemmConfig as C
    M, N, K = 1000, 776, 1544
    a = util.f16_integer_bits((M, K), 31)
    b = util.f16_integer_bits((N, K), 32)
    assert np.array_equal(run_f16(g, a, b, cfg), oracle.cpu_gemm_f16(a, b))
    a = util.f16_uniform_bits((M, K), 33)
    b = util.f16_uniform_bits((N, K), 34)
    ref = oracle.cpu_gemm_f16(a, b)
    c = run_f16(g, a, b, cfg)
    # fp16 keeps 11 significant bits: the bound is the acceptance one, the typical error far lower
    assert oracle.norm_relative_error(c, ref, a, b, f16=True) <= TOL
    assert np.mean(c != ref) < 0.2
    # stream-K and split-K finish fp16 tiles too
    for extra in (C(block_n=128, cluster_m=1, sched=2), C(block_n=128, cluster_m=1, sched=1, split_k=3)):
        assert oracle.norm_relative_error(run_f16(g, a, b, extra), ref, a, b, f16=True) <= TOL


def test_fp16_simt_cross_check(g):
    import torch
    gen = torch.Generator(device="cuda").manual_seed(8)
    a = torch.randint(-5, 5, (2048, 1024), device="cuda", generator=gen).to(torch.float16)
    b = torch.randint(-5, 5, (1536, 1024), device="cuda", generator=gen).to(torch.float16)
    assert torch.equal(g.gemm(a, b).view(torch.int16), g.reference_gpu_gemm(a, b).view(torch.int16))
    assert g.device_status()[0] == 0


# ------------------------------------------------------------------------------------------------
# Boundary behaviour
# ------------------------------------------------------------------------------------------------
def test_run_kernel_column_major(g):
    """runKernel (matmul_h100_optimal.cu:32-59) writes C column-major with leading dimension M."""
    a_bits = util.normal_bits((1024, 2048), 1)
    b_bits = util.normal_bits((1536, 2048), 2, 0.02)
    out = g.run_kernel(util.to_device(a_bits), util.to_device(b_bits))  # [N, M] == C^T
    assert g.device_status()[0] == 0
    ref = oracle.cpu_gemm(a_bits, b_bits)
    assert_close(np.ascontiguousarray(util.to_bits(out).T), ref, a_bits, b_bits)


def test_alpha_beta_scalar_rule(g):
    a = util.uniform_bits((384, 520), 1)
    b = util.uniform_bits((272, 520), 2)
    for alpha, beta in ((2.0, 0.0), (1.0, 3.0), (-0.5, 0.125)):
        assert_close(run(g, a, b, None, alpha, beta), oracle.cpu_gemm(a, b, alpha, beta), a, b)


def test_host_buffer_entry_point(g):
    for (m, n, k) in ((4096, 1024, 512), (300, 200, 77)):
        a = util.uniform_bits((m, k), 5)
        b = util.uniform_bits((n, k), 6)
        c = g.gemm_host(a, b)
        assert g.device_status()[0] == 0
        rows = np.arange(0, m, max(1, m // 32), dtype=np.int32)
        assert_close(c[rows], oracle.cpu_gemm_rows(a, b, rows), a, b, rows=rows)


def test_error_codes(g):
    import torch
    from h100_gemm_b200 import api
    C = api.GemmConfig
    a = torch.zeros(256, 512, dtype=torch.bfloat16, device="cuda")
    b = torch.zeros(256, 512, dtype=torch.bfloat16, device="cuda")
    for bad, status in ((C(block_n=100), api.STATUS_UNSUPPORTED_CFG), (C(block_m=48), api.STATUS_UNSUPPORTED_CFG),
                        (C(block_m=64, block_n=192), api.STATUS_UNSUPPORTED_CFG),
                        # 224 columns: whole tiles of one CTA only
                        (C(block_n=224, cluster_m=1, sched=2), api.STATUS_UNSUPPORTED_CFG),
                        (C(block_n=224, cluster_m=2), api.STATUS_UNSUPPORTED_CFG),
                        (C(block_m=256, block_n=224, cluster_m=1), api.STATUS_UNSUPPORTED_CFG),
                        (C(block_n=224, cluster_m=1, epilogue=3), api.STATUS_UNSUPPORTED_CFG),
                        (C(block_m=128, block_n=512, swap_ab=1), api.STATUS_UNSUPPORTED_CFG),
                        (C(cluster_n=2), api.STATUS_UNSUPPORTED_CFG), (C(block_k=128), api.STATUS_UNSUPPORTED_CFG),
                        (C(block_n=256, cluster_m=1, stages=7), api.STATUS_SMEM), (C(sched=5), api.STATUS_INVALID_ARG)):
        with pytest.raises(api.GemmError) as e:
            g.gemm(a, b, cfg=bad)
        assert e.value.status == status
    lib = api.library()
    out = torch.empty(256, 256, dtype=torch.bfloat16, device="cuda")
    assert lib.b200_gemm_bf16(256, 256, 512, None, b.data_ptr(), out.data_ptr(), 1.0, 0.0, None, None, 0, None) == api.STATUS_INVALID_ARG
    assert lib.b200_gemm_bf16(0, 256, 512, a.data_ptr(), b.data_ptr(), out.data_ptr(), 1.0, 0.0, None, None, 0, None) == api.STATUS_INVALID_ARG
    cfg = C(block_n=128, cluster_m=1, sched=2)._c()
    import ctypes
    assert lib.b200_gemm_bf16(256, 256, 512, a.data_ptr(), b.data_ptr(), out.data_ptr(), 1.0, 0.0,
                              ctypes.byref(cfg), None, 0, None) == api.STATUS_WORKSPACE
    # the context is still healthy
    assert g.device_status()[0] == 0


def test_cycle_counters(g):
    """The tracing variant of the kernel fills eight counters per CTA and leaves results unchanged."""
    import torch
    from h100_gemm_b200 import api
    a = util.integer_bits((2048, 1024), 1)
    b = util.integer_bits((2048, 1024), 2)
    ref = oracle.cpu_gemm(a, b)
    prof = torch.zeros(148 * 8, dtype=torch.int64, device="cuda")
    api.set_profile_buffer(prof)
    try:
        traced = run(g, a, b, api.GemmConfig(block_n=256, cluster_m=2))
    finally:
        api.set_profile_buffer(None)
    assert np.array_equal(traced, ref)
    p = prof.view(148, 8).cpu().numpy()
    tiles = p[:, api.PROFILE_SLOTS.index("tiles")]
    assert tiles.sum() == 2 * (2048 // 256) * (2048 // 256)  # both CTAs of a pair count each tile
    busy = p[tiles > 0]
    assert (busy[:, 0] > 0).all() and (busy[:, 0] >= busy[:, api.PROFILE_SLOTS.index("epi_busy")]).all()
    assert np.array_equal(run(g, a, b, api.GemmConfig(block_n=256, cluster_m=2)), ref)


def test_bounded_wait_gives_up_and_context_survives(g):
    """Failure detection without a fault: a wait nothing satisfies runs out, the kernel returns,
    the status word names it, and the next GEMM on the same context is correct."""
    from h100_gemm_b200 import api
    assert g.device_status()[0] == 0
    api.selftest_bounded_wait(1 << 20)
    rc, words = g.device_status()
    assert rc == api.STATUS_DEVICE_TIMEOUT and words[0] == 9
    assert g.device_status()[0] == 0  # reading clears it
    a = util.integer_bits((256, 256), 1)
    b = util.integer_bits((256, 256), 2)
    assert np.array_equal(run(g, a, b), oracle.cpu_gemm(a, b))


# ------------------------------------------------------------------------------------------------
# Few-rows plan (block_m = 16 / 32 / 64): the caller's rows ride the MMA's N dimension, 128 rows
# of B its M dimension, and the result is stored transposed. Default for M <= 64.
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("M", [1, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("N,K", [(1024, 520), (1000, 77), (136, 8192), (4100, 1024), (19500, 264)])
def test_few_rows_default_integer_exact(g, M, N, K):
    """cfg = NULL on decode-like shapes, tails in every dimension (N % 8 != 0, K % 8 != 0)."""
    cfg = g.default_config(1, M, N, K)
    assert cfg.block_m == (16 if M <= 16 else 32 if M <= 32 else 64)
    assert cfg.sched == (2 if -(-N // 128) > 148 else 0)       # whole tiles up to one wave, stream-K beyond
    a = util.integer_bits((M, K), 31 + M)
    b = util.integer_bits((N, K), 32 + N)
    ref = oracle.cpu_gemm(a, b)
    assert np.array_equal(run(g, a, b), ref)
    assert np.array_equal(run(g, a, b, alpha=0.5, beta=-2.0), oracle.cpu_gemm(a, b, 0.5, -2.0))


@pytest.mark.parametrize("bm", [16, 32, 64])
@pytest.mark.parametrize("sched,max_ctas", [(0, 0), (2, 0), (2, 7), (3, 5), (4, 5)])
def test_few_rows_tiles_over_many_rows(g, bm, sched, max_ctas):
    """block_m < 128 on a problem with many rows: tiles along both dimensions, every schedule."""
    from h100_gemm_b200.api import GemmConfig as C
    M, N, K = 200, 900, 3000
    a = util.integer_bits((M, K), 41)
    b = util.integer_bits((N, K), 42)
    cfg = C(block_m=bm, block_n=128, cluster_m=1, sched=sched, max_ctas=max_ctas)
    assert np.array_equal(run(g, a, b, cfg), oracle.cpu_gemm(a, b))


def test_few_rows_general_inputs_and_column_major(g):
    import torch
    from h100_gemm_b200.api import GemmConfig as C
    M, N, K = 48, 2048, 4096
    a = util.normal_bits((M, K), 51)
    b = util.normal_bits((N, K), 52, sigma=0.02)
    ref = oracle.cpu_gemm(a, b)
    assert_close(run(g, a, b), ref, a, b)
    # column-major C together with the few-rows plan: the kernel's own orientation, stored as it is
    out = g.gemm(util.to_device(a), util.to_device(b), out=torch.empty(N, M, dtype=torch.bfloat16, device="cuda"),
                 cfg=C(block_m=64, block_n=128, cluster_m=1, c_col_major=1))
    assert g.device_status()[0] == 0
    assert_close(np.ascontiguousarray(util.to_bits(out).T), ref, a, b)
    # split-K has no few-rows form
    with pytest.raises(g.GemmError):
        g.gemm(util.to_device(a), util.to_device(b), cfg=C(block_m=16, block_n=128, cluster_m=1, sched=1, split_k=2))


def test_few_rows_fp16_and_batched(g):
    import torch
    from h100_gemm_b200.api import GemmConfig as C
    gen = torch.Generator(device="cuda").manual_seed(61)
    a = torch.randint(-4, 5, (24, 1032), device="cuda", generator=gen).to(torch.float16)
    b = torch.randint(-4, 5, (776, 1032), device="cuda", generator=gen).to(torch.float16)
    out = g.gemm(a, b)
    assert g.default_config(1, 24, 776, 1032).block_m == 32
    assert torch.equal(out, (a.float() @ b.float().t()).to(torch.float16))
    # batched: three problems, bf16
    ab = torch.randint(-4, 5, (3, 40, 520), device="cuda", generator=gen).to(torch.bfloat16)
    bb = torch.randint(-4, 5, (3, 300, 520), device="cuda", generator=gen).to(torch.bfloat16)
    for cfg in (None, C(block_m=16, block_n=128, cluster_m=1, sched=2)):
        ob = g.gemm_batched(ab, bb, cfg=cfg)
        # integer-valued inputs: the fp32 sums are exact, so only the final rounding to bf16 remains
        assert torch.equal(ob, torch.bmm(ab.float(), bb.float().transpose(1, 2)).to(torch.bfloat16))
    assert g.device_status()[0] == 0


def test_random_shapes_match_the_simt_gemm_bit_for_bit(g):
    """Seeded random shapes around every dispatch boundary of cfg = NULL (few rows on either side,
    one wave / several waves, N and K with and without 16-byte rows), integer-valued inputs: the
    tcgen05 path and the plain SIMT GEMM (reference.h:49-90 semantics) must agree in every bit."""
    import torch
    rng = np.random.default_rng(2024)
    gen = torch.Generator(device="cuda").manual_seed(2024)
    shapes = []
    for _ in range(36):
        M = int(rng.choice([1, 3, 15, 16, 17, 31, 32, 33, 63, 64, 65, 100, 128, 129, 200, 300]))
        N = int(rng.choice([1, 7, 64, 127, 128, 129, 136, 1000, 1024, 2500, 19072]))
        K = int(rng.choice([1, 8, 63, 64, 65, 520, 1000, 2048]))
        shapes.append((M, N, K))
    shapes += [(64, 19072, 264), (16, 40000, 72), (33, 129, 4097)]
    for M, N, K in shapes:
        a = torch.randint(-3, 4, (M, K), device="cuda", generator=gen).to(torch.bfloat16)
        b = torch.randint(-3, 4, (N, K), device="cuda", generator=gen).to(torch.bfloat16)
        got = g.gemm(a, b, alpha=0.5, beta=1.0)
        want = g.reference_gpu_gemm(a, b, alpha=0.5, beta=1.0)
        assert g.device_status()[0] == 0, (M, N, K)
        assert torch.equal(got.view(torch.int16), want.view(torch.int16)), (M, N, K)
