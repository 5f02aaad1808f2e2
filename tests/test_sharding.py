"""Multi-rank host logic on CPU: world_size-2 gloo processes shard M, compute their rows (the
oracle stands in for the GPU kernel here — test infrastructure), and the concatenation / the
chunked all-gather must equal the unsharded oracle result bit for bit."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import util
from h100_gemm_b200.sharding import ShardedGemm, chunk_rows, max_over_ranks, shard_rows
from oracle import oracle


def test_shard_rows_partition():
    for M, world, align in ((65536, 8, 1), (1000, 3, 1), (1000, 3, 256), (5, 8, 1), (8192, 1, 256)):
        ranges = [shard_rows(M, world, r, align) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == M
        for (b0, e0), (b1, e1) in zip(ranges, ranges[1:]):
            assert e0 == b1 and b0 <= e0
        assert all((b % align == 0) or b == M for b, _ in ranges)
    assert shard_rows(65536, 8, 3) == (24576, 32768)
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def test_chunk_rows():
    assert chunk_rows(8192, 4) == [(0, 2048), (2048, 4096), (4096, 6144), (6144, 8192)]
    assert chunk_rows(1000, 4) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert chunk_rows(100, 4) == [(0, 100)]
    assert chunk_rows(0, 4) == []


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, N, K, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        a = util.normal_bits((M, K), 1)
        b = util.normal_bits((N, K), 2, 0.02)
        begin, end = shard_rows(M, world, rank)

        def gemm_fn(a_rows, b_t, out_rows):
            res = oracle.cpu_gemm(util.to_bits(a_rows), util.to_bits(b_t))
            out_rows.copy_(torch.from_numpy(res.view(np.int16)).view(torch.bfloat16))

        a_t = torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)[begin:end].clone()
        b_t = torch.from_numpy(b.view(np.int16)).view(torch.bfloat16)
        sg = ShardedGemm(M, a_t, b_t, gemm_fn)
        shard = torch.empty(end - begin, N, dtype=torch.bfloat16)
        sg.compute(shard)
        full = torch.zeros(M, N, dtype=torch.bfloat16)
        sg.compute_and_gather(full, chunks=3)
        ref = oracle.cpu_gemm(a, b)
        ok_shard = np.array_equal(util.to_bits(shard), ref[begin:end])
        ok_full = np.array_equal(util.to_bits(full), ref)
        slowest = max_over_ranks(float(rank + 1))
        q.put((rank, ok_shard, ok_full, slowest))
    finally:
        dist.destroy_process_group()


def test_world_size_2_gloo_sharded_gemm():
    world, M, N, K = 2, 1024, 192, 160
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=60) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, ok_shard, ok_full, slowest in results:
        assert ok_shard and ok_full, f"rank {rank}"
        assert slowest == float(world)


def _leaving_worker(rank, world, port, M, N, K, q):
    """Step 1: both ranks gather. Then rank 1 leaves the job between steps (it never posts the
    exchange of step 2); rank 0's second gather must give up within its time limit."""
    import time
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from h100_gemm_b200.sharding import GatherTimeout
    a = util.integer_bits((M, K), 5)
    b = util.integer_bits((N, K), 6)
    begin, end = shard_rows(M, world, rank)

    def gemm_fn(a_rows, b_t, out_rows):
        res = oracle.cpu_gemm(util.to_bits(a_rows), util.to_bits(b_t))
        out_rows.copy_(torch.from_numpy(res.view(np.int16)).view(torch.bfloat16))

    a_t = torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)[begin:end].clone()
    b_t = torch.from_numpy(b.view(np.int16)).view(torch.bfloat16)
    sg = ShardedGemm(M, a_t, b_t, gemm_fn)
    full = torch.zeros(M, N, dtype=torch.bfloat16)
    sg.compute_and_gather(full, chunks=2, timeout_s=30.0)
    step1_ok = np.array_equal(util.to_bits(full), oracle.cpu_gemm(a, b))
    if rank == 1:
        q.put((rank, step1_ok, None, 0.0))
        time.sleep(8.0)   # gone from the job: no step 2, no collective in flight
        os._exit(0)
    t0 = time.monotonic()
    try:
        sg.compute_and_gather(full, chunks=2, timeout_s=2.0)
        outcome = "completed"
    except GatherTimeout:
        outcome = "timeout"
    q.put((rank, step1_ok, outcome, time.monotonic() - t0))
    q.close()
    q.join_thread()   # the result must reach the parent before the hard exit below
    os._exit(0)       # the process group cannot be torn down cleanly with a peer missing


def test_gather_gives_up_when_a_rank_leaves_between_steps():
    world, M, N, K = 2, 512, 64, 96
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_leaving_worker, args=(r, world, port, M, N, K, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    for _ in range(world):
        rank, step1_ok, outcome, seconds = q.get(timeout=60)
        results[rank] = (step1_ok, outcome, seconds)
    for p in procs:
        p.join(timeout=60)
    assert results[0][0] and results[1][0]          # the step before the rank left was complete
    assert results[0][1] == "timeout"               # the survivor was told, it did not hang
    assert results[0][2] < 6.0                      # within the stated limit (2 s) plus slack
