"""Two real GPUs: the fused GEMM + all-gather over peer-mapped memory (CUDA IPC + NVLink).
Skipped on machines with fewer than two devices; the single-device emulation of the same kernel
path is tests/test_gemm_gpu.py::test_fused_gather_epilogue_on_one_device."""
import os
import socket

import pytest

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import h100_gemm_b200 as g
        from h100_gemm_b200.sharding import FusedGatherGemm
        M, N, K = 2048, 1024, 1024
        gen = torch.Generator(device="cuda").manual_seed(5)            # same B on every rank
        b = (torch.randn(N, K, device="cuda", generator=gen) * 0.05).to(torch.bfloat16)
        gen.manual_seed(100 + rank)                                     # this rank's rows of A
        a = torch.randn(M, K, device="cuda", generator=gen).to(torch.bfloat16)
        import numpy as np
        import util
        from oracle import oracle  # the checker
        fg = FusedGatherGemm(M, N)
        own_ok = full_ok = oracle_ok = True
        side = torch.cuda.Stream()
        for step in range(4):
            # a new A every step (the two full-C buffers alternate); steps 2 and 3 run on a side stream
            a_step = (a * (step + 1)).to(torch.bfloat16)
            stream = side if step >= 2 else None
            if stream is not None:
                stream.wait_stream(torch.cuda.current_stream())
            full = fg.run(a_step, b, stream=stream)
            if stream is not None:
                torch.cuda.current_stream().wait_stream(stream)   # the readers below follow the all-reduce
            mine = g.gemm(a_step, b)
            own_ok &= bool(torch.equal(full[rank * M:(rank + 1) * M].view(torch.int16), mine.view(torch.int16)))
            # what the other rank wrote into my copy must be what it computed for itself
            parts = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(parts, mine)
            full_ok &= bool(torch.equal(full.view(torch.int16), torch.cat(parts).view(torch.int16)))
            if step == 0:
                # and the peer's rows in MY copy equal the CPU oracle on the peer's inputs
                peer = (rank + 1) % world
                gen.manual_seed(100 + peer)
                a_peer = torch.randn(M, K, device="cuda", generator=gen).to(torch.bfloat16)
                rows = np.arange(0, M, 97, dtype=np.int32)
                a_bits, b_bits = util.to_bits(a_peer), util.to_bits(b)
                want = oracle.cpu_gemm_rows(a_bits, b_bits, rows)
                got = util.to_bits(full[peer * M:(peer + 1) * M][rows.tolist()])
                oracle_ok = oracle.norm_relative_error(got, want, a_bits[rows], b_bits) <= 1e-2
        status = g.device_status()[0]
        fg.close()
        q.put((rank, own_ok, full_ok and oracle_ok, status))
    finally:
        dist.destroy_process_group()


def test_fused_gather_two_gpus():
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, own_ok, full_ok, status in results:
        assert own_ok and full_ok and status == 0, f"rank {rank}"
