"""The NVLink load of an W-rank fused GEMM + all-gather on TWO GPUs: each of the two ranks gives
b200_gemm_bf16_gather W destinations — its own copy of C and W - 1 distinct regions of the one
peer's memory — so every tile crosses the link W - 1 times, as it would to W - 1 peers. Separates
what the kernel and one link cost from what a switch and many writers into one memory would add.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        h100_gemm_b200/bench/gather_two_gpu_emulation.py [W=8]

Prints one JSON line: ms per launch (CUDA events, max over the two ranks, 20 launches) for 256 and
128 rows per CTA, and whether every region the peer wrote holds the peer's own result. With
``--roles`` after W it adds, per tile shape, the cycle counters of one traced launch on rank 0
(means over the CTAs): kernel total, MMA issuer waiting for operands, first epilogue warp waiting
for an accumulator, and accumulator-ready to stores-issued."""
import os, sys, json
sys.path.insert(0, str(__import__("pathlib").Path(__file__).resolve().parents[2]))
import torch, torch.distributed as dist
import h100_gemm_b200 as g
from h100_gemm_b200 import api
rank = int(os.environ["RANK"]); local = int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local)
os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
dist.init_process_group("nccl", device_id=torch.device("cuda", local))
M = N = K = 8192
EMUL = int(sys.argv[1]) if len(sys.argv) > 1 else 8
gen = torch.Generator(device="cuda").manual_seed(5)
b = (torch.randn(N, K, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
gen.manual_seed(100 + rank)
a = torch.randn(M, K, device="cuda", generator=gen).to(torch.bfloat16)
nbytes = 16 * M * N * 2
mine = api.DeviceBuffer(nbytes)
handles = [None, None]
dist.all_gather_object(handles, mine.handle())
peer = api.DeviceBuffer.from_handle(handles[1 - rank], nbytes)
ptrs = [mine.ptr if q == rank else peer.ptr + q * M * N * 2 for q in range(EMUL)]
token = torch.zeros(1, device="cuda")
stream = torch.cuda.current_stream()
ref = g.gemm(a, b)
out = {}
for rnd in range(2):
    for tile, cfg in (("256", api.GemmConfig(block_m=256, block_n=256, cluster_m=2, epilogue=1)), ("128", api.GemmConfig(block_m=128, block_n=256, cluster_m=2, epilogue=1))):
        for _ in range(3):
            api.gemm_gather(a, b, ptrs, rank, cfg=cfg, stream=stream); dist.all_reduce(token)
        torch.cuda.synchronize(); dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(20):
            api.gemm_gather(a, b, ptrs, rank, cfg=cfg, stream=stream); dist.all_reduce(token)
        e1.record(); torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 20], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out.setdefault(f"{tile} rows per CTA", []).append(round(float(t.item()), 4))
roles = {}
if "--roles" in sys.argv:
    for tile, cfg in (("256", api.GemmConfig(block_m=256, block_n=256, cluster_m=2, epilogue=1)), ("128", api.GemmConfig(block_m=128, block_n=256, cluster_m=2, epilogue=1))):
        counters = torch.zeros(148 * 8, dtype=torch.int64, device="cuda")
        api.set_profile_buffer(counters)
        try:
            for _ in range(3):
                api.gemm_gather(a, b, ptrs, rank, cfg=cfg, stream=stream); dist.all_reduce(token)
            torch.cuda.synchronize(); dist.barrier()
            counters.zero_()
            api.gemm_gather(a, b, ptrs, rank, cfg=cfg, stream=stream); dist.all_reduce(token)
            torch.cuda.synchronize()
        finally:
            api.set_profile_buffer(None)
        mean = counters.view(148, 8).double().mean(0).tolist()
        roles[f"{tile} rows per CTA"] = {name: int(mean[api.PROFILE_SLOTS.index(name)])
                                        for name in ("total", "mma_wait_full", "epi_wait_full", "epi_busy")}
# correctness of the last variant: what the PEER wrote into my buffer (regions q != peer's rank... it wrote to my_base + q*M*N*2 + peerrank*M*N elements)
dist.barrier(); torch.cuda.synchronize()
full = mine.tensor((16 * M, N))
peer_ref = [torch.empty_like(ref) for _ in range(2)]
dist.all_gather(peer_ref, ref)
ok = True
pr = 1 - rank
for q in range(EMUL):
    if q == pr: continue   # the peer's own copy slot: not written into my memory
    rows0 = q * M + pr * M
    ok &= bool(torch.equal(full[rows0:rows0 + M].view(torch.int16), peer_ref[pr].view(torch.int16)))
own_ok = bool(torch.equal(full[rank * M:(rank + 1) * M].view(torch.int16), ref.view(torch.int16)))
st = g.device_status()[0]
if rank == 0:
    print(json.dumps({"emulated_world": EMUL, "ms": out, "peer_regions_ok": ok, "own_ok": own_ok, "status": st, **({"cycles": roles} if roles else {})}), flush=True)
dist.barrier()
peer.close(); dist.barrier(); mine.close()
dist.destroy_process_group()
