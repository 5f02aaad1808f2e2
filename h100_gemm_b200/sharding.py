"""M-sharded multi-GPU GEMM: host-side logic (one process per GPU, torch.distributed plumbing).

Rows of A and C are split into contiguous shards, one per rank; B is replicated. Shards are
independent, so computing C needs NO collective; an all-gather of C over NCCL/NVLink is optional
and, when asked for, is issued per row chunk on a side stream so that it overlaps the GEMM of
the next chunk. The reference has no multi-GPU path (it is a single-GPU benchmark); this module
covers the M-sharded configuration of the build's benchmark matrix.

The compute step is injected (`gemm_fn`), so the partitioning, chunking and gather logic run
unchanged under the gloo backend on CPU in the tests.
"""
from __future__ import annotations

from typing import Callable, List, Optional, Tuple


def shard_rows(M: int, world: int, rank: int, align: int = 1) -> Tuple[int, int]:
    """Half-open row range of `rank`: equal shards of ceil(M/world) rounded up to `align` rows;
    trailing ranks may get fewer (or zero) rows."""
    if world < 1 or not (0 <= rank < world) or M < 0 or align < 1:
        raise ValueError("bad shard arguments")
    per = (M + world - 1) // world
    per = (per + align - 1) // align * align
    begin = min(M, rank * per)
    return begin, min(M, begin + per)


def chunk_rows(rows: int, chunks: int, align: int = 256) -> List[Tuple[int, int]]:
    """Splits a shard of `rows` rows into at most `chunks` contiguous pieces of `align`-row
    multiples (the last piece takes the remainder)."""
    if rows <= 0:
        return []
    chunks = max(1, chunks)
    per = (rows + chunks - 1) // chunks
    per = max(align, (per + align - 1) // align * align)
    return [(r, min(rows, r + per)) for r in range(0, rows, per)]


def max_over_ranks(value: float, device=None) -> float:
    """Timing rule for every multi-rank number: the slowest rank defines the step."""
    import torch
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    t = torch.tensor([value], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class GatherTimeout(RuntimeError):
    """The exchange of C shards did not complete in time: a peer is gone or has fallen behind."""


class ShardedGemm:
    """C[M,N] = A[M,K] @ B[N,K]^T with A and C row-sharded over the ranks of a process group.

    a_shard : this rank's rows of A, [rows, K]
    b       : the full B, [N, K] (replicated)
    gemm_fn : callable(a_rows, b, out_rows) computing out_rows = a_rows @ b^T in place
    """

    def __init__(self, M: int, a_shard, b, gemm_fn: Callable, group=None):
        import torch.distributed as dist
        self.dist = dist
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.M = M
        self.a, self.b, self.gemm_fn = a_shard, b, gemm_fn
        self.begin, self.end = shard_rows(M, self.world, self.rank)
        if a_shard.shape[0] != self.end - self.begin:
            raise ValueError("a_shard does not match this rank's row range")
        if M % self.world != 0:
            raise ValueError("M must divide evenly over the ranks for the gathered layout")
        self.rows = M // self.world

    def _global(self, group_rank: int) -> int:
        return group_rank if self.group is None else self.dist.get_global_rank(self.group, group_rank)

    def compute(self, out_shard) -> None:
        """No collective: every rank fills its own rows."""
        self.gemm_fn(self.a, self.b, out_shard)

    def compute_and_gather(self, out_full, chunks: int = 4, comm_stream=None, timeout_s: Optional[float] = None) -> None:
        """Fills the FULL C on every rank. Chunk j of every rank's shard is gathered while chunk
        j+1 is being multiplied (side stream on CUDA; sequential under gloo).

        `timeout_s` bounds the host-side wait for the exchange: when a peer has left the job
        between steps (it never posts its sends and receives), the call raises `GatherTimeout`
        after at most that long instead of waiting for ever. (Under NCCL the exchange is
        stream-ordered and the wait returns at once; there the process group's own timeout is the
        bound.)"""
        import torch
        rows, N = self.rows, out_full.shape[1]
        pieces = chunk_rows(rows, chunks)
        use_cuda = out_full.is_cuda
        main = torch.cuda.current_stream() if use_cuda else None
        handles = []
        for (r0, r1) in pieces:
            mine = out_full[self.begin + r0:self.begin + r1]
            self.gemm_fn(self.a[r0:r1], self.b, mine)
            if self.world == 1:
                continue
            # Every peer's piece of this chunk is a contiguous row range of the full C, so the
            # exchange is point-to-point sends and receives straight into place (one grouped NCCL
            # launch, no staging copy), issued on the side stream while the next chunk multiplies.
            ops = []
            for step in range(1, self.world):
                to = (self.rank + step) % self.world
                frm = (self.rank - step) % self.world
                ops.append(self.dist.P2POp(self.dist.isend, mine, self._global(to), group=self.group))
                ops.append(self.dist.P2POp(self.dist.irecv, out_full[frm * rows + r0:frm * rows + r1],
                                           self._global(frm), group=self.group))
            if use_cuda and comm_stream is not None:
                comm_stream.wait_stream(main)
                with torch.cuda.stream(comm_stream):
                    handles.extend(self.dist.batch_isend_irecv(ops))
            else:
                handles.extend(self.dist.batch_isend_irecv(ops))
        if timeout_s is None:
            for h in handles:
                h.wait()
        else:
            import datetime
            import time
            deadline = time.monotonic() + timeout_s
            for h in handles:
                left = deadline - time.monotonic()
                try:
                    done = left > 0 and h.wait(datetime.timedelta(seconds=max(left, 1e-3)))
                except RuntimeError as exc:  # gloo reports an expired wait as an error
                    raise GatherTimeout(f"rank {self.rank}: gather did not complete within {timeout_s} s: {exc}") from exc
                if done is False:
                    raise GatherTimeout(f"rank {self.rank}: gather did not complete within {timeout_s} s")
        if use_cuda and comm_stream is not None:
            main.wait_stream(comm_stream)


class FusedGatherGemm:
    """C = A @ B^T with A row-sharded over the ranks of one node and the all-gather of C done by
    the GEMM kernel itself: every rank owns full-C buffers that the other ranks map through CUDA
    IPC, and each rank's epilogue stores its tiles into all of them over NVLink (TMA stores to
    peer memory; no multicast, no library collective on the data path).

    Ordering. `run` enqueues, on ONE stream, the fused kernel and then a one-element all-reduce;
    the all-reduce of step n completes on a rank only after every rank's kernel of step n has
    completed, so work enqueued on that stream after `run` returns sees the whole C. Two full-C
    buffers alternate between steps: the kernels of step n + 1 write into the other buffer, and
    those of step n + 2 start only after the all-reduce of step n + 1, i.e. after every rank has
    run — in stream order — everything it enqueued between its steps n and n + 1. So the readers
    of a step's result must be enqueued on the same stream (or that stream must be made to wait
    for them) before the next `run`; then no rank overwrites a buffer a peer still reads.
    """

    def __init__(self, M_shard: int, N: int, group=None):
        import torch
        import torch.distributed as dist
        from . import api
        self.api, self.dist, self.group, self.torch = api, dist, group, torch
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        if self.world > 8:
            raise ValueError("the fused gather covers the ranks of one node (at most 8)")
        self.M, self.N = M_shard, N
        self.nbytes = self.world * M_shard * N * 2
        self.mine = api.DeviceBuffer(2 * self.nbytes)
        handles = [None] * self.world
        dist.all_gather_object(handles, self.mine.handle(), group=group)
        self.peers = [self.mine if p == self.rank else api.DeviceBuffer.from_handle(handles[p], 2 * self.nbytes)
                      for p in range(self.world)]
        both = self.mine.tensor((2, self.world * M_shard, N))
        self.buffers = [both[0], both[1]]
        self.ptrs = [[b.ptr + half * self.nbytes for b in self.peers] for half in (0, 1)]
        self.step = 0
        self.full = self.buffers[0]  # the buffer the most recent run() filled
        self._token = torch.zeros(1, device="cuda")

    def run(self, a_shard, b, cfg=None, stream=None):
        """Enqueues the fused kernel and the completion all-reduce on `stream` (default: the
        current stream) and returns this step's full C (also `self.full`)."""
        torch = self.torch
        stream = stream if stream is not None else torch.cuda.current_stream()
        half = self.step & 1
        with torch.cuda.stream(stream):
            self.api.gemm_gather(a_shard, b, self.ptrs[half], self.rank, cfg=cfg, stream=stream)
            self.dist.all_reduce(self._token, group=self.group)
        self.full = self.buffers[half]
        self.step += 1
        return self.full

    def close(self) -> None:
        self.torch.cuda.synchronize()
        self.dist.barrier(group=self.group)
        for p, buf in enumerate(self.peers):
            if p != self.rank:
                buf.close()
        self.dist.barrier(group=self.group)
        self.mine.close()
