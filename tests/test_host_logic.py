"""Scheduler and descriptor arithmetic, compiled for the host (csrc/host_shim.cpp)."""
import ctypes
from collections import defaultdict

import pytest

from h100_gemm_b200 import build


@pytest.fixture(scope="module")
def shim():
    lib = ctypes.CDLL(str(build.build_host_shim()))
    lib.hs_smem_desc.restype = ctypes.c_ulonglong
    lib.hs_num_slots.restype = ctypes.c_longlong
    return lib


def segments(shim, tm, tn, batch, kt, mode, split, workers, w):
    buf = (ctypes.c_int * (5 * 8192))()
    n = shim.hs_segments(tm, tn, batch, kt, mode, split, workers, w, buf, 8192)
    assert n <= 8192
    return [tuple(buf[5 * i:5 * i + 5]) for i in range(n)]


def test_instruction_descriptor_bits(shim):
    # bf16 x bf16 -> fp32, K-major A and B, M=256 (CTA pair), N=256
    d = shim.hs_instr_desc(256, 256, 1)
    assert (d >> 4) & 0x3 == 1          # accumulator fp32
    assert (d >> 7) & 0x7 == 1          # A = bf16
    assert (d >> 10) & 0x7 == 1         # B = bf16
    assert (d >> 15) & 0x3 == 0         # both K-major
    assert (d >> 17) & 0x3F == 256 >> 3
    assert (d >> 24) & 0x1F == 256 >> 4
    d = shim.hs_instr_desc(128, 64, 0)
    assert (d >> 7) & 0x7 == 0 and (d >> 10) & 0x7 == 0
    assert (d >> 17) & 0x3F == 8 and (d >> 24) & 0x1F == 8


def test_smem_descriptor_bits(shim):
    d = shim.hs_smem_desc(0x12400)
    assert d & 0x3FFF == 0x12400 >> 4
    assert (d >> 16) & 0x3FFF == 0                # leading byte offset unused
    assert (d >> 32) & 0x3FFF == 1024 >> 4        # 8 rows x 128 B between row groups
    assert (d >> 46) & 0x3 == 1                   # descriptor version
    assert (d >> 49) & 0x7 == 0                   # base offset (1024-B aligned tiles)
    assert (d >> 61) & 0x7 == 2                   # 128-byte swizzle


def test_swizzle_offsets_are_a_permutation(shim):
    # Within each 8-row x 128-byte atom the 64 sixteen-byte chunks map one-to-one.
    for base_row in (0, 8, 24):
        seen = {shim.hs_sw128_offset(base_row + r, c) for r in range(8) for c in range(8)}
        assert seen == {base_row * 128 + 16 * i for i in range(64)}
    assert shim.hs_sw128_offset(0, 3) == 48 and shim.hs_sw128_offset(1, 0) == 128 + 16


@pytest.mark.parametrize("tm,tn,batch,group,raster", [(4, 4, 1, 8, 0), (32, 32, 1, 8, 0), (13, 7, 1, 4, 0),
                                                       (13, 7, 3, 4, 1), (1, 224, 1, 8, 0), (5, 1, 2, 2, 1)])
def test_tile_coord_is_a_bijection(shim, tm, tn, batch, group, raster):
    out = (ctypes.c_int * 3)()
    seen = set()
    for t in range(tm * tn * batch):
        shim.hs_tile_coord(tm, tn, batch, group, raster, t, out)
        m, n, b = out[0], out[1], out[2]
        assert 0 <= m < tm and 0 <= n < tn and 0 <= b < batch
        seen.add((m, n, b))
    assert len(seen) == tm * tn * batch


def streamk_base(mode, tiles, workers):
    """First tile of the part that is cut stream-K style."""
    full = tiles // workers
    if mode == 2:
        return 0
    if mode == 3:
        return full * workers
    if full * workers == tiles:
        return tiles                       # mode 4 without a partly filled wave: all tiles stay whole
    return max(full - 1, 0) * workers


CASES = [(4, 4, 1, 16), (32, 32, 1, 128), (1, 224, 1, 128), (3, 5, 2, 9), (1, 1, 1, 1), (1, 3, 1, 200), (7, 3, 1, 2)]


@pytest.mark.parametrize("tm,tn,batch,kt", CASES)
@pytest.mark.parametrize("mode,split", [(0, 1), (1, 2), (1, 3), (1, 5), (2, 1), (3, 1), (4, 1)])
@pytest.mark.parametrize("workers", [1, 7, 66, 74, 132, 148])
def test_every_k_iteration_is_visited_exactly_once(shim, tm, tn, batch, kt, mode, split, workers):
    tiles = tm * tn * batch
    if mode == 1:
        split = min(split, kt)
        if split <= 1:
            mode, split = 0, 1
    if mode in (3, 4) and tiles <= workers:
        mode = 0  # what the launcher does: a single wave has nothing to balance against
    units = tiles * (split if mode == 1 else 1) if mode != 2 else tiles * kt
    workers = min(workers, units)
    visits = defaultdict(int)
    slots_by_tile = defaultdict(list)
    used_slots = set()
    per_worker = {}
    for w in range(workers):
        segs = segments(shim, tm, tn, batch, kt, mode, split, workers, w)
        per_worker[w] = segs
        for i, (tile, kb, ke, slot, finish) in enumerate(segs):
            assert 0 <= tile < tiles and 0 <= kb < ke <= kt
            for k in range(kb, ke):
                visits[(tile, k)] += 1
            full = kb == 0 and ke == kt
            if mode == 0:
                assert slot < 0 and finish == 0
            if mode in (2, 3, 4):
                # partials are contributed only by a worker's first stream-K segment, into its own
                # slot; the holder of the tile's head finishes it
                base = streamk_base(mode, tiles, workers)
                first_sk = next((j for j, sg in enumerate(segs) if sg[0] >= base), None)
                assert (slot >= 0) == (kb > 0) and (slot < 0 or (slot == w and i == first_sk))
                if tile < base:
                    assert full and i < first_sk if first_sk is not None else full
                assert finish == (1 if (kb == 0 and ke < kt) else 0)
                assert not full or (slot < 0 and finish == 0)
            if slot >= 0:
                assert slot not in used_slots, "two segments share a partial slot"
                used_slots.add(slot)
                slots_by_tile[tile].append((kb, slot))
    assert len(visits) == tiles * kt and set(visits.values()) == {1}
    nslots = shim.hs_num_slots(tm, tn, batch, kt, mode, split, workers)
    assert all(s < nslots for s in used_slots)
    buf = (ctypes.c_int * 64)()
    if mode == 1:
        # the fix-up pass must find exactly the slots that were written, in K order
        for tile in range(tiles):
            n = shim.hs_tile_slots(tm, tn, batch, kt, mode, split, workers, tile, buf, 64)
            assert n <= 64
            assert [buf[i] for i in range(n)] == [s for _, s in sorted(slots_by_tile[tile])]
    if mode in (2, 3, 4):
        # every finisher's contributors are the next workers' first segments and tile the rest of K
        base = streamk_base(mode, tiles, workers)
        first = ctypes.c_int()
        for w, segs in per_worker.items():
            for tile, kb, ke, slot, finish in segs:
                if not finish:
                    continue
                n = shim.hs_streamk_contributors(tm, tn, batch, kt, mode, workers, w, tile, ctypes.byref(first))
                assert n >= 1 and first.value == w + 1
                pos = ke
                for c in range(first.value, first.value + n):
                    ctile, ckb, cke, cslot, cfin = next(sg for sg in per_worker[c] if sg[0] >= base)
                    assert ctile == tile and ckb == pos and cslot == c and cfin == 0
                    pos = cke
                assert pos == kt
        # and every contributed slot is consumed by exactly one finisher
        finished_tiles = {tile for segs in per_worker.values() for tile, _, _, _, f in segs if f}
        assert set(slots_by_tile) == finished_tiles


def test_streamk_balances_work(shim):
    # Skinny decode shape: 1 x 224 tiles of 128 K-tiles over 148 workers.
    loads = []
    for w in range(148):
        loads.append(sum(ke - kb for _, kb, ke, _, _ in segments(shim, 1, 224, 1, 128, 2, 1, 148, w)))
    assert sum(loads) == 224 * 128 and max(loads) - min(loads) <= 1
