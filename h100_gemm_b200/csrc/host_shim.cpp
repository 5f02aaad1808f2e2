// Host-only C exports of the scheduler and descriptor helpers, so their arithmetic can be
// unit-tested without a GPU (built with g++, no CUDA). Not part of the product library.
#include "sm100/desc.cuh"
#include "sm100/scheduler.cuh"

using namespace b200;

extern "C" {

unsigned int hs_instr_desc(unsigned int m, unsigned int n, int bf16) {
  return make_instr_desc(m, n, bf16 ? InFormat::BF16 : InFormat::F16);
}
unsigned long long hs_smem_desc(unsigned int addr) { return make_smem_desc_sw128(addr); }
unsigned int hs_sw128_offset(unsigned int row, unsigned int chunk) { return sw128_offset(row, chunk); }

static SchedParams make(int tiles_m, int tiles_n, int batch, int k_tiles, int group, int raster,
                        int mode, int split_k, int workers) {
  SchedParams p;
  p.tiles_m = tiles_m;
  p.tiles_n = tiles_n;
  p.batch = batch;
  p.num_tiles = tiles_m * tiles_n * batch;
  p.k_tiles = k_tiles;
  p.group = group;
  p.raster = raster;
  p.mode = mode;
  p.split_k = split_k;
  p.num_workers = workers;
  return p;
}

void hs_tile_coord(int tiles_m, int tiles_n, int batch, int group, int raster, int tile, int* out) {
  SchedParams p = make(tiles_m, tiles_n, batch, 1, group, raster, 0, 1, 1);
  TileCoord c = tile_coord(p, tile);
  out[0] = c.m;
  out[1] = c.n;
  out[2] = c.b;
}

// Writes up to cap segments (tile, k_begin, k_end, slot, finish) of one worker; returns the count.
int hs_segments(int tiles_m, int tiles_n, int batch, int k_tiles, int mode, int split_k, int workers,
                int worker, int* out, int cap) {
  SchedParams p = make(tiles_m, tiles_n, batch, k_tiles, 8, 0, mode, split_k, workers);
  WorkIter it(p, worker);
  Segment s;
  int n = 0;
  while (it.next(s)) {
    if (n < cap) {
      out[5 * n + 0] = s.tile;
      out[5 * n + 1] = s.k_begin;
      out[5 * n + 2] = s.k_end;
      out[5 * n + 3] = s.slot;
      out[5 * n + 4] = s.finish;
    }
    ++n;
  }
  return n;
}

int hs_tile_slots(int tiles_m, int tiles_n, int batch, int k_tiles, int mode, int split_k, int workers,
                  int tile, int* out, int cap) {
  SchedParams p = make(tiles_m, tiles_n, batch, k_tiles, 8, 0, mode, split_k, workers);
  return tile_partial_slots(p, tile, out, cap);
}

int hs_streamk_contributors(int tiles_m, int tiles_n, int batch, int k_tiles, int mode, int workers, int worker,
                            int tile, int* first) {
  SchedParams p = make(tiles_m, tiles_n, batch, k_tiles, 8, 0, mode, 1, workers);
  return streamk_contributors(p, worker, tile, first);
}

long long hs_num_slots(int tiles_m, int tiles_n, int batch, int k_tiles, int mode, int split_k, int workers) {
  SchedParams p = make(tiles_m, tiles_n, batch, k_tiles, 8, 0, mode, split_k, workers);
  return sched_num_slots(p);
}
}
