// Persistent tile scheduler: which (tile, K-range) segments each worker (a CTA, or a CTA pair)
// processes, and in which order tiles are rasterised over the output.
//
// Replaces the reference's static along-N TileScheduler (matmul_h100.cu.jinja:392-439) and the
// 16x8 supertile Schedule (matmul_utils.cuh:348-378). Three decompositions share one iterator:
//   mode 0  data-parallel : worker w takes tiles w, w+W, w+2W, ... over the full K range
//   mode 1  split-K       : every tile is cut into `split_k` K-slices; partial sums go to slots
//   mode 2  stream-K      : the tiles x k_tiles iteration space is cut into W equal contiguous
//                           ranges; a range's first/last tile may be partial
//   mode 3  hybrid        : the full waves of tiles run data-parallel; only the tiles of the last,
//                           partly filled wave are cut stream-K style, so every worker finishes at
//                           the same time without paying for partial tiles on the full waves
//   mode 4  hybrid, two waves : as mode 3, but the last FULL wave is cut stream-K style together
//                           with the partly filled one, so every worker's share is at least one
//                           tile long and a tile has at most three contributors however few tiles
//                           the last wave holds
// Partial segments carry a slot index into an fp32 workspace. Split-K slots are summed in slot
// order by a fix-up pass. Under stream-K a tile cut across workers is finished inside the GEMM
// kernel: the worker holding the tile's head (k_begin == 0) adds the partial tiles of the workers
// holding its later K-ranges, in K order. Those partials are always the FIRST segment of their
// worker, so the finisher never waits on work that is queued behind its own. Either way the
// summation order is fixed and results do not depend on timing.
//
// Everything here compiles for the host as well, so coverage (every (tile, k) iteration visited
// exactly once) is tested exhaustively without a GPU.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define B200_SCHED_HD __host__ __device__ __forceinline__
#else
#define B200_SCHED_HD inline
#endif

namespace b200 {

enum SchedMode : int { kDataParallel = 0, kSplitK = 1, kStreamK = 2, kHybrid = 3, kHybridTwoWaves = 4 };

B200_SCHED_HD bool sched_has_streamk_part(int mode) {
  return mode == kStreamK || mode == kHybrid || mode == kHybridTwoWaves;
}

struct SchedParams {
  int tiles_m;      // output tiles along M
  int tiles_n;      // output tiles along N
  int batch;        // independent problems
  int num_tiles;    // tiles_m * tiles_n * batch
  int k_tiles;      // K-tiles (of 64 elements) per output tile
  int group;        // raster group width in tiles (>= 1)
  int raster;       // 0: groups of `group` M-tiles, walked M-fastest; 1: same along N
  int mode;         // SchedMode
  int split_k;      // K-slices per tile (mode 1)
  int num_workers;  // CTAs (or CTA pairs) in the grid
};

struct TileCoord {
  int m;  // tile index along M
  int n;  // tile index along N
  int b;  // batch index
};

struct Segment {
  int tile;     // linear tile id
  int k_begin;  // first K-tile (inclusive)
  int k_end;    // last K-tile (exclusive)
  int slot;     // >= 0: write the fp32 partial tile to this slot; < 0: write the output
  int finish;   // 1: (stream-K) before writing the output, add the partial slots of the workers
                //    that hold the rest of this tile's K range (see streamk_contributors)
};

// Linear tile id -> coordinates. Inside a batch, tiles are grouped into bands of `group` tiles
// along the grouped dimension and walked fastest along it, so that the tiles in flight at one
// time (consecutive ids) form a compact block of the output and share operand panels in L2.
B200_SCHED_HD TileCoord tile_coord(const SchedParams& p, int tile) {
  TileCoord c;
  const int per_batch = p.tiles_m * p.tiles_n;
  c.b = tile / per_batch;
  int t = tile - c.b * per_batch;
  const int major = p.raster == 0 ? p.tiles_m : p.tiles_n;  // grouped dimension
  const int minor = p.raster == 0 ? p.tiles_n : p.tiles_m;
  const int band_size = p.group * minor;
  const int band = t / band_size;
  const int first = band * p.group;
  const int width = (major - first) < p.group ? (major - first) : p.group;
  const int r = t - band * band_size;
  const int a = first + r % width;
  const int o = r / width;
  c.m = p.raster == 0 ? a : o;
  c.n = p.raster == 0 ? o : a;
  return c;
}

B200_SCHED_HD long long sched_total_iters(const SchedParams& p) {
  return static_cast<long long>(p.num_tiles) * p.k_tiles;
}

// First tile of the stream-K part: 0 for pure stream-K, the end of the last full wave for hybrid.
B200_SCHED_HD int streamk_tile_base(const SchedParams& p) {
  if (p.mode == kStreamK) return 0;
  if (p.mode == kHybrid) return (p.num_tiles / p.num_workers) * p.num_workers;
  if (p.mode == kHybridTwoWaves) {
    const int full = p.num_tiles / p.num_workers;
    if (full * p.num_workers == p.num_tiles) return p.num_tiles;  // no partly filled wave: nothing to cut
    return (full > 0 ? full - 1 : 0) * p.num_workers;
  }
  return p.num_tiles;
}

// Iterations (tile, k-tile) in the stream-K part.
B200_SCHED_HD long long streamk_iters(const SchedParams& p) {
  return static_cast<long long>(p.num_tiles - streamk_tile_base(p)) * p.k_tiles;
}

// First iteration of worker w's contiguous range in the stream-K part.
B200_SCHED_HD long long streamk_begin(const SchedParams& p, int w) {
  return streamk_iters(p) * w / p.num_workers;
}

// K-range of slice s under split-K.
B200_SCHED_HD int splitk_begin(const SchedParams& p, int s) {
  return static_cast<int>(static_cast<long long>(p.k_tiles) * s / p.split_k);
}

// Number of fp32 partial slots the workspace must hold.
B200_SCHED_HD long long sched_num_slots(const SchedParams& p) {
  if (p.mode == kSplitK) return p.split_k > 1 ? static_cast<long long>(p.split_k) * p.num_tiles : 0;
  if (sched_has_streamk_part(p.mode)) {
    return streamk_iters(p) > 0 ? p.num_workers : 0;  // one per worker: its first stream-K segment
  }
  return 0;
}

// Iterates over the segments of one worker. All roles of a CTA (producer, MMA issuer, epilogue)
// run their own copy and therefore agree on the sequence without communicating.
struct WorkIter {
  const SchedParams& p;
  int worker;
  long long cur;       // data-parallel / split-K phase: next unit id
  long long unit_end;  // data-parallel / split-K phase: end of units
  long long sk_cur;    // stream-K phase: next iteration
  long long sk_end;    // stream-K phase: end of this worker's range
  long long sk_range_begin;
  int sk_tile_base;

  B200_SCHED_HD WorkIter(const SchedParams& params, int w) : p(params), worker(w) {
    sk_tile_base = streamk_tile_base(p);
    cur = w;
    unit_end = p.mode == kSplitK ? static_cast<long long>(p.num_tiles) * p.split_k : sk_tile_base;
    if (p.mode == kDataParallel) unit_end = p.num_tiles;
    sk_cur = streamk_begin(p, w);
    sk_end = streamk_begin(p, w + 1);
    sk_range_begin = sk_cur;
    if (p.mode == kDataParallel || p.mode == kSplitK) sk_cur = sk_end = 0;
  }

  B200_SCHED_HD bool next(Segment& s) {
    if (cur < unit_end) {
      if (p.mode == kSplitK) {
        const int slice = static_cast<int>(cur / p.num_tiles);
        s.tile = static_cast<int>(cur - static_cast<long long>(slice) * p.num_tiles);
        s.k_begin = splitk_begin(p, slice);
        s.k_end = splitk_begin(p, slice + 1);
        s.slot = p.split_k > 1 ? slice * p.num_tiles + s.tile : -1;
      } else {
        s.tile = static_cast<int>(cur);
        s.k_begin = 0;
        s.k_end = p.k_tiles;
        s.slot = -1;
      }
      s.finish = 0;
      cur += p.num_workers;
      return true;
    }
    if (sk_cur >= sk_end) return false;
    const int t = static_cast<int>(sk_cur / p.k_tiles);  // tile index inside the stream-K part
    const long long tile_first = static_cast<long long>(t) * p.k_tiles;
    s.tile = sk_tile_base + t;
    s.k_begin = static_cast<int>(sk_cur - tile_first);
    long long stop = tile_first + p.k_tiles;
    if (stop > sk_end) stop = sk_end;
    s.k_end = static_cast<int>(stop - tile_first);
    // A range that starts inside a tile contributes a partial; the range holding the tile's head
    // finishes it when the tile's tail belongs to other workers.
    s.slot = s.k_begin > 0 ? worker : -1;
    s.finish = (s.k_begin == 0 && s.k_end < p.k_tiles) ? 1 : 0;
    sk_cur = stop;
    return true;
  }
};

// For the fix-up pass: the slots that hold partial sums of `tile`, in summation order.
// Returns the count (0 when the tile was produced whole); writes at most `cap` slot ids.
B200_SCHED_HD int tile_partial_slots(const SchedParams& p, int tile, int* slots, int cap) {
  int n = 0;
  if (p.mode == kSplitK) {
    if (p.split_k <= 1) return 0;
    for (int s = 0; s < p.split_k; ++s) {
      if (splitk_begin(p, s + 1) == splitk_begin(p, s)) continue;  // empty slice
      if (n < cap) slots[n] = s * p.num_tiles + tile;
      ++n;
    }
    return n;
  }
  return 0;
}

// Stream-K: the workers whose partial slots complete the tile that `worker` holds the head of.
// They are the consecutive workers after `worker` whose ranges start before the tile ends;
// worker w's partial lives in slot w. Returns their count; *first = worker + 1.
B200_SCHED_HD int streamk_contributors(const SchedParams& p, int worker, int tile, int* first) {
  const long long tile_end = (static_cast<long long>(tile - streamk_tile_base(p)) + 1) * p.k_tiles;
  *first = worker + 1;
  int n = 0;
  for (int w = worker + 1; w < p.num_workers && streamk_begin(p, w) < tile_end; ++w) ++n;
  return n;
}

}  // namespace b200
