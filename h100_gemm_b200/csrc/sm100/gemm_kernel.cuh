// The one warp-specialised persistent GEMM kernel for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T,
// 16-bit inputs (bf16 or fp16), fp32 accumulation in tensor memory, output in the input type.
//
// It takes the place of both reference kernels — gpu_gemm_kernel (matmul_h100.cu.jinja:734-925:
// producer warpgroup + two ping-pong WGMMA consumer warpgroups) and matmulKernel
// (matmul_utils.cuh:380-566: producer + two cooperative consumers) — with a Blackwell design:
//
//   warp 0      TMA producer   one lane streams A/B K-tiles into a shared-memory ring
//   warp 1      MMA issuer     one lane issues tcgen05.mma; owns tensor-memory alloc/dealloc
//   warps 2-5   epilogue       tcgen05.ld -> bf16 -> either swizzled smem -> TMA store, or
//   (4-11 if MT = 2; then      16-byte global stores straight from registers
//    warps 2-3 idle)
//
// Barriers (all mbarriers in shared memory, every wait bounded):
//   full[s]       TMA bytes of stage s have landed           (producer -> MMA issuer)
//   empty[s]      MMAs reading stage s have completed        (tcgen05.commit -> producer)
//   tmem_full[a]  accumulator buffer a holds a finished tile (tcgen05.commit -> epilogue)
//   tmem_empty[a] accumulator buffer a has been read out     (epilogue -> MMA issuer)
// Two accumulator buffers in tensor memory let the epilogue of one tile overlap the main loop of
// the next; this replaces the reference's two consumer warpgroups and its OrderedBarrier
// (matmul_h100.cu.jinja:61-113).
//
// PAIR = 1 runs a CTA pair (cluster of 2 along M) as one worker: tcgen05.mma.cta_group::2 computes
// a 256 x BN tile, each CTA stages its own 128 rows of A and BN/2 rows of B with plain (unicast)
// TMA loads that complete on the leader CTA's full[s]; the leader alone issues MMAs and signals
// empty[s] / tmem_full[a] in both CTAs with one commit.
//
// MT = 2 gives every CTA two 128-row sub-tiles of A per K-tile (a 256 x BN accumulator per CTA,
// 512 x BN per pair): the B tile is then reused by twice as many MMAs per byte loaded, which cuts
// L2 -> shared-memory traffic per FLOP by a quarter. With BN = 256 the two accumulators fill all
// 512 tensor-memory columns, so there is one accumulator buffer: what is exposed of a tile's
// epilogue is the read-out of the accumulator (the epilogue warps drain it into registers and
// hand it back before they store anything); the stores run under the next tile's main loop.
#pragma once

#include <cuda_bf16.h>

#include "desc.cuh"
#include "ptx.cuh"
#include "scheduler.cuh"

namespace b200 {

static constexpr int kBlockK = 64;          // one 128-byte swizzle row of 16-bit elements
static constexpr int kUmmaK = 16;           // K of one tcgen05.mma (16-bit inputs)
static constexpr int kCtaRows = 128;        // accumulator rows (TMEM lanes) per CTA
static constexpr int kMaxStages = 24;
static constexpr int kEpiChunkCols = 64;    // columns per TMA store (128 bytes of bf16)
static constexpr int kEpiSlabBytes = 32 * kEpiChunkCols * 2;       // one warp, one buffer: 4 KB
static constexpr int kBarrierBytes = 512;

// Device status codes written to the status word when a bounded wait gives up.
enum DeviceStatus : unsigned int {
  kStatusOk = 0,
  kStatusProducerTimeout = 1,   // producer waited for empty[s]
  kStatusMmaFullTimeout = 2,    // MMA issuer waited for full[s]
  kStatusMmaTmemTimeout = 3,    // MMA issuer waited for tmem_empty[a]
  kStatusEpilogueTimeout = 4,   // epilogue waited for tmem_full[a]
  kStatusStreamKTimeout = 5,    // stream-K finisher waited for another worker's partial tile
  kStatusSelfTestTimeout = 9,   // the bounded-wait self-test (an mbarrier nothing arrives on)
};

// Per-CTA cycle counters written when GemmArgs::profile is set: where each role spent its time.
// (The reference passes a debug buffer "DB" to runKernel for the same purpose but its kernel never
// writes it, matmul_h100_optimal.cu:132-139,167-198.)
enum ProfileSlot : int {
  kProfTotal = 0,          // kernel entry to exit (thread 0)
  kProfProducerWait = 1,   // TMA producer waiting for a free stage
  kProfMmaWaitFull = 2,    // MMA issuer waiting for operands
  kProfMmaWaitTmem = 3,    // MMA issuer waiting for an accumulator buffer
  kProfEpiWaitFull = 4,    // first epilogue warp waiting for a finished accumulator
  kProfEpiDrain = 5,       // first epilogue warp: accumulator ready -> buffer handed back
  kProfEpiBusy = 6,        // first epilogue warp: accumulator ready -> tile's stores issued
  kProfTiles = 7,          // segments processed
  kProfileSlots = 8
};

enum StoreMode : int {
  kStoreTma = 0,     // staging slab in shared memory, then a TMA tile store
  kStoreVector = 1,  // 16-byte global stores from registers (needs 16-byte aligned rows of C)
  kStoreScalar = 2,  // predicated 2-byte stores (any alignment)
  kStoreStaged = 3,  // transpose through a per-warp shared-memory slab, then coalesced 16-byte stores
};

struct GemmArgs {
  int M, N, K, batch;
  SchedParams sched;
  int stages;
  int gather_world;           // fused all-gather: number of destination copies of C (0 = plain GEMM)
  int f16;                    // 0: bf16 inputs and output; 1: IEEE fp16 (selects the F16 kernel; used by fix-up)
  int store_mode;             // StoreMode: how the epilogue writes C
  int epi_bytes;              // shared memory reserved for TMA-store staging (0 unless kStoreTma)
  __nv_bfloat16* C;           // used when c_direct
  long long ldc;              // elements between rows of C
  long long c_batch_stride;   // elements between batches of C
  float* partial;             // fp32 slots for split-K / stream-K partial tiles
  unsigned long long* flags;  // stream-K: 16 words per slot (CTA rank x epilogue warp), set to `epoch`
  unsigned long long epoch;   // value that marks a slot as written by THIS launch
  long long* profile;         // optional: kProfileSlots cycle counters per CTA (see ProfileSlot)
  int a_rows;                 // rows of A staged per CTA and K-tile (128, or fewer when M < 128)
  int a_stage_bytes;          // a_rows * 128
  float alpha, beta;
  int scale;                  // 1: C = acc * alpha + beta (the scalar-beta rule of reference.h:40)
  int c_transposed;           // 1: element (row, col) of the kernel's product goes to C[col * ldc + row]
                              //    (few-rows plan: the caller's rows ride the MMA's N; 2-byte stores only)
  unsigned int* status;       // 4 words: code, block, tile, detail
};

template <int BN, int PAIR, int MT>
struct KernelTraits {
  static_assert(BN == 16 || BN == 32 || (BN % 64 == 0 && BN >= 64 && BN <= 256) || (BN == 224 && MT == 1),
                "BN must be 16, 32, 64, 128, 192, 224 (whole tiles, one sub-tile) or 256");
  static_assert(MT == 1 || MT == 2, "one or two 128-row sub-tiles of A per CTA");
  static constexpr int kCtaGroup = PAIR ? 2 : 1;
  static constexpr int kUmmaM = kCtaRows * kCtaGroup;         // rows of one tcgen05.mma
  static constexpr int kCtaM = kCtaRows * MT;                 // rows of C per CTA
  static constexpr int kBlockM = kCtaM * kCtaGroup;           // rows of C per worker tile
  static constexpr int kBRowsCta = BN / kCtaGroup;
  static constexpr int kABytes = kCtaM * kBlockK * 2;         // with a full A tile
  static constexpr int kBBytes = kBRowsCta * kBlockK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kChunks = MT * BN / kEpiChunkCols;     // 64-column chunks of a CTA's accumulator
  static constexpr int kEpiWarps = 4 * MT;                    // one per TMEM lane quadrant and sub-tile
  // First epilogue warp. With two sub-tiles the epilogue warps form warpgroups of their own (warps
  // 4-11; warps 2 and 3 idle) so that the register file can be re-partitioned per warpgroup:
  // 56 registers for the warpgroup of the two single-thread roles, 224 for the epilogue warps,
  // which hold a whole 32 x 256 accumulator share packed to 16 bits while the buffer is handed back.
  // The registers are re-divided inside what the CTA was launched with (384 threads x 168): a split
  // that asks for more never gets it and the warps asking would wait for ever.
  static constexpr int kEpiWarp0 = MT == 2 ? 4 : 2;
  static constexpr int kThreads = 32 * (kEpiWarp0 + kEpiWarps);
  static constexpr int kRoleRegs = 56;
  static constexpr int kEpiRegs = 224;
  static_assert(MT == 1 || 128 * kRoleRegs + 256 * kEpiRegs <= 384 * 168,
                "register split exceeds the CTA's launch allocation");
  static constexpr int kSlabsPerWarp = 2 / MT;                // TMA-store staging slabs per warp
  static constexpr int kEpiBytes = kEpiWarps * kSlabsPerWarp * kEpiSlabBytes;  // 32 KB
  // TMEM columns of one accumulator buffer (a 224-column tile gets 256: buffers start on 64-column steps)
  static constexpr int kAccCols = MT * (BN < 64 ? BN : (BN + 63) / 64 * 64);
  static constexpr int kAccStages = (2 * kAccCols <= 512) ? 2 : 1;
  // One accumulator buffer of two sub-tiles: each sub-tile gets its own full/empty barrier pair, so
  // sub-tile 0 is read out while the tile's last MMAs still run on sub-tile 1, and the next tile's
  // first MMAs start on sub-tile 0 while sub-tile 1 is read out.
  static constexpr bool kSplitAcc = (kAccStages == 1 && MT == 2);
  static constexpr int kTmemCols = (kAccStages * kAccCols <= 32)    ? 32
                                   : (kAccStages * kAccCols <= 64)  ? 64
                                   : (kAccStages * kAccCols <= 128) ? 128
                                   : (kAccStages * kAccCols <= 256) ? 256
                                                                    : 512;
  static_assert(kAccStages * kAccCols <= 512, "accumulators exceed tensor memory");
  static constexpr uint32_t kIdescBf16 = make_instr_desc(kUmmaM, BN, InFormat::BF16);
  static constexpr uint32_t kIdescF16 = make_instr_desc(kUmmaM, BN, InFormat::F16);
  static constexpr int smem_bytes(int stages) {
    return 1024 + stages * kStageBytes + kEpiBytes + kBarrierBytes;  // full-height A tile
  }
  static constexpr int max_stages() {
    int s = (232448 - 1024 - kEpiBytes - kBarrierBytes) / kStageBytes;
    return s > kMaxStages ? kMaxStages : s;
  }
};

__device__ __forceinline__ void report_timeout(const GemmArgs& args, unsigned int code, int tile,
                                               int detail, volatile uint32_t* abort_flag) {
  if (atomicCAS(args.status, 0u, code) == 0u) {
    args.status[1] = blockIdx.x;
    args.status[2] = static_cast<unsigned int>(tile);
    args.status[3] = static_cast<unsigned int>(detail);
  }
  *abort_flag = 1u;
}

// Failure-detection self-test: waits, with a short cycle budget, on an mbarrier that nothing
// ever arrives on, and reports the give-up through the same status word the GEMM roles use.
// The kernel returns normally; the context stays usable.
__global__ void bounded_wait_selftest_kernel(unsigned int* status, long long budget_cycles) {
  __shared__ __align__(8) unsigned long long bar;
  if (threadIdx.x == 0) {
    const uint32_t b = ptx::smem_u32(&bar);
    ptx::mbar_init(b, 1);
    ptx::fence_mbar_init();
    if (!ptx::mbar_wait(b, 0, budget_cycles)) {
      if (atomicCAS(status, 0u, static_cast<unsigned int>(kStatusSelfTestTimeout)) == 0u) {
        status[1] = blockIdx.x;
        status[2] = 0u;
        status[3] = 0u;
      }
    }
  }
}

// Layout of an fp32 partial tile (split-K / stream-K slot) of block_m x BN elements. The tile is
// stored as the epilogue warps hold it: a fragment is the 32 rows x 64 columns one warp reads from
// tensor memory in one step; inside a fragment the order is [16-byte piece (16)][row (32)][4 floats].
// Returns the offset, in floats, of the fragment that holds `row_in_tile` and 64-column chunk `c`
// (the row's own position inside the fragment, (row % 32) * 4, and the piece index are added by
// the caller). Host-compilable so the fix-up kernel and the tests share it.
template <int BN>
__host__ __device__ __forceinline__ int partial_fragment_offset(int row_in_tile, int c) {
  return ((row_in_tile >> 5) * (BN / kEpiChunkCols) + c) * (32 * kEpiChunkCols);
}
__host__ __device__ __forceinline__ long long partial_element_offset(int block_n, int row, int col) {
  const int frag = (row >> 5) * (block_n / kEpiChunkCols) + (col / kEpiChunkCols);
  const int piece = (col % kEpiChunkCols) / 4;
  return static_cast<long long>(frag) * (32 * kEpiChunkCols) + piece * 128 + (row & 31) * 4 + (col & 3);
}

// Two fp32 values -> one 32-bit word of two 16-bit outputs (lo in the low half), round to nearest
// even; F16 selects IEEE half instead of bfloat16. The type is a compile-time choice: the epilogue
// shares issue slots with the MMA issuer, and a run-time selection (two predicated conversions per
// word) slowed the double-buffered main loop by 4 % (measured).
template <int F16>
__device__ __forceinline__ uint32_t pack16(float lo, float hi) {
  uint32_t r;
  if constexpr (F16) {
    asm("cvt.rn.f16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(lo), "f"(hi));
  } else {
    asm("cvt.rn.bf16x2.f32 %0, %2, %1;" : "=r"(r) : "f"(lo), "f"(hi));
  }
  return r;
}

// Tensor maps the epilogue stores C through: one for an ordinary GEMM; one per destination when
// the kernel also performs the all-gather of a row-sharded C (every rank's copy of the full C,
// this rank's own included, reached through peer-mapped device memory over NVLink).
static constexpr int kMaxGatherPeers = 8;
// Fused all-gather: every destination's store is a bulk group of its own, and the warp waits for
// it to complete before it issues the next one. A store into a peer's memory completes when the
// link has taken it, so a CTA never has more than one 4 KB block per epilogue warp in flight.
// Without the limit the stores pile up behind the link inside the SM's path to memory and the
// operand loads of the next tile queue behind them (measured with the cycle counters: at eight
// ranks the MMA issuer waits for operands for 30 % of the kernel, against 4 % without peers).
// Two GPUs carrying eight ranks' traffic: 1.507 -> 1.453 ms (128 rows per CTA), 1.515 -> 1.491 ms
// (256); four ranks' traffic 0.923 -> 0.885 ms. Allowing one more group in flight gives it all back.
B200_DEVICE void gather_store_issued() {
  ptx::tma_store_commit();
  ptx::tma_store_wait<0>();
}

// Before a warp refills a staging slab: the stores that read it last must have read it. With one
// bulk group per block that is "all but the newest kSlabs - 1 groups"; with one group per
// destination (NP > 1) the groups of one block are counted out by waiting for all of them.
template <int NP, int kSlabs>
B200_DEVICE void slab_reuse_wait() {
  if constexpr (NP > 1) {
    ptx::tma_store_wait_read<0>();
  } else {
    ptx::tma_store_wait_read<kSlabs - 1>();
  }
}

template <int NP>
struct StoreMaps {
  CUtensorMap m[NP];
};

template <int BN, int PAIR, int MT, int PROF, int F16, int NP>
__global__ void __launch_bounds__((KernelTraits<BN, PAIR, MT>::kThreads), 1)
gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
            const __grid_constant__ StoreMaps<NP> maps_c, const __grid_constant__ GemmArgs args) {
  using T = KernelTraits<BN, PAIR, MT>;
  constexpr int G = T::kCtaGroup;
  constexpr int kAccStages = T::kAccStages;
  extern __shared__ uint8_t smem_raw[];

  const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x) / 32, 0);
  const uint32_t lane = ptx::lane_id();
  const uint32_t cta_rank = PAIR ? ptx::cluster_ctarank() : 0u;
  const int worker = PAIR ? static_cast<int>(ptx::cluster_id_x()) : static_cast<int>(blockIdx.x);

  // Tracing is a compile-time variant: even a never-taken branch around the cycle-counter reads
  // in the wait loops slows the main loop measurably.
  constexpr bool prof = PROF != 0;
  const long long t_kernel = prof ? clock64() : 0;
  long long* prof_out = prof ? args.profile + static_cast<long long>(blockIdx.x) * kProfileSlots : nullptr;
  const int stages = args.stages;
  // A stage holds a_rows x 64 of A followed by the B tile. With fewer than 128 rows of A staged
  // (M < 128) the MMA still reads 128 rows: the extra rows are whatever follows in shared
  // memory, they only feed accumulator rows >= M, which are never written out.
  const uint32_t stage_bytes = static_cast<uint32_t>(args.a_stage_bytes) + T::kBBytes;
  const uint32_t smem_base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t epi_base = smem_base + static_cast<uint32_t>(stages) * stage_bytes;
  const uint32_t bar_base = epi_base + static_cast<uint32_t>(args.epi_bytes);
  auto a_addr = [&](int s) { return smem_base + static_cast<uint32_t>(s) * stage_bytes; };
  auto b_addr = [&](int s) { return a_addr(s) + static_cast<uint32_t>(args.a_stage_bytes); };
  auto full_bar = [&](int s) { return bar_base + 8u * static_cast<uint32_t>(s); };
  auto empty_bar = [&](int s) { return bar_base + 8u * static_cast<uint32_t>(kMaxStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * static_cast<uint32_t>(2 * kMaxStages + a); };
  auto tmem_empty_bar = [&](int a) {
    return bar_base + 8u * static_cast<uint32_t>(2 * kMaxStages + 2 + a);
  };
  const uint32_t tmem_ptr_addr = bar_base + 8u * (2 * kMaxStages + 4);
  uint8_t* generic_bar = smem_raw + (bar_base - ptx::smem_u32(smem_raw));
  volatile uint32_t* tmem_ptr_slot =
      reinterpret_cast<volatile uint32_t*>(generic_bar + 8 * (2 * kMaxStages + 4));
  volatile uint32_t* abort_flag = tmem_ptr_slot + 1;

  // ---------------------------------------------------------------- set-up
  ptx::grid_launch_dependents();  // the next kernel in the stream may begin its own set-up
  if (warp == 0 && lane == 0) {
    ptx::prefetch_tensormap(&map_a);
    ptx::prefetch_tensormap(&map_b);
    for (int p = 0; p < (NP > 1 ? args.gather_world : 1); ++p) ptx::prefetch_tensormap(&maps_c.m[p]);
    for (int s = 0; s < stages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < (T::kSplitAcc ? 2 : kAccStages); ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      ptx::mbar_init(tmem_empty_bar(a), (T::kSplitAcc ? 4 : T::kEpiWarps) * G);
    }
    *abort_flag = 0u;
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc<G>(tmem_ptr_addr, T::kTmemCols);
    ptx::tmem_relinquish<G>();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (PAIR) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr_slot;
  // Programmatic dependent launch: everything above (barriers, tensor memory, descriptor prefetch)
  // may overlap the tail of the previous kernel in the stream; nothing below may, because it reads
  // or writes global memory that kernel may still be using (operands, C, partial tiles, flags).
  ptx::grid_dependency_wait();

  // ---------------------------------------------------------------- roles
  if (warp < T::kEpiWarp0) {
  if constexpr (MT == 2) ptx::setmaxnreg_dec<T::kRoleRegs>();
  if (warp == 0) {
    // ===== TMA producer =====
    if (lane == 0) {
      const uint32_t full_base_leader = PAIR ? ptx::map_to_cta(full_bar(0), 0) : full_bar(0);
      WorkIter it(args.sched, worker);
      Segment seg;
      int stage = 0;
      uint32_t phase = 0;
      // running addresses of the current stage (kept by addition: the ring is latency-critical)
      uint32_t a_cur = smem_base, full_cur = full_bar(0), empty_cur = empty_bar(0);
      uint32_t full_leader_cur = full_base_leader;
      const uint32_t b_off = static_cast<uint32_t>(args.a_stage_bytes);
      bool ok = true;
      long long waited = 0;
      while (ok && it.next(seg)) {
        const TileCoord tc = tile_coord(args.sched, seg.tile);
        const int row_a = tc.m * T::kBlockM + static_cast<int>(cta_rank) * T::kCtaM;
        const int row_b = tc.n * BN + static_cast<int>(cta_rank) * T::kBRowsCta;
        for (int kt = seg.k_begin; kt < seg.k_end; ++kt) {
          const long long tw = prof ? clock64() : 0;
          if (!ptx::mbar_wait(empty_cur, phase ^ 1u)) {
            report_timeout(args, kStatusProducerTimeout, seg.tile, kt, abort_flag);
            ok = false;
            break;
          }
          if (prof) waited += clock64() - tw;
          if (cta_rank == 0) ptx::mbar_arrive_expect_tx(full_cur, stage_bytes * G);
          if (PAIR) {
            ptx::tma_load_3d_pair(a_cur, &map_a, full_leader_cur, kt * kBlockK, row_a, tc.b);
            ptx::tma_load_3d_pair(a_cur + b_off, &map_b, full_leader_cur, kt * kBlockK, row_b, tc.b);
          } else {
            ptx::tma_load_3d(a_cur, &map_a, full_cur, kt * kBlockK, row_a, tc.b);
            ptx::tma_load_3d(a_cur + b_off, &map_b, full_cur, kt * kBlockK, row_b, tc.b);
          }
          a_cur += stage_bytes;
          full_cur += 8u;
          empty_cur += 8u;
          full_leader_cur += 8u;
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
            a_cur = smem_base;
            full_cur = full_bar(0);
            empty_cur = empty_bar(0);
            full_leader_cur = full_base_leader;
          }
        }
      }
      if (prof) prof_out[kProfProducerWait] = waited;
    }
    __syncwarp();
  } else if (warp == 1) {
    // ===== MMA issuer (leader CTA only) =====
    if (lane == 0 && cta_rank == 0) {
      WorkIter it(args.sched, worker);
      Segment seg;
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      uint32_t full_cur = full_bar(0), empty_cur = empty_bar(0);
      constexpr uint32_t idesc = F16 ? T::kIdescF16 : T::kIdescBf16;
      // operand descriptors of the current stage, advanced by addition
      const uint64_t desc_stage_step = static_cast<uint64_t>(stage_bytes >> 4);
      const uint64_t desc_a0 = make_smem_desc_sw128(smem_base);
      const uint64_t desc_b0 = make_smem_desc_sw128(smem_base + static_cast<uint32_t>(args.a_stage_bytes));
      uint64_t desc_a_cur = desc_a0, desc_b_cur = desc_b0;
      bool ok = true;
      long long wait_full = 0, wait_tmem = 0;
      while (ok && it.next(seg)) {
        if constexpr (!T::kSplitAcc) {
          const long long tw0 = prof ? clock64() : 0;
          if (!ptx::mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1u)) {
            report_timeout(args, kStatusMmaTmemTimeout, seg.tile, acc, abort_flag);
            break;
          }
          if (prof) wait_tmem += clock64() - tw0;
          ptx::tc_fence_after_sync();
        }
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * T::kAccCols);
        for (int kt = seg.k_begin; kt < seg.k_end; ++kt) {
          const long long tw1 = prof ? clock64() : 0;
          if (!ptx::mbar_wait(full_cur, phase)) {
            report_timeout(args, kStatusMmaFullTimeout, seg.tile, kt, abort_flag);
            ok = false;
            break;
          }
          if (prof) wait_full += clock64() - tw1;
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            // sub-tile mt: rows [128*mt, 128*mt + 128) of this CTA's A tile -> columns [BN*mt, ...)
            const uint64_t desc_a = desc_a_cur + static_cast<uint64_t>(mt * ((kCtaRows * kBlockK * 2) >> 4));
            if constexpr (T::kSplitAcc) {
              if (kt == seg.k_begin) {  // the first MMA overwrites the sub-tile: it must have been read out
                const long long tw0 = prof ? clock64() : 0;
                if (!ptx::mbar_wait(tmem_empty_bar(mt), acc_phase ^ 1u)) {
                  report_timeout(args, kStatusMmaTmemTimeout, seg.tile, mt, abort_flag);
                  ok = false;
                  break;
                }
                if (prof) wait_tmem += clock64() - tw0;
                ptx::tc_fence_after_sync();
              }
            }
#pragma unroll
            for (int k = 0; k < kBlockK / kUmmaK; ++k) {
              ptx::umma_f16<G>(tmem_d + mt * BN, desc_a + k * kDescKStep, desc_b_cur + k * kDescKStep,
                               idesc, (kt > seg.k_begin || k > 0) ? 1u : 0u);
            }
            if constexpr (T::kSplitAcc) {
              if (kt == seg.k_end - 1) {  // this sub-tile is complete once the MMAs issued so far are
                if (PAIR) {
                  ptx::umma_commit_pair(tmem_full_bar(mt), 3);
                } else {
                  ptx::umma_commit_1cta(tmem_full_bar(mt));
                }
              }
            }
          }
          if (!ok) break;
          if (PAIR) {
            ptx::umma_commit_pair(empty_cur, 3);
          } else {
            ptx::umma_commit_1cta(empty_cur);
          }
          desc_a_cur += desc_stage_step;
          desc_b_cur += desc_stage_step;
          full_cur += 8u;
          empty_cur += 8u;
          if (++stage == stages) {
            stage = 0;
            phase ^= 1u;
            desc_a_cur = desc_a0;
            desc_b_cur = desc_b0;
            full_cur = full_bar(0);
            empty_cur = empty_bar(0);
          }
        }
        if (!ok) break;
        if constexpr (!T::kSplitAcc) {
          if (PAIR) {
            ptx::umma_commit_pair(tmem_full_bar(acc), 3);
          } else {
            ptx::umma_commit_1cta(tmem_full_bar(acc));
          }
        }
        if (++acc == kAccStages) {
          acc = 0;
          acc_phase ^= 1u;
        }
      }
      if (prof) {
        prof_out[kProfMmaWaitFull] = wait_full;
        prof_out[kProfMmaWaitTmem] = wait_tmem;
      }
    }
    __syncwarp();
  }
  } else {
    // ===== epilogue warps =====
    if constexpr (MT == 2) ptx::setmaxnreg_inc<T::kEpiRegs>();
    // Epilogue warp e reads TMEM lane quadrant q = warp % 4 of sub-tile e / 4: rows q*32..q*32+31
    // of that 128-row sub-tile, 64 columns at a time. The accumulator buffer is handed back to the
    // MMA issuer right after the warp's last TMEM read; conversion and stores of that last chunk
    // happen after the hand-back.
    // (a 224-column tile ends in half a chunk: its last 32 columns are stored straight from registers)
    constexpr int kChunksPerSub = (BN + kEpiChunkCols - 1) / kEpiChunkCols;
    constexpr bool kHalfTail = BN >= kEpiChunkCols && BN % kEpiChunkCols != 0;
    const int e = warp - T::kEpiWarp0;
    const int q = warp & 3;
    const int mt = e >> 2;
    // TMA mode: kSlabsPerWarp staging slabs per warp; staged-store mode: one transpose slab per warp
    const uint32_t slab0 =
        epi_base + static_cast<uint32_t>(e) * (args.store_mode == kStoreTma ? T::kSlabsPerWarp * kEpiSlabBytes
                                                                             : kEpiSlabBytes);
    const uint32_t tmem_empty_leader =
        PAIR ? ptx::map_to_cta(tmem_empty_bar(0), 0) : tmem_empty_bar(0);
    // stream-K flag word of this warp inside a slot's 16: (CTA rank, epilogue warp)
    const int flag_lane = static_cast<int>(cta_rank) * 8 + e;
    WorkIter it(args.sched, worker);
    Segment seg;
    int acc = 0;
    uint32_t acc_phase = 0;
    uint32_t store_count = 0;
    const bool prof_epi = prof && warp == T::kEpiWarp0 && lane == 0;
    long long epi_wait = 0, epi_drain = 0, epi_busy = 0, epi_tiles = 0;
    while (it.next(seg)) {
      const long long te0 = prof_epi ? clock64() : 0;
      // Everything that does not need the accumulator is worked out before the wait for it: the
      // divisions of tile_coord alone are several hundred cycles, and with a single accumulator
      // buffer every cycle between "accumulator ready" and "buffer handed back" idles the tensor cores.
      const TileCoord tc = tile_coord(args.sched, seg.tile);
      const int cta_row0 = static_cast<int>(cta_rank) * T::kCtaM;  // this CTA's first row in the tile
      const int n_tile = tc.n * BN;
      const bool to_slot = seg.slot >= 0;
      const bool plain = !to_slot && !seg.finish;
      // Stream-K finisher: wait for the other workers' partial tiles. They were written long ago
      // (a contributor's partial is the first thing it computes), so for tiles of up to 128 columns
      // this thread's share of their sum is fetched into registers NOW, while the tensor cores are
      // still busy with this tile's K range: what remains after the accumulator is ready — the tail
      // of the whole kernel for a decode shape — is one tensor-memory read, one add, the stores.
      int contrib_first = 0, contrib_count = 0;
      if (seg.finish) {
        contrib_count = streamk_contributors(args.sched, worker, seg.tile, &contrib_first);
        bool ok = true;
        for (int j = 0; j < contrib_count && ok; ++j) {
          const unsigned long long* flag =
              args.flags + static_cast<long long>(contrib_first + j) * 16 + flag_lane;
          const long long t0 = clock64();
          while (ptx::ld_acquire_u64(flag) != args.epoch) {
            if (clock64() - t0 > ptx::kWaitBudgetCycles) {
              ok = false;
              break;
            }
            __nanosleep(64);
          }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok && lane == 0) {
          report_timeout(args, kStatusStreamKTimeout, seg.tile, contrib_first, abort_flag);
        }
      }
      constexpr bool kPrefetchPartials = (BN < kEpiChunkCols) || (BN <= 64 && MT == 1);
      float pre[kPrefetchPartials ? BN : 1];
      if constexpr (kPrefetchPartials) {
        const int row_in_tile = cta_row0 + mt * kCtaRows + q * 32 + static_cast<int>(lane);
        if (contrib_count > 0 && tc.m * T::kBlockM + row_in_tile < args.M) {
          for (int w = 0; w < contrib_count; ++w) {
            const float* slot = args.partial + static_cast<long long>(contrib_first + w) * (T::kBlockM * BN);
            if constexpr (BN < kEpiChunkCols) {
              const float* src = slot + row_in_tile * 4;
#pragma unroll
              for (int j = 0; j < BN; j += 4) {
                const float4 f = __ldcg(reinterpret_cast<const float4*>(src + (j / 4) * (T::kBlockM * 4)));
                pre[j + 0] = w == 0 ? f.x : __fadd_rn(pre[j + 0], f.x);
                pre[j + 1] = w == 0 ? f.y : __fadd_rn(pre[j + 1], f.y);
                pre[j + 2] = w == 0 ? f.z : __fadd_rn(pre[j + 2], f.z);
                pre[j + 3] = w == 0 ? f.w : __fadd_rn(pre[j + 3], f.w);
              }
            } else {
#pragma unroll
              for (int c = 0; c < BN / kEpiChunkCols; ++c) {
                const float* src = slot + partial_fragment_offset<BN>(row_in_tile, c) + lane * 4;
#pragma unroll
                for (int k = 0; k < kEpiChunkCols; k += 4) {
                  const float4 f = __ldcg(reinterpret_cast<const float4*>(src + (k / 4) * 128));
                  float* d = &pre[c * kEpiChunkCols + k];
                  d[0] = w == 0 ? f.x : __fadd_rn(d[0], f.x);
                  d[1] = w == 0 ? f.y : __fadd_rn(d[1], f.y);
                  d[2] = w == 0 ? f.z : __fadd_rn(d[2], f.z);
                  d[3] = w == 0 ? f.w : __fadd_rn(d[3], f.w);
                }
              }
            }
          }
        }
      }
      const int acc_bar = T::kSplitAcc ? mt : acc;  // barrier pair of this warp's accumulator (sub-)buffer
      if (!ptx::mbar_wait(tmem_full_bar(acc_bar), acc_phase)) {
        if (lane == 0) report_timeout(args, kStatusEpilogueTimeout, seg.tile, acc_bar, abort_flag);
        break;
      }
      ptx::tc_fence_after_sync();
      const long long te1 = prof_epi ? clock64() : 0;
      if (prof_epi) epi_wait += te1 - te0;

      if constexpr (BN < kEpiChunkCols) {
        // Narrow tile (16 or 32 columns): one tensor-memory read is the warp's whole share, so the
        // accumulator buffer goes back to the MMA issuer before anything is stored.
        const int tile_row = cta_row0 + mt * kCtaRows + q * 32;  // this warp's first row in the tile
        const int m_slab = tc.m * T::kBlockM + tile_row;
        const int row_in_tile = tile_row + static_cast<int>(lane);
        const int row = m_slab + static_cast<int>(lane);
        const bool row_live = row < args.M;
        const bool live = m_slab < args.M;                  // warp-uniform
        uint32_t v[BN];
        if (live) {
          ptx::tmem_ld_cols(tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                static_cast<uint32_t>(acc * T::kAccCols + mt * BN),
                            v);
          ptx::tmem_ld_wait();
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive_cluster(tmem_empty_leader + 8u * static_cast<uint32_t>(acc_bar));
        if (prof_epi) epi_drain += clock64() - te1;
        // fp32 partial tile of a narrow kernel: [4-column piece][row of the tile][4 floats], so the
        // 32 lanes of a warp write 512 contiguous bytes per store instruction.
        constexpr int kPieceStride = T::kBlockM * 4;
        if (live && row_live) {
          if (to_slot) {
            float* dst = args.partial + static_cast<long long>(seg.slot) * (T::kBlockM * BN) + row_in_tile * 4;
#pragma unroll
            for (int j = 0; j < BN; j += 4) {
              __stcg(reinterpret_cast<float4*>(dst + (j / 4) * kPieceStride),
                     make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                 __uint_as_float(v[j + 3])));
            }
          } else {
            if (contrib_count > 0) {  // (narrow tiles always have their contributors' sum in `pre`)
#pragma unroll
              for (int j = 0; j < BN; ++j) v[j] = __float_as_uint(__fadd_rn(__uint_as_float(v[j]), pre[j]));
            }
            if (args.scale) {
#pragma unroll
              for (int j = 0; j < BN; ++j) {
                v[j] = __float_as_uint(__fadd_rn(__fmul_rn(__uint_as_float(v[j]), args.alpha), args.beta));
              }
            }
            uint16_t* cbase = reinterpret_cast<uint16_t*>(args.C) + tc.b * args.c_batch_stride;
            if (args.c_transposed) {
              // column j of the product is a row of the caller's C: the warp's lanes write 32
              // consecutive 16-bit elements of it
#pragma unroll
              for (int j = 0; j < BN; ++j) {
                if (n_tile + j < args.N) {
                  cbase[static_cast<long long>(n_tile + j) * args.ldc + row] =
                      static_cast<uint16_t>(pack16<F16>(__uint_as_float(v[j]), 0.0f) & 0xFFFFu);
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < BN; ++j) {
                if (n_tile + j < args.N) {
                  cbase[static_cast<long long>(row) * args.ldc + n_tile + j] =
                      static_cast<uint16_t>(pack16<F16>(__uint_as_float(v[j]), 0.0f) & 0xFFFFu);
                }
              }
            }
          }
        }
      } else {
      bool drained = false;
      if constexpr (kAccStages == 1) {
        // One accumulator buffer (the two sub-tiles fill tensor memory): the tensor cores idle until
        // this buffer is handed back. So the warp first reads ALL of its share out — the first 64
        // columns go straight into its staging slab, the rest is kept in registers packed to 16 bits —
        // hands the buffer back, and only then issues the stores: the stores of tile i run under the
        // main loop of tile i + 1. (Everything in registers would need more than the 168 a thread of
        // a 320-thread CTA can have.)
        if (plain && args.store_mode == kStoreTma) {
          const int tile_row = cta_row0 + mt * kCtaRows + q * 32;
          const int m_slab = tc.m * T::kBlockM + tile_row;
          const bool rows_live = m_slab < args.M;  // warp-uniform
          const uint32_t slab_first = slab0 + (store_count & (T::kSlabsPerWarp - 1)) * kEpiSlabBytes;
          uint32_t packed[kChunksPerSub - 1][32];
          if (rows_live) {
            const uint32_t taddr0 = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                                    static_cast<uint32_t>(acc * T::kAccCols + mt * BN);
            if (lane == 0) slab_reuse_wait<NP, T::kSlabsPerWarp>();  // the slab's last store has read it
            __syncwarp();
            // 32 columns per read, two register buffers: the read of piece i + 1 is in flight while
            // piece i is converted. (Columns beyond N hold products of zero-filled rows of B: they
            // are read like the others and never stored.)
            constexpr int kPieces = 2 * kChunksPerSub;
            uint32_t v[2][32];
            ptx::tmem_ld_32x32b_x32(taddr0, v[0]);
#pragma unroll
            for (int i = 0; i < kPieces; ++i) {
              const int c = i >> 1, h = i & 1;
              ptx::tmem_ld_wait();
              if (i + 1 < kPieces) ptx::tmem_ld_32x32b_x32(taddr0 + static_cast<uint32_t>((i + 1) * 32), v[(i + 1) & 1]);
              uint32_t(&x)[32] = v[i & 1];
              if (args.scale) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  x[j] = __float_as_uint(__fadd_rn(__fmul_rn(__uint_as_float(x[j]), args.alpha), args.beta));
                }
              }
              if (c == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  ptx::st_shared_v4(slab_first + sw128_offset(lane, static_cast<uint32_t>(h * 4 + j)),
                                    pack16<F16>(__uint_as_float(x[8 * j + 0]), __uint_as_float(x[8 * j + 1])),
                                    pack16<F16>(__uint_as_float(x[8 * j + 2]), __uint_as_float(x[8 * j + 3])),
                                    pack16<F16>(__uint_as_float(x[8 * j + 4]), __uint_as_float(x[8 * j + 5])),
                                    pack16<F16>(__uint_as_float(x[8 * j + 6]), __uint_as_float(x[8 * j + 7])));
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  packed[c - 1 < 0 ? 0 : c - 1][h * 16 + j] =
                      pack16<F16>(__uint_as_float(x[2 * j]), __uint_as_float(x[2 * j + 1]));
                }
              }
            }
          }
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) ptx::mbar_arrive_cluster(tmem_empty_leader + 8u * static_cast<uint32_t>(acc_bar));
          if (prof_epi) epi_drain += clock64() - te1;
          if (rows_live) {
#pragma unroll
            for (int c = 0; c < kChunksPerSub; ++c) {
              const int n0 = n_tile + c * kEpiChunkCols;
              if (n0 < args.N) {
                const uint32_t slab = slab0 + (store_count & (T::kSlabsPerWarp - 1)) * kEpiSlabBytes;
                if (c > 0) {
                  if (lane == 0) slab_reuse_wait<NP, T::kSlabsPerWarp>();
                  __syncwarp();
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      const uint32_t* w = &packed[c - 1 < 0 ? 0 : c - 1][h * 16 + 4 * j];
                      ptx::st_shared_v4(slab + sw128_offset(lane, static_cast<uint32_t>(h * 4 + j)), w[0], w[1], w[2],
                                        w[3]);
                    }
                  }
                }
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                  if constexpr (NP > 1) {
                    for (int p = 0; p < args.gather_world; ++p) {
                      ptx::tma_store_3d(&maps_c.m[p], slab, n0, m_slab, tc.b);
                      gather_store_issued();
                    }
                  } else {
                    ptx::tma_store_3d(&maps_c.m[0], slab, n0, m_slab, tc.b);
                    ptx::tma_store_commit();
                  }
                }
                ++store_count;
              }
            }
          }
          drained = true;
        }
      }
      if (!drained) {
#pragma unroll 1
      for (int c = 0; c < kChunksPerSub; ++c) {  // 64-column chunks of this warp's sub-tile
        const int tile_row = cta_row0 + mt * kCtaRows + q * 32;  // this warp's first row in the tile
        const int m_slab = tc.m * T::kBlockM + tile_row;
        const int row_in_tile = tile_row + static_cast<int>(lane);
        const bool row_live = (tc.m * T::kBlockM + row_in_tile) < args.M;
        const int n0 = n_tile + c * kEpiChunkCols;
        // warp-uniform: does this chunk hold anything that is written out?
        const bool live = (m_slab < args.M) && (to_slot || n0 < args.N);
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                               static_cast<uint32_t>(acc * T::kAccCols + mt * BN + c * kEpiChunkCols);
        uint32_t v[2][32];
        if (live) {
          ptx::tmem_ld_32x32b_x32(taddr, v[0]);
          ptx::tmem_ld_32x32b_x32(taddr + 32, v[1]);
          ptx::tmem_ld_wait();
        }
        if (c == kChunksPerSub - 1) {
          // This warp has read all it needs from the accumulator buffer: hand it back.
          ptx::tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) {
            ptx::mbar_arrive_cluster(tmem_empty_leader + 8u * static_cast<uint32_t>(acc_bar));
          }
          if (prof_epi) epi_drain += clock64() - te1;
        }
        if (!live) continue;

        if (!plain) {
          if (to_slot) {
            // fp32 partial tile in FRAGMENT order (see partial_fragment_offset): the 32 lanes of a
            // warp write consecutive 16-byte pieces, so every store instruction fills four whole
            // 128-byte lines. Rows >= M are never read back and are not written.
            if (row_live) {
              float* dst = args.partial + static_cast<long long>(seg.slot) * (T::kBlockM * BN) +
                           partial_fragment_offset<BN>(row_in_tile, c) + lane * 4;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                  float4 f = make_float4(__uint_as_float(v[h][j]), __uint_as_float(v[h][j + 1]),
                                         __uint_as_float(v[h][j + 2]), __uint_as_float(v[h][j + 3]));
                  __stcg(reinterpret_cast<float4*>(dst + (h * 8 + j / 4) * 128), f);
                }
              }
            }
            continue;
          }
          if constexpr (kPrefetchPartials) {
            if (row_live && contrib_count > 0) {
#pragma unroll
              for (int cc = 0; cc < kChunksPerSub; ++cc) {  // (static register indexing: c is a run-time value)
                if (cc == c) {
#pragma unroll
                  for (int h = 0; h < 2; ++h) {
#pragma unroll
                    for (int k = 0; k < 32; ++k) {
                      v[h][k] = __float_as_uint(
                          __fadd_rn(__uint_as_float(v[h][k]), pre[(cc * kEpiChunkCols + h * 32 + k) % (kPrefetchPartials ? BN : 1)]));
                    }
                  }
                }
              }
            }
          } else if (row_live) {
            for (int j = 0; j < contrib_count; ++j) {
              const float* src = args.partial + static_cast<long long>(contrib_first + j) * (T::kBlockM * BN) +
                                 partial_fragment_offset<BN>(row_in_tile, c) + lane * 4;
#pragma unroll
              for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int k = 0; k < 32; k += 4) {
                  const float4 f = __ldcg(reinterpret_cast<const float4*>(src + (h * 8 + k / 4) * 128));
                  v[h][k + 0] = __float_as_uint(__fadd_rn(__uint_as_float(v[h][k + 0]), f.x));
                  v[h][k + 1] = __float_as_uint(__fadd_rn(__uint_as_float(v[h][k + 1]), f.y));
                  v[h][k + 2] = __float_as_uint(__fadd_rn(__uint_as_float(v[h][k + 2]), f.z));
                  v[h][k + 3] = __float_as_uint(__fadd_rn(__uint_as_float(v[h][k + 3]), f.w));
                }
              }
            }
          }
        }

        if (args.scale) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[h][j] = __float_as_uint(
                  __fadd_rn(__fmul_rn(__uint_as_float(v[h][j]), args.alpha), args.beta));
            }
          }
        }

        if constexpr (kHalfTail) {
          if (c == kChunksPerSub - 1) {
            // The tile's last 32 columns (v[0]; v[1] lies beyond the tile): 64 bytes of this lane's row.
            // Whole data-parallel tiles only — the launcher admits no other schedule for this width.
            if (row_live) {
              __nv_bfloat16* dst = args.C + tc.b * args.c_batch_stride +
                                   static_cast<long long>(m_slab + static_cast<int>(lane)) * args.ldc + n0;
              if (args.store_mode != kStoreScalar) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (n0 + 8 * j < args.N) {  // N is a multiple of 8 in these modes
                    uint4 w;
                    w.x = pack16<F16>(__uint_as_float(v[0][8 * j + 0]), __uint_as_float(v[0][8 * j + 1]));
                    w.y = pack16<F16>(__uint_as_float(v[0][8 * j + 2]), __uint_as_float(v[0][8 * j + 3]));
                    w.z = pack16<F16>(__uint_as_float(v[0][8 * j + 4]), __uint_as_float(v[0][8 * j + 5]));
                    w.w = pack16<F16>(__uint_as_float(v[0][8 * j + 6]), __uint_as_float(v[0][8 * j + 7]));
                    *reinterpret_cast<uint4*>(dst + 8 * j) = w;
                  }
                }
              } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (n0 + j < args.N) {
                    reinterpret_cast<uint16_t*>(dst)[j] =
                        static_cast<uint16_t>(pack16<F16>(__uint_as_float(v[0][j]), 0.0f) & 0xFFFFu);
                  }
                }
              }
            }
            continue;
          }
        }

        if (args.store_mode == kStoreStaged) {
          // Each lane holds one row; a row-per-lane store touches 32 lines per instruction. Write
          // the 32 x 64 block to this warp's slab instead and read it back so that 8 lanes cover
          // one row: every global store instruction then writes four complete 128-byte lines.
          const uint32_t slab = slab0;
          __syncwarp();  // the previous chunk's reads of the slab are done
#pragma unroll
          for (int h = 0; h < 2; ++h) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              ptx::st_shared_v4(
                  slab + sw128_offset(lane, static_cast<uint32_t>(h * 4 + j)),
                  pack16<F16>(__uint_as_float(v[h][8 * j + 0]), __uint_as_float(v[h][8 * j + 1])),
                  pack16<F16>(__uint_as_float(v[h][8 * j + 2]), __uint_as_float(v[h][8 * j + 3])),
                  pack16<F16>(__uint_as_float(v[h][8 * j + 4]), __uint_as_float(v[h][8 * j + 5])),
                  pack16<F16>(__uint_as_float(v[h][8 * j + 6]), __uint_as_float(v[h][8 * j + 7])));
            }
          }
          __syncwarp();
          const uint32_t piece = lane & 7u;  // 16-byte piece of a row
          const int col = n0 + static_cast<int>(piece) * 8;
          __nv_bfloat16* base = args.C + tc.b * args.c_batch_stride + col;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t r = (lane >> 3) + 4u * static_cast<uint32_t>(i);
            const uint4 w = ptx::ld_shared_v4(slab + sw128_offset(r, piece));
            const int m = m_slab + static_cast<int>(r);
            if (m < args.M && col < args.N) {
              *reinterpret_cast<uint4*>(base + static_cast<long long>(m) * args.ldc) = w;
            }
          }
          continue;
        }

        if (args.store_mode != kStoreTma) {
          if (row_live) {
            __nv_bfloat16* dst = args.C + tc.b * args.c_batch_stride +
                                 static_cast<long long>(m_slab + static_cast<int>(lane)) * args.ldc + n0;
            if (args.store_mode == kStoreVector && n0 + kEpiChunkCols <= args.N) {
              // 128 contiguous bytes of this lane's row, as eight 16-byte stores
#pragma unroll
              for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  uint4 w;
                  w.x = pack16<F16>(__uint_as_float(v[h][8 * j + 0]), __uint_as_float(v[h][8 * j + 1]));
                  w.y = pack16<F16>(__uint_as_float(v[h][8 * j + 2]), __uint_as_float(v[h][8 * j + 3]));
                  w.z = pack16<F16>(__uint_as_float(v[h][8 * j + 4]), __uint_as_float(v[h][8 * j + 5]));
                  w.w = pack16<F16>(__uint_as_float(v[h][8 * j + 6]), __uint_as_float(v[h][8 * j + 7]));
                  *reinterpret_cast<uint4*>(dst + h * 32 + j * 8) = w;
                }
              }
            } else if (args.c_transposed) {
              // few-rows plan: column j of the product is a row of the caller's C
              uint16_t* cbase = reinterpret_cast<uint16_t*>(args.C) + tc.b * args.c_batch_stride +
                                (m_slab + static_cast<int>(lane));
#pragma unroll
              for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (n0 + h * 32 + j < args.N) {
                    cbase[static_cast<long long>(n0 + h * 32 + j) * args.ldc] =
                        static_cast<uint16_t>(pack16<F16>(__uint_as_float(v[h][j]), 0.0f) & 0xFFFFu);
                  }
                }
              }
            } else {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  if (n0 + h * 32 + j < args.N) {
                    reinterpret_cast<uint16_t*>(dst)[h * 32 + j] =
                        static_cast<uint16_t>(pack16<F16>(__uint_as_float(v[h][j]), 0.0f) & 0xFFFFu);
                  }
                }
              }
            }
          }
          continue;
        }

        // bf16 -> swizzled staging slab -> TMA store of a 32-row x 64-column box.
        const uint32_t slab = slab0 + (store_count & (T::kSlabsPerWarp - 1)) * kEpiSlabBytes;
        if (lane == 0) slab_reuse_wait<NP, T::kSlabsPerWarp>();  // the slab's last store has read it
        __syncwarp();
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t chunk16 = static_cast<uint32_t>(h * 4 + j);
            ptx::st_shared_v4(
                slab + sw128_offset(lane, chunk16),
                pack16<F16>(__uint_as_float(v[h][8 * j + 0]), __uint_as_float(v[h][8 * j + 1])),
                pack16<F16>(__uint_as_float(v[h][8 * j + 2]), __uint_as_float(v[h][8 * j + 3])),
                pack16<F16>(__uint_as_float(v[h][8 * j + 4]), __uint_as_float(v[h][8 * j + 5])),
                pack16<F16>(__uint_as_float(v[h][8 * j + 6]), __uint_as_float(v[h][8 * j + 7])));
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if constexpr (NP > 1) {
            // fused all-gather: the same staged block goes to every rank's copy of C
            for (int p = 0; p < args.gather_world; ++p) {
              ptx::tma_store_3d(&maps_c.m[p], slab, n0, m_slab, tc.b);
              gather_store_issued();
            }
          } else {
            ptx::tma_store_3d(&maps_c.m[0], slab, n0, m_slab, tc.b);
            ptx::tma_store_commit();
          }
        }
        ++store_count;
      }
      }  // chunk by chunk
      }  // wide tiles
      if (prof_epi) {
        epi_busy += clock64() - te1;
        ++epi_tiles;
      }
      if (to_slot && args.sched.mode != kSplitK) {
        // Publish this warp's part of the partial tile: every lane's stores, then the flag.
        __threadfence();
        __syncwarp();
        if (lane == 0) {
          ptx::st_release_u64(args.flags + static_cast<long long>(seg.slot) * 16 + flag_lane, args.epoch);
        }
      }
      if (++acc == kAccStages) {
        acc = 0;
        acc_phase ^= 1u;
      }
    }
    if (lane == 0) ptx::tma_store_wait<0>();
    __syncwarp();
    if (prof_epi) {
      prof_out[kProfEpiWaitFull] = epi_wait;
      prof_out[kProfEpiDrain] = epi_drain;
      prof_out[kProfEpiBusy] = epi_busy;
      prof_out[kProfTiles] = epi_tiles;
    }
  }

  // ---------------------------------------------------------------- teardown
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0u) {
    // A wait gave up: give this CTA's outstanding bulk copies time to land before its shared
    // memory and tensor memory are released.
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  if (PAIR) {
    ptx::cluster_arrive();
    ptx::cluster_wait();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc<G>(tmem_base, T::kTmemCols);
  }
  if (prof && threadIdx.x == 0) prof_out[kProfTotal] = clock64() - t_kernel;
}

}  // namespace b200
