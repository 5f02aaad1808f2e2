// Host launcher and C ABI (include/b200_gemm.h) of the sm_100a GEMM.
//
// Replaces the reference's host launchers gpu_gemm() (matmul_h100.cu.jinja:927-985) and
// runKernel() (matmul_h100_optimal.cu:32-59) and its tensor-map builder make_tma_copy_desc()
// (tma.cuh:83-181). Differences that matter to a caller:
//   * errors are returned, never exit()/assert();
//   * tensor maps and function attributes are cached instead of being rebuilt inside the timed
//     loop (matmul_h100.cu.jinja:938-957);
//   * the grid is sized from the device (SM count, co-resident clusters) instead of the
//     hard-coded NUM_SM = 128 (matmul_h100_optimal.cu:40).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <map>
#include <random>
#include <string>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/b200_gemm.h"
#include "sm100/gemm_kernel.cuh"

namespace {

using namespace b200;

thread_local int g_last_cuda_error = 0;

#define B200_CUDA_TRY(expr)                           \
  do {                                                \
    cudaError_t e__ = (expr);                         \
    if (e__ != cudaSuccess) {                         \
      g_last_cuda_error = static_cast<int>(e__);      \
      (void)cudaGetLastError();                       \
      return B200_ERR_CUDA;                           \
    }                                                 \
  } while (0)

// Device-side status word (one per device that loads this library).
__device__ unsigned int g_device_status[4];

// ------------------------------------------------------------------------------------------
// Auxiliary kernels
// ------------------------------------------------------------------------------------------

// Copies rows of K 16-bit elements to a pitch of Kp elements (Kp % 8 == 0) so that the copy can
// be read through a tensor map. Elements K..Kp-1 are never read (the map's extent stays K).
__global__ void repitch_rows_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst,
                                    long long rows, int K, int Kp) {
  const long long total = rows * K;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long r = i / K;
    const int k = static_cast<int>(i - r * K);
    dst[r * Kp + k] = src[i];
  }
}

// Sums the fp32 partial slots of every split tile in slot order and writes the bf16 result.
__global__ void fixup_kernel(GemmArgs args, int block_m, int block_n) {
  __shared__ int slots[64];
  __shared__ int nslots;
  for (int tile = blockIdx.x; tile < args.sched.num_tiles; tile += gridDim.x) {
    __syncthreads();
    if (threadIdx.x == 0) nslots = tile_partial_slots(args.sched, tile, slots, 64);
    __syncthreads();
    const int n = nslots;
    if (n == 0) continue;
    const TileCoord tc = tile_coord(args.sched, tile);
    const int m0 = tc.m * block_m;
    const int n0 = tc.n * block_n;
    const int rows = min(block_m, args.M - m0);
    const int vec_per_row = block_n / 4;
    const long long slot_elems = static_cast<long long>(block_m) * block_n;
    for (int idx = threadIdx.x; idx < rows * vec_per_row; idx += blockDim.x) {
      const int r = idx / vec_per_row;
      const int c = (idx - r * vec_per_row) * 4;
      if (n0 + c >= args.N) continue;
      // slots are stored in the epilogue's fragment order (partial_element_offset)
      const long long off = partial_element_offset(block_n, r, c);
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int s = 0; s < n; ++s) {
        const float4 p = *reinterpret_cast<const float4*>(args.partial + slots[s] * slot_elems + off);
        acc.x += p.x;
        acc.y += p.y;
        acc.z += p.z;
        acc.w += p.w;
      }
      float v[4] = {acc.x, acc.y, acc.z, acc.w};
      __nv_bfloat16* dst =
          args.C + tc.b * args.c_batch_stride + static_cast<long long>(m0 + r) * args.ldc + n0 + c;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (n0 + c + j < args.N) {
          float x = v[j];
          if (args.scale) x = __fadd_rn(__fmul_rn(x, args.alpha), args.beta);
          if (args.f16) {
            reinterpret_cast<__half*>(dst)[j] = __float2half_rn(x);
          } else {
            dst[j] = __float2bfloat16_rn(x);
          }
        }
      }
    }
  }
}

// Plain SIMT GEMM, the on-device cross-check (semantics of reference.h:49-76: k ascending, fp32
// accumulate, (bf16)(acc * alpha + beta)); one thread per 4x4 outputs.
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float to_float(__half x) { return __half2float(x); }
__device__ __forceinline__ void from_float(__nv_bfloat16* p, float x) { *p = __float2bfloat16_rn(x); }
__device__ __forceinline__ void from_float(__half* p, float x) { *p = __float2half_rn(x); }

template <typename T>
__global__ void naive_gemm_kernel(int M, int N, int K, const T* __restrict__ A, const T* __restrict__ B,
                                  T* __restrict__ C, float alpha, float beta) {
  const int n0 = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  const int m0 = blockIdx.y * 4;
  if (n0 >= N || m0 >= M) return;
  float acc[4][4] = {};
  for (int k = 0; k < K; ++k) {
    float a[4], b[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      a[i] = m0 + i < M ? to_float(A[static_cast<long long>(m0 + i) * K + k]) : 0.f;
      b[i] = n0 + i < N ? to_float(B[static_cast<long long>(n0 + i) * K + k]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = __fmaf_rn(a[i], b[j], acc[i][j]);
  }
  for (int i = 0; i < 4; ++i)
    for (int j = 0; j < 4; ++j)
      if (m0 + i < M && n0 + j < N)
        from_float(&C[static_cast<long long>(m0 + i) * N + n0 + j], __fadd_rn(__fmul_rn(acc[i][j], alpha), beta));
}

// ------------------------------------------------------------------------------------------
// Kernel table
// ------------------------------------------------------------------------------------------
using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const StoreMaps<1>, const GemmArgs);
using GatherFn = void (*)(const CUtensorMap, const CUtensorMap, const StoreMaps<kMaxGatherPeers>, const GemmArgs);

struct KernelEntry {
  int bn;
  int pair;
  int mt;         // 128-row sub-tiles of A per CTA
  KernelFn fn;
  KernelFn fn_traced;  // same kernel with the cycle counters compiled in
  KernelFn fn_f16;     // same kernel for IEEE fp16 operands and output
  GatherFn fn_gather;  // same kernel storing every tile to up to 8 copies of C (256-column pair tiles only)
  GatherFn fn_gather_traced;
  int b_bytes;    // bytes of B staged per CTA and K-tile
  int b_rows_cta;
  int block_m;    // rows of C per worker tile
  int threads;
  int epi_bytes;  // epilogue staging shared memory
};

template <int BN, int PAIR, int MT, int PROF>
GatherFn gather_variant() {
  if constexpr (BN == 256 && PAIR == 1) {
    return &gemm_kernel<BN, PAIR, MT, PROF, 0, kMaxGatherPeers>;
  } else {
    return nullptr;
  }
}

template <int BN, int PAIR, int MT>
KernelEntry make_entry() {
  using T = KernelTraits<BN, PAIR, MT>;
  return KernelEntry{BN,
                     PAIR,
                     MT,
                     &gemm_kernel<BN, PAIR, MT, 0, 0, 1>,
                     &gemm_kernel<BN, PAIR, MT, 1, 0, 1>,
                     &gemm_kernel<BN, PAIR, MT, 0, 1, 1>,
                     gather_variant<BN, PAIR, MT, 0>(),
                     gather_variant<BN, PAIR, MT, 1>(),
                     T::kBBytes,
                     T::kBRowsCta,
                     T::kBlockM,
                     T::kThreads,
                     T::kEpiBytes};
}

const KernelEntry* find_kernel(int bn, int pair, int mt) {
  static const KernelEntry table[] = {
      make_entry<16, 0, 1>(),  make_entry<32, 0, 1>(),
      make_entry<64, 0, 1>(),  make_entry<128, 0, 1>(), make_entry<192, 0, 1>(), make_entry<224, 0, 1>(),
      make_entry<256, 0, 1>(),
      make_entry<64, 1, 1>(),  make_entry<128, 1, 1>(), make_entry<192, 1, 1>(), make_entry<256, 1, 1>(),
      make_entry<128, 0, 2>(), make_entry<256, 0, 2>(), make_entry<128, 1, 2>(), make_entry<256, 1, 2>(),
      // narrow accumulators as CTA pairs and with two sub-tiles: the few-rows plan only
      make_entry<16, 1, 1>(),  make_entry<32, 1, 1>(),
      make_entry<16, 0, 2>(),  make_entry<32, 0, 2>(),  make_entry<64, 0, 2>(),
      make_entry<16, 1, 2>(),  make_entry<32, 1, 2>(),  make_entry<64, 1, 2>(),
  };
  for (const auto& e : table)
    if (e.bn == bn && e.pair == pair && e.mt == mt) return &e;
  return nullptr;
}

// ------------------------------------------------------------------------------------------
// Per-device state
// ------------------------------------------------------------------------------------------
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct DeviceState {
  bool ready = false;
  int sm_count = 0;
  int smem_optin = 0;
  unsigned int* status = nullptr;
  std::map<std::tuple<const void*, int>, int> max_workers;  // (kernel, smem) -> co-resident workers
};

std::mutex g_mutex;
long long* g_profile = nullptr;      // optional device buffer for per-CTA cycle counters
size_t g_profile_bytes = 0;
DeviceState g_devices[64];
EncodeTiledFn g_encode = nullptr;

int get_device_state(DeviceState** out) {
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200_ERR_INVALID_ARG;
  DeviceState& st = g_devices[dev];
  if (!st.ready) {
    B200_CUDA_TRY(cudaDeviceGetAttribute(&st.sm_count, cudaDevAttrMultiProcessorCount, dev));
    B200_CUDA_TRY(cudaDeviceGetAttribute(&st.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    void* p = nullptr;
    B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_device_status));
    st.status = static_cast<unsigned int*>(p);
    B200_CUDA_TRY(cudaMemset(st.status, 0, sizeof(unsigned int) * 4));
    if (g_encode == nullptr) {
      void* fn = nullptr;
      cudaDriverEntryPointQueryResult qres;
      B200_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
      if (fn == nullptr || qres != cudaDriverEntryPointSuccess) {
        g_last_cuda_error = static_cast<int>(cudaErrorNotSupported);
        return B200_ERR_CUDA;
      }
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    st.ready = true;
  }
  *out = &st;
  return B200_OK;
}

// Workers (CTAs, or CTA pairs) that can be resident at once for this kernel and smem size.
int max_resident_workers(DeviceState& st, const KernelEntry& e, int smem, int* out) {
  auto key = std::make_tuple(reinterpret_cast<const void*>(e.fn), smem);
  auto it = st.max_workers.find(key);
  if (it != st.max_workers.end()) {
    *out = it->second;
    return B200_OK;
  }
  // Opt in to the device maximum once, so a later launch with fewer stages cannot shrink it.
  B200_CUDA_TRY(cudaFuncSetAttribute(e.fn, cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
  B200_CUDA_TRY(cudaFuncSetAttribute(e.fn_traced, cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
  B200_CUDA_TRY(cudaFuncSetAttribute(e.fn_f16, cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
  if (e.fn_gather != nullptr) {
    B200_CUDA_TRY(cudaFuncSetAttribute(e.fn_gather, cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
    B200_CUDA_TRY(cudaFuncSetAttribute(e.fn_gather_traced, cudaFuncAttributeMaxDynamicSharedMemorySize, st.smem_optin));
  }
  if (smem > st.smem_optin) return B200_ERR_SMEM;
  int workers = st.sm_count;
  if (e.pair) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(st.sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(static_cast<unsigned>(e.threads), 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int clusters = 0;
    B200_CUDA_TRY(cudaOccupancyMaxActiveClusters(&clusters, e.fn, &cfg));
    workers = clusters;
  }
  if (workers <= 0) return B200_ERR_SMEM;
  st.max_workers[key] = workers;
  *out = workers;
  return B200_OK;
}

// ------------------------------------------------------------------------------------------
// Tensor maps (bf16, rank 3: {inner, rows, batch}), 128-byte swizzle, zero fill out of bounds
// ------------------------------------------------------------------------------------------
struct MapKey {
  const void* base;
  uint64_t inner, rows, batch, pitch_bytes, batch_pitch_bytes;
  uint32_t box_inner, box_rows;
  bool operator<(const MapKey& o) const {
    return std::tie(base, inner, rows, batch, pitch_bytes, batch_pitch_bytes, box_inner, box_rows) <
           std::tie(o.base, o.inner, o.rows, o.batch, o.pitch_bytes, o.batch_pitch_bytes,
                    o.box_inner, o.box_rows);
  }
};
std::map<MapKey, CUtensorMap> g_map_cache;

int make_tensor_map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t rows,
                    uint64_t batch, uint64_t pitch_bytes, uint64_t batch_pitch_bytes,
                    uint32_t box_inner, uint32_t box_rows) {
  MapKey key{base, inner, rows, batch, pitch_bytes, batch_pitch_bytes, box_inner, box_rows};
  auto it = g_map_cache.find(key);
  if (it != g_map_cache.end()) {
    *out = it->second;
    return B200_OK;
  }
  cuuint64_t dims[3] = {inner, rows, batch};
  cuuint64_t strides[2] = {pitch_bytes, batch > 1 ? batch_pitch_bytes : pitch_bytes * rows};
  if (strides[1] % 16 != 0) strides[1] = (strides[1] + 15) / 16 * 16;  // unused when batch == 1
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t elem_strides[3] = {1, 1, 1};
  CUtensorMap m;
  CUresult r = g_encode(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims,
                        strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda_error = static_cast<int>(r);
    return B200_ERR_CUDA;
  }
  if (g_map_cache.size() >= 256) g_map_cache.clear();
  g_map_cache[key] = m;
  *out = m;
  return B200_OK;
}

// ------------------------------------------------------------------------------------------
// Configuration
// ------------------------------------------------------------------------------------------
struct Plan {
  const KernelEntry* kernel;
  int pair;
  int stages;
  int smem;
  int mode;
  int split_k;
  int raster;
  int group;
  int max_ctas;
  int c_col_major;
  int store_mode;  // StoreMode to use when C is 16-byte aligned
  int few_rows;    // 1: the caller's rows ride the MMA's N (operands swapped inside)
};

// Default configuration from the shape. For M > 128 the candidates are ranked by a small cost
// model: waves of tiles over the workers x tile area per SM x a penalty for the L2 -> shared
// memory traffic each tile shape needs per FLOP (larger tiles move fewer bytes, which on a
// power-limited part buys clock; smaller tiles fill the machine when there are few of them).
// Cost model of the data-parallel tile shapes: waves of tiles over the workers x tile area x a
// penalty for the L2 -> shared-memory traffic the shape needs per FLOP (time per unit of tile area
// relative to the best shape, from tuner runs at 8192^3).
struct TileCand {
  int block_m, block_n, cluster_m;
  double penalty;
};
const TileCand kTileCands[] = {
    {256, 256, 2, 1.00}, {256, 256, 1, 1.04}, {128, 256, 2, 1.05}, {256, 128, 1, 1.17},
    {128, 256, 1, 1.27}, {128, 128, 1, 1.58}, {128, 64, 1, 2.13},
};

double tile_cost(int block_m, int block_n, int cluster_m, int batch, int M, int N, int K, int sms) {
  double penalty = 1.2;  // a shape the table above does not list
  for (const TileCand& k : kTileCands) {
    if (k.block_m == block_m && k.block_n == block_n && k.cluster_m == (cluster_m >= 2 ? 2 : 1)) penalty = k.penalty;
  }
  const int pair = cluster_m >= 2 ? 2 : 1;
  const long long tile_m = static_cast<long long>(block_m) * pair;
  const long long tiles = ((M + tile_m - 1) / tile_m) * ((N + block_n - 1) / block_n) * batch;
  const long long workers = sms / pair;
  const long long waves = (tiles + workers - 1) / workers;
  double exposure = 1.0;
  // A 256-row CTA tile has a single accumulator buffer, so the read-out of the accumulator (a
  // fixed number of cycles per tile, about 2 000 of 139 000 at K = 8192) is exposed; the penalties
  // above include it for K = 8192.
  if (block_m == 256 && block_n == 256) exposure = 1.0 + 0.02 * (8192.0 / (K < 512 ? 512 : K) - 1.0);
  return static_cast<double>(waves) * block_m * block_n * penalty * exposure;
}

int heuristic_sm_count() {
  static std::atomic<int> cached[64];  // per device; 0 = not asked yet
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64) {
    v = cached[dev].load(std::memory_order_relaxed);
    if (v > 0) return v;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) {
      cached[dev].store(v, std::memory_order_relaxed);
      return v;
    }
  }
  (void)cudaGetLastError();
  return 148;  // a full B200, when there is no device to ask (sizing a workspace on a build machine)
}

b200_gemm_cfg heuristic_cfg(int batch, int M, int N, int K, int sms = 0) {
  if (sms <= 0) sms = heuristic_sm_count();
  b200_gemm_cfg c;
  std::memset(&c, 0, sizeof(c));
  c.block_m = 128;
  c.block_k = 64;
  c.cluster_n = 1;
  c.group = 8;
  if (M <= 64 && N >= 128) {
    // Very few rows: let them ride the MMA's N dimension (block_m = 16, 32 or 64) and put 128 rows
    // of B on its M dimension. The tensor cores then compute block_m x 128 per tile instead of a
    // 128-row tile that is mostly padding — an eighth of the tensor work at M = 16, which matters
    // because this shape runs into the power cap long before it runs out of HBM bandwidth. The K
    // loop is split evenly over all SMs (stream-K) so that every SM streams the same share of B.
    c.cluster_m = 1;
    c.block_m = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    c.block_n = 128;
    // Up to one wave of tiles, whole tiles win: the kernel is bound by HBM, which 64 SMs already
    // drive at 4.8 TB/s, and finishing split tiles costs about 2 us (measured at N = 8192 and
    // 16384: 28.2 / 46.4 us data-parallel against 29.6 / 48.6 us stream-K). Beyond one wave the
    // even split wins (N = 20480, 160 tiles: 58.2 us against 65.7 us).
    const long long tiles = static_cast<long long>((N + 127) / 128) * batch;
    c.sched = tiles <= sms ? kDataParallel : kStreamK;
    return c;
  }
  if (M <= 128) {
    // Few rows: one CTA per tile, narrower tiles, and an even split of the K loop over all SMs
    // so that every SM streams the same share of B.
    c.cluster_m = 1;
    c.block_n = M <= 32 ? 64 : 128;
    c.sched = kStreamK;
    // Almost nothing is written (M rows): store straight from registers and give the staging
    // memory to the B ring instead (16+ stages in flight; measured best at 28672 x 8192).
    c.epilogue = 2;
    // With nearly 128 real rows and no more 256-column tiles than SMs, one whole 128 x 256 tile per
    // SM wins: no tile is cut, and every 16 KB of A staged serves 32 KB of B instead of 16
    // (128 x 28672 x 8192, 112 tiles: 82.4 us in a burst and 88.7 us sustained against 83.8 / 89.5;
    // at 96 rows it is level in a burst and 1.5 % slower sustained, so the bound is 96).
    // When 224-column tiles are no more than the SMs either, they are taken instead, with stores
    // straight from registers: N = 28672 is then 128 tiles on 128 SMs instead of 112 on 112, and the
    // 44 KB stages fit five deep without staging slabs (220 KB of loads in flight per SM against
    // 192 KB). Measured on two boxes, same process, interleaved: 82.9 against 84.6 us and 78.6
    // against 80.3 us in a burst, 87.5 / 90.2 and 82.2 / 83.7 us sustained.
    // The 224-column tile also wins below 96 rows (80 x 28672 x 8192: 79.4 against 80.9 us stream-K
    // in a burst, 83.7 / 85.5 sustained; 96 rows: 80.1 / 81.7 and 84.9 / 86.4).
    // Whole tiles only while they keep more than half of the SMs busy: a narrow C with a long K is
    // better cut along K.
    const long long tiles224 = static_cast<long long>((N + 223) / 224) * batch;
    const long long tiles256 = static_cast<long long>((N + 255) / 256) * batch;
    if (M > 64 && tiles224 <= sms && 2 * tiles224 > sms) {
      c.block_n = 224;
      c.sched = kDataParallel;
      c.epilogue = 2;
    } else if (M > 96 && tiles256 <= sms && 2 * tiles256 > sms) {
      c.block_n = 256;
      c.sched = kDataParallel;
      c.epilogue = 1;
    }
    return c;
  }
  double best = 0.0;
  for (const TileCand& k : kTileCands) {
    const double cost = tile_cost(k.block_m, k.block_n, k.cluster_m, batch, M, N, K, sms);
    // (The hybrid schedule — full waves data-parallel, last wave stream-K — is available as
    // sched = 3 but is not chosen here: measured on 3072^3..6144^3 it does not beat plain
    // data-parallel tiles, the partial-tile round trip costs about what the shorter wave saves.)
    if (best == 0.0 || cost < best) {
      best = cost;
      c.block_m = k.block_m;
      c.block_n = k.block_n;
      c.cluster_m = k.cluster_m;
      c.sched = kDataParallel;
    }
  }
  // When whole tiles quantise badly (768 x 8192: 96 pair tiles on 74 CTA pairs are two waves, the
  // second a third full), cutting the tiles x K-tiles space evenly over the workers wins although
  // the partial tiles cost about 28 % (measured with 256 x 256 pair tiles: 768 x 8192 x 8192 88.8
  // against 105 us, 256 x 28672 x 8192 102.9 against 105.7 us; 1024 x 8192 x 8192 loses, 113.8
  // against 104.1 us, and the model says so).
  {
    const long long tiles = ((M + 255) / 256) * static_cast<long long>((N + 255) / 256) * batch;
    const double workers = static_cast<double>(sms / 2);
    // (with several row tiles sharing a panel of B the even cut also costs their phase alignment in
    // K — the panel is then read from HBM more than once — hence the larger factor)
    const double cut_cost = (M + 255) / 256 == 1 ? 1.28 : 1.5;
    const double cost = static_cast<double>(tiles) / workers * 128 * 256 * 1.05 * cut_cost;
    if (tiles > workers && cost < best) {
      best = cost;
      c.block_m = 128;
      c.block_n = 256;
      c.cluster_m = 2;
      c.sched = kStreamK;
    }
    // Hybrid: the full waves as whole tiles, only the last, partly filled wave cut over all workers.
    // The cut wave costs a fixed 15-20 us on top of its fill — 0.43 of a wave at K = 8192 (measured:
    // 768 x 8192 x 8192, one full wave + 22 of 74 tiles, 80.7 against 93.1 us whole tiles and 89.9 us
    // stream-K; 4096^3, three full + 34 of 74, loses 97.2 to 94.3) —, so it pays only when the last
    // wave is less than a third full.
    const long long w = static_cast<long long>(workers);
    const long long full = tiles / w;
    const double fill = static_cast<double>(tiles - full * w) / workers;
    if (full >= 1 && fill > 0.0 && fill < 0.34) {
      const double hybrid = (static_cast<double>(full) + fill + 0.43 * 8192.0 / (K < 512 ? 512 : K)) * 128 * 256 * 1.05;
      if (hybrid < best) {
        c.block_m = 128;
        c.block_n = 256;
        c.cluster_m = 2;
        c.sched = kHybrid;
      }
    }
  }
  return c;
}

int resolve_plan(const b200_gemm_cfg& c, Plan* p) {
  if (c.block_k != 0 && c.block_k != 64) return B200_ERR_UNSUPPORTED_CFG;
  if (c.cluster_n != 0 && c.cluster_n != 1) return B200_ERR_UNSUPPORTED_CFG;
  int cm = c.cluster_m == 0 ? 1 : c.cluster_m;
  if (cm < 1 || cm > 16 || (cm & (cm - 1)) != 0) return B200_ERR_UNSUPPORTED_CFG;
  p->few_rows = 0;
  if (c.swap_ab != 0 || c.block_m == 16 || c.block_m == 32 || c.block_m == 64) {
    // Few-rows plan: the operands are swapped inside — rows of B ride the MMA's M dimension (128 per
    // sub-tile, block_n = 128 or 256 of them per CTA), block_m rows of A ride its N dimension — and
    // the product is stored transposed. cluster_m = 2 runs a CTA pair: each CTA then stages only
    // half of the block_m rows of A next to its own rows of B.
    const int rows = c.block_m == 0 ? 128 : c.block_m;
    if (rows != 16 && rows != 32 && rows != 64 && rows != 128) return B200_ERR_UNSUPPORTED_CFG;
    const int b_rows = c.block_n == 0 ? 128 : c.block_n;
    if (b_rows != 128 && b_rows != 256) return B200_ERR_UNSUPPORTED_CFG;
    if (cm > 2) return B200_ERR_UNSUPPORTED_CFG;
    if (c.sched == kSplitK) return B200_ERR_UNSUPPORTED_CFG;  // the fix-up pass writes whole rows of C
    p->few_rows = 1;
    p->pair = cm == 2 ? 1 : 0;
    p->kernel = find_kernel(rows, p->pair, b_rows / 128);
  } else {
    if (c.block_m != 0 && c.block_m != 128 && c.block_m != 256) return B200_ERR_UNSUPPORTED_CFG;
    const int mt = c.block_m == 256 ? 2 : 1;
    const int bn = c.block_n == 0 ? 128 : c.block_n;
    if (bn < 64) return B200_ERR_UNSUPPORTED_CFG;  // the narrow kernels serve the few-rows plan only
    p->pair = cm >= 2 ? 1 : 0;
    p->kernel = find_kernel(bn, p->pair, mt);
    if (p->kernel != nullptr && mt == 2 && bn < 128) p->kernel = nullptr;  // few-rows instantiations only
  }
  if (p->kernel == nullptr) return B200_ERR_UNSUPPORTED_CFG;
  if (c.stages < 0) return B200_ERR_INVALID_ARG;
  p->stages = c.stages;  // 0 = as many as fit; settled by fit_stages() once the A tile is known
  if (p->stages > kMaxStages) return B200_ERR_UNSUPPORTED_CFG;
  if (p->stages == 1) return B200_ERR_UNSUPPORTED_CFG;
  p->smem = 0;
  if (c.sched < 0 || c.sched > 4) return B200_ERR_INVALID_ARG;
  p->mode = c.sched;
  p->split_k = c.split_k <= 1 ? 1 : c.split_k;
  if (p->split_k > 64) return B200_ERR_UNSUPPORTED_CFG;
  if (p->mode == kSplitK && p->split_k == 1) p->mode = kDataParallel;
  p->raster = c.raster ? 1 : 0;
  p->group = c.group > 0 ? c.group : 8;
  if (cm > 2) p->group = p->group * (cm / 2);
  if (c.epilogue < 0 || c.epilogue > 3) return B200_ERR_INVALID_ARG;
  p->store_mode = c.epilogue == 1 ? kStoreTma : c.epilogue == 2 ? kStoreVector : c.epilogue == 3 ? kStoreStaged
                                                                                                : kStoreTma;
  p->max_ctas = c.max_ctas;
  p->c_col_major = c.c_col_major ? 1 : 0;
  if (p->few_rows) p->store_mode = kStoreScalar;  // transposed (or 16/32-column) stores: no TMA staging
  // A width that is not a whole number of 64-column chunks (224) exists for whole tiles only: the
  // partial-tile layouts and the staged store work in whole chunks.
  if (!p->few_rows && p->kernel->bn % kEpiChunkCols != 0 &&
      (p->mode != kDataParallel || p->store_mode == kStoreStaged)) {
    return B200_ERR_UNSUPPORTED_CFG;
  }
  return B200_OK;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Rows of A staged per CTA and K-tile: a full 128-row tile, or M rounded up to 8 when a single
// CTA tile already covers all of M (the MMA's remaining rows feed outputs that are never stored).
int a_rows_for(const Plan& p, int M) {
  if (p.pair || p.kernel->mt > 1 || M >= kCtaRows) return kCtaRows * p.kernel->mt;
  return (M + 7) / 8 * 8;
}

// Shared memory the epilogue needs for a store mode: two TMA staging slabs per warp (one when a
// CTA has eight epilogue warps), or one transpose slab per warp.
int epi_bytes_for(const Plan& p, int store_mode) {
  if (store_mode == kStoreTma) return p.kernel->epi_bytes;
  if (store_mode == kStoreStaged) return 4 * p.kernel->mt * kEpiSlabBytes;
  return 0;
}

// Settles the ring depth and the dynamic shared-memory size for a given A tile height.
int fit_stages(Plan* p, int a_rows, int epi_bytes) {
  const int stage_bytes = a_rows * kBlockK * 2 + p->kernel->b_bytes;
  // With a short A tile the MMA still reads a full-height tile from the stage's base address.
  // Whatever lies beyond the stage only feeds accumulator rows that are never stored, but it must
  // be shared memory this CTA owns: pad the allocation by the worst over-read of the last stage.
  const int full_a_bytes = kCtaRows * p->kernel->mt * kBlockK * 2;
  const int over_read = full_a_bytes > stage_bytes ? full_a_bytes - stage_bytes : 0;
  epi_bytes += over_read;
  int max_stages = (232448 - 1024 - epi_bytes - kBarrierBytes) / stage_bytes;
  if (max_stages > kMaxStages) max_stages = kMaxStages;
  if (p->stages == 0) p->stages = max_stages;
  if (p->stages > max_stages) return B200_ERR_SMEM;
  p->smem = 1024 + p->stages * stage_bytes + epi_bytes + kBarrierBytes;
  return B200_OK;
}

// ------------------------------------------------------------------------------------------
// Tuning table: measured configurations per shape class, consulted before the heuristic
// ------------------------------------------------------------------------------------------
// The reference's tuner searches one shape and leaves the result to the reader (a JSON file and a
// rendered best_matmul_h100.cu, gemm_tuner.py:126-145). Here the tuner's result is fed back: a
// table of (batch, M, N, K) -> configuration that the cfg == NULL dispatch looks up first.
// A shape's class is (batch > 1, ceil(log2 M), ceil(log2 N), ceil(log2 K)). A lookup takes the
// exact shape if the table has it, otherwise the entry of the same class nearest in log2
// distance, otherwise the built-in heuristic.
struct TunedEntry {
  int batch, M, N, K;
  b200_gemm_cfg cfg;
};
std::vector<TunedEntry> g_tuned;
std::mutex g_tuned_mutex;
std::once_flag g_tuned_env_once;
constexpr size_t kMaxTunedEntries = 4096;

int log2_ceil(long long x) {
  int b = 0;
  while ((1LL << b) < x) ++b;
  return b;
}

// An entry must name a kernel that exists; which shapes it is good for is the table's business.
int tuning_validate(int batch, int M, int N, int K, const b200_gemm_cfg& cfg) {
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARG;
  if (cfg.c_col_major != 0 || cfg.max_ctas != 0) return B200_ERR_INVALID_ARG;  // per-call choices, not tunables
  Plan plan;
  return resolve_plan(cfg, &plan);
}

void tuning_add_locked(const TunedEntry& n) {
  for (TunedEntry& e : g_tuned) {
    if (e.batch == n.batch && e.M == n.M && e.N == n.N && e.K == n.K) {
      e.cfg = n.cfg;
      return;
    }
  }
  g_tuned.push_back(n);
}

// Text format, one entry per line, '#' starts a comment:
//   batch M N K block_m block_n cluster_m stages sched split_k raster group epilogue [swap_ab]
// Returns the number of entries added (>= 0), or -B200_ERR_* when the file cannot be opened, a
// line is malformed or names a configuration without a kernel; then nothing is added.
int tuning_load_file(const char* path) {
  FILE* f = std::fopen(path, "r");
  if (f == nullptr) return -B200_ERR_INVALID_ARG;
  std::vector<TunedEntry> read;
  char line[512];
  int status = B200_OK;
  while (status == B200_OK && std::fgets(line, sizeof line, f) != nullptr) {
    char* hash = std::strchr(line, '#');
    if (hash != nullptr) *hash = '\0';
    int v[14] = {};
    char extra;
    const int n = std::sscanf(line, "%d %d %d %d %d %d %d %d %d %d %d %d %d %d %c", &v[0], &v[1], &v[2], &v[3], &v[4],
                              &v[5], &v[6], &v[7], &v[8], &v[9], &v[10], &v[11], &v[12], &v[13], &extra);
    if (n <= 0) continue;  // blank line or comment
    if (n != 13 && n != 14) {  // the fourteenth column (swap_ab) is optional
      status = B200_ERR_INVALID_ARG;
      break;
    }
    TunedEntry e;
    std::memset(&e, 0, sizeof e);
    e.batch = v[0];
    e.M = v[1];
    e.N = v[2];
    e.K = v[3];
    e.cfg.block_m = v[4];
    e.cfg.block_n = v[5];
    e.cfg.block_k = kBlockK;
    e.cfg.cluster_m = v[6];
    e.cfg.cluster_n = 1;
    e.cfg.stages = v[7];
    e.cfg.sched = v[8];
    e.cfg.split_k = v[9];
    e.cfg.raster = v[10];
    e.cfg.group = v[11];
    e.cfg.epilogue = v[12];
    e.cfg.swap_ab = n == 14 ? v[13] : 0;
    status = tuning_validate(e.batch, e.M, e.N, e.K, e.cfg);
    if (status == B200_OK && read.size() >= kMaxTunedEntries) status = B200_ERR_INVALID_ARG;
    if (status == B200_OK) read.push_back(e);
  }
  std::fclose(f);
  if (status != B200_OK) return -status;
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  if (g_tuned.size() + read.size() > kMaxTunedEntries) return -B200_ERR_INVALID_ARG;
  for (const TunedEntry& e : read) tuning_add_locked(e);
  return static_cast<int>(read.size());
}

// The table loaded before the first lookup: the file B200_GEMM_TUNING_TABLE names, or — when the
// variable is not set — the measured table shipped beside the library,
// <directory of this shared object>/../tuner/b200_measured.table. Setting the variable to an empty
// string starts with an empty table. Errors are ignored here (the table simply stays empty);
// b200_gemm_tuning_load reports them.
void tuning_load_default() {
  const char* path = std::getenv("B200_GEMM_TUNING_TABLE");
  if (path != nullptr) {
    if (path[0] != '\0') (void)tuning_load_file(path);
    return;
  }
  Dl_info info;
  if (dladdr(reinterpret_cast<const void*>(&tuning_load_default), &info) == 0 || info.dli_fname == nullptr) return;
  std::string lib(info.dli_fname);
  const size_t slash = lib.rfind('/');
  if (slash == std::string::npos) return;
  (void)tuning_load_file((lib.substr(0, slash) + "/../tuner/b200_measured.table").c_str());
}

bool tuning_lookup(int batch, int M, int N, int K, b200_gemm_cfg* out) {
  std::call_once(g_tuned_env_once, tuning_load_default);
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  if (g_tuned.empty()) return false;
  const int cm = log2_ceil(M), cn = log2_ceil(N), ck = log2_ceil(K);
  const TunedEntry* best = nullptr;
  double best_d = 0.0;
  for (const TunedEntry& e : g_tuned) {
    if ((e.batch > 1) != (batch > 1)) continue;
    if (e.batch == batch && e.M == M && e.N == N && e.K == K) {
      *out = e.cfg;
      return true;
    }
    if (log2_ceil(e.M) != cm || log2_ceil(e.N) != cn || log2_ceil(e.K) != ck) continue;
    const double d = std::fabs(std::log2(static_cast<double>(e.M) / M)) +
                     std::fabs(std::log2(static_cast<double>(e.N) / N)) +
                     std::fabs(std::log2(static_cast<double>(e.K) / K));
    if (best == nullptr || d < best_d) {
      best = &e;
      best_d = d;
    }
  }
  if (best == nullptr) return false;
  // A neighbour's measured configuration carries over unless this shape quantises badly with it:
  // for whole-tile schedules of many-row problems the cost model (waves x tile area) must not
  // rate it more than a quarter above the heuristic's own choice. (1536^3 next to a 2048^3 entry
  // of 128 x 256 tiles: 72 tiles on 148 SMs, where 128 x 128 tiles fill the machine.)
  const b200_gemm_cfg& c = best->cfg;
  if (M > 128 && c.sched == kDataParallel && !c.swap_ab && c.block_m >= 128) {
    const int sms = heuristic_sm_count();
    const b200_gemm_cfg h = heuristic_cfg(batch, M, N, K, sms);
    const double mine = tile_cost(c.block_m, c.block_n ? c.block_n : 128, c.cluster_m, batch, M, N, K, sms);
    const double theirs = tile_cost(h.block_m, h.block_n, h.cluster_m, batch, M, N, K, sms);
    if (mine > 1.25 * theirs) return false;
  }
  *out = c;
  return true;
}

// What cfg == NULL means: the tuning table's answer for the shape's class, else the heuristic.
b200_gemm_cfg default_cfg(int batch, int M, int N, int K) {
  b200_gemm_cfg c;
  if (tuning_lookup(batch, M, N, K, &c)) {
    // An entry tuned on a neighbouring shape may ask for more stages than this shape's A tile
    // leaves room for: then take as many as fit.
    Plan plan;
    if (resolve_plan(c, &plan) == B200_OK) {
      if (fit_stages(&plan, a_rows_for(plan, plan.few_rows ? N : M), epi_bytes_for(plan, plan.store_mode)) !=
          B200_OK) {
        c.stages = 0;
      }
      return c;
    }
  }
  return heuristic_cfg(batch, M, N, K);
}

struct Problem {
  int batch, M, N, K;          // as the kernel sees them (after a column-major swap)
  const void* A;
  const void* B;
  void* C;
  long long strideA, strideB, strideC;
};

// Workspace layout: [stream-K flags][fp32 partial slots][re-pitched A][re-pitched B]
struct WorkspaceLayout {
  size_t flag_bytes;
  size_t partial_bytes;
  size_t a_bytes;
  size_t b_bytes;
  int k_pitch;
  bool repitch;
  size_t total() const { return flag_bytes + partial_bytes + a_bytes + b_bytes; }
};

bool needs_repitch(const Problem& pr) {
  if (pr.K % 8 != 0) return true;
  if ((reinterpret_cast<uintptr_t>(pr.A) & 15u) || (reinterpret_cast<uintptr_t>(pr.B) & 15u)) return true;
  if (pr.batch > 1 && ((pr.strideA % 8) || (pr.strideB % 8))) return true;
  return false;
}

void build_sched(const Plan& p, const Problem& pr, int workers, SchedParams* s) {
  const int block_m = p.kernel->block_m;
  s->tiles_m = (pr.M + block_m - 1) / block_m;
  s->tiles_n = (pr.N + p.kernel->bn - 1) / p.kernel->bn;
  s->batch = pr.batch;
  s->num_tiles = s->tiles_m * s->tiles_n * pr.batch;
  s->k_tiles = (pr.K + kBlockK - 1) / kBlockK;
  s->group = p.group;
  s->raster = p.raster;
  s->mode = p.mode;
  s->split_k = p.split_k;
  if (s->mode == kSplitK && s->split_k > s->k_tiles) s->split_k = s->k_tiles;
  if (s->mode == kSplitK && s->split_k <= 1) {
    s->mode = kDataParallel;
    s->split_k = 1;
  }
  if ((s->mode == kHybrid || s->mode == kHybridTwoWaves) && s->num_tiles <= workers) {
    s->mode = kDataParallel;  // a single wave: nothing to balance against
  }
  long long units = s->num_tiles;
  if (s->mode == kSplitK) units *= s->split_k;
  if (s->mode == kStreamK) units = sched_total_iters(*s);
  s->num_workers = static_cast<int>(units < workers ? units : workers);
  if (s->num_workers < 1) s->num_workers = 1;
  if (s->mode == kStreamK && s->num_workers > 1) {
    // Stream-K: with W workers every worker takes tiles / W of a tile's worth of K-tiles, and the cuts
    // between workers fall at multiples of that fraction. When tiles / W reduces to p / q with a small
    // q, the cuts repeat every q workers and few tiles are cut at all (224 tiles on 112 workers:
    // none; on 140: eight tiles per five workers); on 148 workers (56 / 37) nearly every tile is cut
    // somewhere else, and every cut costs a partial tile written, read back and added. A decode
    // shape is bound by memory, not by the number of SMs that stream it, so the largest worker
    // count within a quarter of the maximum whose q is at most 8 is taken (64 x 28672 x 8192: 78.0 us
    // on 140 workers against 81.8 us on 148).
    auto gcd = [](long long a, long long b) {
      while (b != 0) {
        const long long t = a % b;
        a = b;
        b = t;
      }
      return a;
    };
    const int floor_w = s->num_workers - s->num_workers / 4;
    for (int w = s->num_workers; w >= floor_w && w >= 1; --w) {
      if (w / gcd(s->num_tiles, w) <= 8) {
        s->num_workers = w;
        break;
      }
    }
  }
  if (s->mode == kDataParallel || s->mode == kSplitK) {
    // Whole units in waves: with w waves needed anyway, ceil(units / w) workers finish at the same
    // time as all of them would, and the SMs left idle return their share of the power budget to
    // the ones that work (200 tiles on 74 CTA pairs are 3 waves; so are they on 67).
    const long long waves = (units + s->num_workers - 1) / s->num_workers;
    const long long needed = (units + waves - 1) / waves;
    if (needed < s->num_workers) s->num_workers = static_cast<int>(needed);
  }
}

WorkspaceLayout workspace_layout(const Plan& p, const Problem& pr, const SchedParams& s) {
  WorkspaceLayout w{};
  const int block_m = p.kernel->block_m;
  w.flag_bytes = sched_has_streamk_part(s.mode) ? align_up(static_cast<size_t>(sched_num_slots(s)) * 16 * sizeof(unsigned long long), 256) : 0;
  w.partial_bytes =
      align_up(static_cast<size_t>(sched_num_slots(s)) * block_m * p.kernel->bn * sizeof(float), 256);
  w.repitch = needs_repitch(pr);
  w.k_pitch = (pr.K + 7) / 8 * 8;
  if (w.repitch) {
    w.a_bytes = align_up(static_cast<size_t>(pr.batch) * pr.M * w.k_pitch * 2, 256);
    w.b_bytes = align_up(static_cast<size_t>(pr.batch) * pr.N * w.k_pitch * 2, 256);
  }
  return w;
}

// Stream-K marks a partial tile as written by storing the launch's epoch in its flag words. The
// epochs of one process start at a random 64-bit value and count up, so stale workspace contents
// (any earlier launch, or uninitialised memory) do not pass for this launch's.
unsigned long long next_epoch() {
  static std::atomic<unsigned long long> counter{[] {
    std::random_device rd;
    unsigned long long v = (static_cast<unsigned long long>(rd()) << 32) ^ rd();
    return v | (1ull << 63);
  }()};
  return counter.fetch_add(1) + 1;
}

int nominal_workers(const Plan& p, int sm_count) {
  int w = p.pair ? sm_count / 2 : sm_count;
  if (p.max_ctas > 0) {
    const int cap = p.pair ? p.max_ctas / 2 : p.max_ctas;
    if (cap < w) w = cap;
  }
  return w < 1 ? 1 : w;
}

int validate(int batch, int M, int N, int K, const void* A, const void* B, const void* C) {
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARG;
  if (A == nullptr || B == nullptr || C == nullptr) return B200_ERR_INVALID_ARG;
  return B200_OK;
}

int run_gemm(int batch, int M, int N, int K, const void* A, long long strideA, const void* B,
             long long strideB, void* C, long long strideC, float alpha, float beta,
             const b200_gemm_cfg* user_cfg, void* workspace, size_t workspace_bytes,
             cudaStream_t stream, int f16 = 0, void* const* gather_dst = nullptr, int gather_world = 0) {
  int rc = validate(batch, M, N, K, A, B, C);
  if (rc != B200_OK) return rc;
  b200_gemm_cfg cfg = user_cfg ? *user_cfg : default_cfg(batch, M, N, K);
  Plan plan;
  rc = resolve_plan(cfg, &plan);
  if (rc != B200_OK) return rc;

  Problem pr{batch, M, N, K, A, B, C, strideA, strideB, strideC};
  // The kernel computes P[pr.M, pr.N] = pr.A * pr.B^T. Two things swap the operands:
  //  * column-major C[M,N] (ld M) is row-major C^T[N,M] = B * A^T;
  //  * the few-rows plan puts the caller's rows on the MMA's N dimension, so the kernel computes
  //    C^T as well — and stores it transposed, which makes it the caller's row-major C again.
  // Both at once: the kernel's product C^T is what a column-major C holds, stored as it is.
  const bool swap_operands = plan.c_col_major || plan.few_rows;
  const int c_transposed = (plan.few_rows && !plan.c_col_major) ? 1 : 0;
  if (swap_operands) {
    pr.M = N;
    pr.N = M;
    pr.A = B;
    pr.B = A;
    pr.strideA = strideB;
    pr.strideB = strideA;
  }

  // C can be written in 16-byte pieces (TMA tiles or vector stores) when its row pitch, base and
  // batch pitch are 16-byte aligned; otherwise the epilogue falls back to 2-byte stores.
  const bool c_aligned = (pr.N % 8 == 0) && ((reinterpret_cast<uintptr_t>(pr.C) & 15u) == 0) &&
                         (pr.batch == 1 || pr.strideC % 8 == 0);
  const int store_mode = (!c_aligned || plan.few_rows) ? kStoreScalar : plan.store_mode;
  const int epi_bytes = epi_bytes_for(plan, store_mode);
  const int a_rows = a_rows_for(plan, pr.M);
  rc = fit_stages(&plan, a_rows, epi_bytes);
  if (rc != B200_OK) return rc;

  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* st = nullptr;
  rc = get_device_state(&st);
  if (rc != B200_OK) return rc;

  int resident = 0;
  rc = max_resident_workers(*st, *plan.kernel, plan.smem, &resident);
  if (rc != B200_OK) return rc;
  int workers = nominal_workers(plan, st->sm_count);
  if (workers > resident) workers = resident;

  GemmArgs args;
  std::memset(&args, 0, sizeof(args));
  build_sched(plan, pr, workers, &args.sched);
  const WorkspaceLayout ws = workspace_layout(plan, pr, args.sched);
  if (ws.total() > 0 && (workspace == nullptr || workspace_bytes < ws.total())) return B200_ERR_WORKSPACE;
  if (ws.total() > 0 && (reinterpret_cast<uintptr_t>(workspace) & 255u)) return B200_ERR_INVALID_ARG;

  const void* a_src = pr.A;
  const void* b_src = pr.B;
  long long a_pitch = pr.K, b_pitch = pr.K;
  long long a_bstride = pr.strideA, b_bstride = pr.strideB;
  if (ws.repitch) {
    uint8_t* base = static_cast<uint8_t*>(workspace) + ws.flag_bytes + ws.partial_bytes;
    uint16_t* a_dst = reinterpret_cast<uint16_t*>(base);
    uint16_t* b_dst = reinterpret_cast<uint16_t*>(base + ws.a_bytes);
    const int threads = 256;
    for (int b = 0; b < pr.batch; ++b) {
      const long long rows_a = pr.M, rows_b = pr.N;
      const int blocks_a = static_cast<int>(std::min<long long>((rows_a * pr.K + threads - 1) / threads, 148 * 16));
      const int blocks_b = static_cast<int>(std::min<long long>((rows_b * pr.K + threads - 1) / threads, 148 * 16));
      repitch_rows_kernel<<<blocks_a, threads, 0, stream>>>(
          static_cast<const uint16_t*>(pr.A) + b * pr.strideA,
          a_dst + static_cast<long long>(b) * pr.M * ws.k_pitch, rows_a, pr.K, ws.k_pitch);
      repitch_rows_kernel<<<blocks_b, threads, 0, stream>>>(
          static_cast<const uint16_t*>(pr.B) + b * pr.strideB,
          b_dst + static_cast<long long>(b) * pr.N * ws.k_pitch, rows_b, pr.K, ws.k_pitch);
    }
    B200_CUDA_TRY(cudaGetLastError());
    a_src = a_dst;
    b_src = b_dst;
    a_pitch = b_pitch = ws.k_pitch;
    a_bstride = static_cast<long long>(pr.M) * ws.k_pitch;
    b_bstride = static_cast<long long>(pr.N) * ws.k_pitch;
  }

  const bool c_tma = store_mode == kStoreTma;

  CUtensorMap map_a, map_b, map_c;
  StoreMaps<kMaxGatherPeers> gather_maps;
  rc = make_tensor_map(&map_a, a_src, pr.K, pr.M, pr.batch, a_pitch * 2, a_bstride * 2, kBlockK, a_rows);
  if (rc != B200_OK) return rc;
  rc = make_tensor_map(&map_b, b_src, pr.K, pr.N, pr.batch, b_pitch * 2, b_bstride * 2, kBlockK,
                       plan.kernel->b_rows_cta);
  if (rc != B200_OK) return rc;
  if (c_tma) {
    rc = make_tensor_map(&map_c, pr.C, pr.N, pr.M, pr.batch, static_cast<uint64_t>(pr.N) * 2,
                         pr.strideC * 2, kEpiChunkCols, 32);
    if (rc != B200_OK) return rc;
  } else {
    map_c = map_a;  // never dereferenced by the store path
  }
  if (gather_world > 0) {
    // Fused all-gather: needs the TMA-store epilogue, whole data-parallel tiles and the kernel
    // variant that takes one map per destination.
    if (!c_tma || plan.kernel->fn_gather == nullptr || args.sched.mode != kDataParallel || f16 ||
        gather_world > kMaxGatherPeers || pr.batch != 1) {
      return B200_ERR_UNSUPPORTED_CFG;
    }
    for (int p = 0; p < kMaxGatherPeers; ++p) {
      const int src = p < gather_world ? p : 0;
      rc = make_tensor_map(&gather_maps.m[p], gather_dst[src], pr.N, pr.M, 1, static_cast<uint64_t>(pr.N) * 2, 0,
                           kEpiChunkCols, 32);
      if (rc != B200_OK) return rc;
    }
  }

  args.M = pr.M;
  args.N = pr.N;
  args.K = pr.K;
  args.batch = pr.batch;
  args.stages = plan.stages;
  args.f16 = f16;
  args.store_mode = store_mode;
  args.epi_bytes = epi_bytes;
  args.C = static_cast<__nv_bfloat16*>(pr.C);
  args.ldc = c_transposed ? pr.M : pr.N;
  args.c_transposed = c_transposed;
  args.c_batch_stride = pr.strideC;
  args.flags = ws.flag_bytes ? static_cast<unsigned long long*>(workspace) : nullptr;
  args.partial = ws.partial_bytes
                     ? reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ws.flag_bytes)
                     : nullptr;
  args.epoch = next_epoch();
  args.profile = (g_profile != nullptr &&
                  g_profile_bytes >= static_cast<size_t>(args.sched.num_workers) * (plan.pair ? 2 : 1) *
                                         kProfileSlots * sizeof(long long))
                     ? g_profile
                     : nullptr;
  args.a_rows = a_rows;
  args.a_stage_bytes = a_rows * kBlockK * 2;
  args.alpha = alpha;
  args.beta = beta;
  args.scale = (alpha != 1.0f || beta != 0.0f) ? 1 : 0;
  args.status = st->status;

  cudaLaunchConfig_t lc = {};
  const int ctas = args.sched.num_workers * (plan.pair ? 2 : 1);
  lc.gridDim = dim3(static_cast<unsigned>(ctas), 1, 1);
  lc.blockDim = dim3(static_cast<unsigned>(plan.kernel->threads), 1, 1);
  lc.dynamicSmemBytes = static_cast<size_t>(plan.smem);
  lc.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = plan.pair ? 2 : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // Let this kernel's set-up overlap the tail of whatever runs before it in the stream; the
  // kernel itself waits (griddepcontrol.wait) before it touches global memory.
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = std::getenv("B200_GEMM_NO_PDL") ? 0 : 1;
  lc.attrs = attr;
  lc.numAttrs = 2;
  // (the tracing build exists for bf16 only; fp16 launches are never traced)
  if (f16) args.profile = nullptr;
  args.gather_world = gather_world;
  if (gather_world > 0) {
    const GatherFn fn = args.profile ? plan.kernel->fn_gather_traced : plan.kernel->fn_gather;
    B200_CUDA_TRY(cudaLaunchKernelEx(&lc, fn, map_a, map_b, gather_maps, args));
  } else {
    const KernelFn fn = f16 ? plan.kernel->fn_f16 : (args.profile ? plan.kernel->fn_traced : plan.kernel->fn);
    StoreMaps<1> one;
    one.m[0] = map_c;
    B200_CUDA_TRY(cudaLaunchKernelEx(&lc, fn, map_a, map_b, one, args));
  }

  if (args.sched.mode == kSplitK && sched_num_slots(args.sched) > 0) {
    const int block_m = plan.kernel->block_m;
    const int blocks = args.sched.num_tiles < st->sm_count * 4 ? args.sched.num_tiles : st->sm_count * 4;
    fixup_kernel<<<blocks, 256, 0, stream>>>(args, block_m, plan.kernel->bn);
    B200_CUDA_TRY(cudaGetLastError());
  }
  return B200_OK;
}

// ------------------------------------------------------------------------------------------
// Host-buffer path: device staging buffers kept between calls
// ------------------------------------------------------------------------------------------
struct HostPath {
  void* dA = nullptr;
  void* dB = nullptr;
  void* dC = nullptr;
  void* ws = nullptr;
  size_t a_cap = 0, b_cap = 0, c_cap = 0, ws_cap = 0;
  cudaStream_t copy_in = nullptr, compute = nullptr, copy_out = nullptr;
  std::vector<cudaEvent_t> events;
};
// One set of staging buffers, streams and events per device; calls are serialised by the mutex
// (two host threads may use the entry point, one after the other).
HostPath g_host[64];
std::mutex g_host_mutex;

int grow(void** p, size_t* cap, size_t need) {
  if (need <= *cap) return B200_OK;
  if (*p) B200_CUDA_TRY(cudaFree(*p));
  *p = nullptr;
  *cap = 0;
  B200_CUDA_TRY(cudaMalloc(p, need));
  *cap = need;
  return B200_OK;
}

}  // namespace

// ==========================================================================================
// C ABI
// ==========================================================================================
extern "C" {

int b200_gemm_bf16(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                   float beta, const b200_gemm_cfg* cfg, void* workspace, size_t workspace_bytes,
                   void* stream) {
  return run_gemm(1, M, N, K, A, 0, B, 0, C, 0, alpha, beta, cfg, workspace, workspace_bytes,
                  static_cast<cudaStream_t>(stream));
}

int b200_gemm_batched_bf16(int batch, int M, int N, int K, const void* A, long long strideA,
                           const void* B, long long strideB, void* C, long long strideC,
                           float alpha, float beta, const b200_gemm_cfg* cfg, void* workspace,
                           size_t workspace_bytes, void* stream) {
  if (cfg != nullptr && cfg->c_col_major && batch > 1) return B200_ERR_UNSUPPORTED_CFG;
  return run_gemm(batch, M, N, K, A, strideA, B, strideB, C, strideC, alpha, beta, cfg, workspace,
                  workspace_bytes, static_cast<cudaStream_t>(stream));
}

int b200_gemm_f16(int M, int N, int K, const void* A, const void* B, void* C, float alpha, float beta,
                  const b200_gemm_cfg* cfg, void* workspace, size_t workspace_bytes, void* stream) {
  return run_gemm(1, M, N, K, A, 0, B, 0, C, 0, alpha, beta, cfg, workspace, workspace_bytes,
                  static_cast<cudaStream_t>(stream), /*f16=*/1);
}

size_t b200_gemm_workspace_bytes(int batch, int M, int N, int K, const b200_gemm_cfg* user_cfg) {
  if (batch <= 0 || M <= 0 || N <= 0 || K <= 0) return 0;
  b200_gemm_cfg cfg = user_cfg ? *user_cfg : default_cfg(batch, M, N, K);
  Plan plan;
  if (resolve_plan(cfg, &plan) != B200_OK) return 0;
  Problem pr{batch, M, N, K, reinterpret_cast<const void*>(16), reinterpret_cast<const void*>(16),
             nullptr, 8, 8, 8};
  if (plan.c_col_major || plan.few_rows) {
    pr.M = N;
    pr.N = M;
  }
  // Without a device, size for a full B200 (148 SMs); the launcher re-checks against the real
  // grid and reports B200_ERR_WORKSPACE if the buffer is too small.
  int sm = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) {
    int v = 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && v > 0) sm = v;
  } else {
    (void)cudaGetLastError();
  }
  SchedParams s;
  build_sched(plan, pr, nominal_workers(plan, sm), &s);
  return workspace_layout(plan, pr, s).total();
}

int b200_gemm_default_cfg(int batch, int M, int N, int K, b200_gemm_cfg* cfg) {
  if (cfg == nullptr || batch <= 0 || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARG;
  *cfg = default_cfg(batch, M, N, K);
  Plan plan;
  int rc = resolve_plan(*cfg, &plan);
  if (rc != B200_OK) return rc;
  rc = fit_stages(&plan, a_rows_for(plan, plan.few_rows ? N : M),
                  epi_bytes_for(plan, N % 8 == 0 ? plan.store_mode : kStoreScalar));
  if (rc != B200_OK) return rc;
  cfg->stages = plan.stages;
  return B200_OK;
}

// ------------------------------------------------------------------------------------------
// Tuning table (C ABI)
// ------------------------------------------------------------------------------------------
int b200_gemm_tuning_load(const char* path) {
  if (path == nullptr) return -B200_ERR_INVALID_ARG;
  std::call_once(g_tuned_env_once, tuning_load_default);  // explicit entries go on top of the default table
  return tuning_load_file(path);
}

int b200_gemm_tuning_add(int batch, int M, int N, int K, const b200_gemm_cfg* cfg) {
  if (cfg == nullptr) return B200_ERR_INVALID_ARG;
  const int rc = tuning_validate(batch, M, N, K, *cfg);
  if (rc != B200_OK) return rc;
  std::call_once(g_tuned_env_once, tuning_load_default);
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  if (g_tuned.size() >= kMaxTunedEntries) return B200_ERR_INVALID_ARG;
  tuning_add_locked(TunedEntry{batch, M, N, K, *cfg});
  return B200_OK;
}

void b200_gemm_tuning_clear(void) {
  std::call_once(g_tuned_env_once, [] {});  // a table cleared before its first use stays empty
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  g_tuned.clear();
}

int b200_gemm_tuning_size(void) {
  std::call_once(g_tuned_env_once, tuning_load_default);
  std::lock_guard<std::mutex> lock(g_tuned_mutex);
  return static_cast<int>(g_tuned.size());
}

int b200_gemm_heuristic_cfg(int batch, int M, int N, int K, b200_gemm_cfg* cfg) {
  if (cfg == nullptr || batch <= 0 || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARG;
  *cfg = heuristic_cfg(batch, M, N, K);
  return B200_OK;
}

int b200_gemm_heuristic_cfg_for_sms(int batch, int M, int N, int K, int sm_count, b200_gemm_cfg* cfg) {
  if (cfg == nullptr || batch <= 0 || M <= 0 || N <= 0 || K <= 0 || sm_count <= 0) return B200_ERR_INVALID_ARG;
  *cfg = heuristic_cfg(batch, M, N, K, sm_count);
  return B200_OK;
}

int b200_run_kernel(int M, int N, int K, void* A, void* B, void* C, int* DB) {
  (void)DB;
  if (M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARG;
  // Column-major C: the kernel computes C^T[N, M], so the shape it sees is (N, M) — except that
  // block_m < 128 always counts the CALLER's rows (they ride the MMA's N dimension).
  b200_gemm_cfg cfg;
  if (M <= 64 && N >= 128) {
    cfg = heuristic_cfg(1, M, N, K);  // few caller rows
  } else {
    cfg = default_cfg(1, N, M, K);
    if (cfg.block_m < 128 || cfg.swap_ab) {
      // few kernel rows (small N): one CTA per 128-column tile with a short A stage
      std::memset(&cfg, 0, sizeof(cfg));
      cfg.block_m = 128;
      cfg.block_n = 128;
      cfg.block_k = 64;
      cfg.cluster_m = 1;
      cfg.cluster_n = 1;
      cfg.epilogue = 2;
    }
  }
  cfg.sched = kDataParallel;
  cfg.c_col_major = 1;
  return run_gemm(1, M, N, K, A, 0, B, 0, C, 0, 1.0f, 0.0f, &cfg, nullptr, 0, nullptr);
}

// ------------------------------------------------------------------------------------------
// GEMM for callers that may not allocate device memory
// ------------------------------------------------------------------------------------------
// Some hosts of this library cannot hand it a workspace: a serving loop that sizes all of its
// device memory once at start-up and forbids cudaMalloc afterwards (the call synchronises the
// device and can fail late, under memory pressure), or a plug-in interface that passes operands
// and nothing else. For them the few-rows stream-K GEMM keeps its partial tiles and flag words in
// the array below, which is part of the library image: every GPU that loads the library holds
// these 10 MiB until the process exits.
//
// kStaticScratchBytes covers the largest layout the few-rows configuration produces: one
// 128 x 128 fp32 partial tile and 16 flag words per SM for 148 SMs (9 718 272 bytes).
static constexpr size_t kStaticScratchBytes = 10u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` only names the symbol; it is not a device address. The address a
// kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
static void* g_static_scratch_ptr[64] = {};
static std::mutex g_static_scratch_mutex;

// The plan of the fixed-scratch entry point is pinned here, apart from the built-in heuristic and
// the tuning table, because kStaticScratchBytes is sized for exactly these tiles: single-CTA
// stream-K with 128-column tiles — 16/32/64 rows riding the MMA's N for M <= 64, a 128-row tile
// with a short A stage above that.
static b200_gemm_cfg fixed_scratch_cfg(int M, int N) {
  b200_gemm_cfg c;
  std::memset(&c, 0, sizeof(c));
  c.block_k = 64;
  c.cluster_m = 1;
  c.cluster_n = 1;
  c.group = 8;
  c.block_n = 128;
  c.sched = kStreamK;
  if (M <= 64 && N >= 128) {
    c.block_m = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  } else {
    c.block_m = 128;
    c.epilogue = 2;
  }
  return c;
}

int b200_gemm_fixed_scratch_cfg(int M, int N, int K, b200_gemm_cfg* cfg) {
  if (cfg == nullptr || M <= 0 || N <= 0 || K <= 0) return B200_ERR_INVALID_ARG;
  if (M > kCtaRows) return B200_ERR_STATIC_SCRATCH;
  *cfg = fixed_scratch_cfg(M, N);
  return B200_OK;
}

int b200_gemm_bf16_fixed_scratch(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                                 float beta, void* stream) {
  int rc = validate(1, M, N, K, A, B, C);
  if (rc != B200_OK) return rc;
  // Only the few-rows shapes (M <= 128) run stream-K by default and need scratch at all; the
  // re-pitched operand copies that K % 8 != 0 or unaligned A/B would need do not fit the budget.
  if (M > kCtaRows || K % 8 != 0 || (reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u)) {
    return B200_ERR_STATIC_SCRATCH;
  }
  b200_gemm_cfg cfg = fixed_scratch_cfg(M, N);  // never the tuning table: the scratch is sized for this plan
  if (b200_gemm_workspace_bytes(1, M, N, K, &cfg) > kStaticScratchBytes) return B200_ERR_STATIC_SCRATCH;

  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200_ERR_INVALID_ARG;
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
      void* p = nullptr;
      B200_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
      if (p == nullptr) return B200_ERR_CUDA;
      g_static_scratch_ptr[dev] = p;
    }
    scratch = g_static_scratch_ptr[dev];
  }
  // Nothing in the array has to start at zero: a flag word counts as set only when it holds this
  // launch's epoch, which no earlier launch (and not the zero-filled image) can have written.
  rc = run_gemm(1, M, N, K, A, 0, B, 0, C, 0, alpha, beta, &cfg, scratch, kStaticScratchBytes,
                static_cast<cudaStream_t>(stream));
  return rc == B200_ERR_WORKSPACE ? B200_ERR_STATIC_SCRATCH : rc;
}

// ------------------------------------------------------------------------------------------
// Row-sharded GEMM fused with the all-gather of C
// ------------------------------------------------------------------------------------------
int b200_gemm_bf16_gather(int M, int N, int K, const void* A, const void* B, void* const* C_all, int world,
                          int rank, const b200_gemm_cfg* cfg, void* stream) {
  if (C_all == nullptr || world < 1 || world > kMaxGatherPeers || rank < 0 || rank >= world) {
    return B200_ERR_INVALID_ARG;
  }
  if (M <= 0 || N <= 0 || K <= 0 || N % 8 != 0) return B200_ERR_INVALID_ARG;
  // Destination p is rank p's copy of the full [world * M, N] matrix; this rank's rows start at
  // rank * M in every copy.
  // The kernel stores to its destinations in list order; the list starts with this rank's own copy
  // and continues with rank+1, rank+2, ... so that at any moment the ranks aim at different peers.
  void* dst[kMaxGatherPeers] = {};
  for (int i = 0; i < world; ++i) {
    const int p = (rank + i) % world;
    if (C_all[p] == nullptr) return B200_ERR_INVALID_ARG;
    dst[i] = static_cast<__nv_bfloat16*>(C_all[p]) + static_cast<size_t>(rank) * M * N;
  }
  b200_gemm_cfg c = cfg ? *cfg : heuristic_cfg(1, M, N, K);
  if (cfg == nullptr) {
    // the fused epilogue exists for 256-column pair tiles with TMA stores
    c.cluster_m = 2;
    c.block_n = 256;
    // 256 rows per CTA is the faster GEMM; from four ranks on the peer stores weigh more and the
    // 128-row tile, whose epilogue overlaps the next main loop and has half as many warps storing at
    // once, measures faster (two GPUs carrying four ranks' traffic: 0.885 against 0.902 ms; eight ranks':
    // 1.453 against 1.491 ms; two ranks: 0.782 against 0.746 ms).
    if (c.block_m != 256 || world >= 4) c.block_m = 128;
    c.sched = kDataParallel;
    c.epilogue = 1;
  }
  return run_gemm(1, M, N, K, A, 0, B, 0, dst[0], 0, 1.0f, 0.0f, &c, nullptr, 0, static_cast<cudaStream_t>(stream),
                  /*f16=*/0, dst, world);
}

// Peer-visible device memory for the call above: plain cudaMalloc allocations whose CUDA IPC
// handles the ranks of one node exchange (over any channel that moves 64 bytes).
int b200_peer_alloc(size_t bytes, void** ptr) {
  if (ptr == nullptr || bytes == 0) return B200_ERR_INVALID_ARG;
  B200_CUDA_TRY(cudaMalloc(ptr, bytes));
  return B200_OK;
}

int b200_peer_free(void* ptr) {
  B200_CUDA_TRY(cudaFree(ptr));
  return B200_OK;
}

int b200_peer_export(void* ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
  if (ptr == nullptr || handle == nullptr) return B200_ERR_INVALID_ARG;
  cudaIpcMemHandle_t h;
  B200_CUDA_TRY(cudaIpcGetMemHandle(&h, ptr));
  std::memcpy(handle, &h, sizeof(h));
  return B200_OK;
}

int b200_peer_import(const unsigned char handle[64], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return B200_ERR_INVALID_ARG;
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle, sizeof(h));
  B200_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return B200_OK;
}

int b200_peer_close(void* ptr) {
  B200_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return B200_OK;
}

// ------------------------------------------------------------------------------------------
// Several GPUs of one node driven from ONE process: the M-sharded GEMM behind a C handle
// ------------------------------------------------------------------------------------------
// The reference's second harness (matmul_h100_optimal.cu:115-229) is a single-process C++ main
// around one launcher call; this is the same shape of interface for the row-sharded problem: rank
// p of `world` holds M rows of A, all of B and either its own M rows of C (gather = 0, no exchange
// at all) or a full copy of C that every rank's kernel writes into (gather = 1: the fused epilogue
// of b200_gemm_bf16_gather over peer access, which one process gets from
// cudaDeviceEnablePeerAccess without any IPC). One stream and one pair of events per device; the
// time of a run is the maximum over the devices.
struct b200_mgemm {
  int world = 0, M = 0, N = 0, K = 0, gather = 0;
  int device[kMaxGatherPeers] = {};
  void* A[kMaxGatherPeers] = {};
  void* B[kMaxGatherPeers] = {};
  void* C[kMaxGatherPeers] = {};
  void* ws[kMaxGatherPeers] = {};
  size_t ws_bytes = 0;
  cudaStream_t stream[kMaxGatherPeers] = {};
  cudaEvent_t start[kMaxGatherPeers] = {}, stop[kMaxGatherPeers] = {};
};

namespace {
struct DeviceRestore {
  int saved = -1;
  DeviceRestore() {
    if (cudaGetDevice(&saved) != cudaSuccess) saved = -1;
  }
  ~DeviceRestore() {
    if (saved >= 0) cudaSetDevice(saved);
  }
};
}  // namespace

int b200_mgemm_destroy(b200_mgemm* h) {
  if (h == nullptr) return B200_OK;
  DeviceRestore restore;
  for (int p = 0; p < h->world; ++p) {
    if (cudaSetDevice(h->device[p]) != cudaSuccess) continue;
    if (h->stream[p]) cudaStreamSynchronize(h->stream[p]);
    if (h->A[p]) cudaFree(h->A[p]);
    if (h->B[p]) cudaFree(h->B[p]);
    if (h->C[p]) cudaFree(h->C[p]);
    if (h->ws[p]) cudaFree(h->ws[p]);
    if (h->start[p]) cudaEventDestroy(h->start[p]);
    if (h->stop[p]) cudaEventDestroy(h->stop[p]);
    if (h->stream[p]) cudaStreamDestroy(h->stream[p]);
  }
  (void)cudaGetLastError();
  delete h;
  return B200_OK;
}

int b200_mgemm_create(b200_mgemm** out, int world, const int* devices, int M_shard, int N, int K, int gather) {
  if (out == nullptr || world < 1 || world > kMaxGatherPeers || M_shard <= 0 || N <= 0 || K <= 0) {
    return B200_ERR_INVALID_ARG;
  }
  if (gather != 0 && gather != 1) return B200_ERR_INVALID_ARG;
  if (gather && N % 8 != 0) return B200_ERR_INVALID_ARG;
  *out = nullptr;
  DeviceRestore restore;
  b200_mgemm* h = new b200_mgemm();
  h->world = world;
  h->M = M_shard;
  h->N = N;
  h->K = K;
  h->gather = gather;
  int rc = B200_OK;
  auto fail = [&](int code) {
    b200_mgemm_destroy(h);
    return code;
  };
  h->ws_bytes = b200_gemm_workspace_bytes(1, M_shard, N, K, nullptr);
  for (int p = 0; p < world; ++p) h->device[p] = devices ? devices[p] : p;
  for (int p = 0; p < world && rc == B200_OK; ++p) {
    if (cudaSetDevice(h->device[p]) != cudaSuccess) return fail(B200_ERR_CUDA);
    const size_t c_bytes = static_cast<size_t>(gather ? world : 1) * M_shard * N * 2;
    cudaError_t e = cudaMalloc(&h->A[p], static_cast<size_t>(M_shard) * K * 2);
    if (e == cudaSuccess) e = cudaMalloc(&h->B[p], static_cast<size_t>(N) * K * 2);
    if (e == cudaSuccess) e = cudaMalloc(&h->C[p], c_bytes);
    if (e == cudaSuccess && h->ws_bytes > 0) e = cudaMalloc(&h->ws[p], h->ws_bytes);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&h->stream[p], cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&h->start[p]);
    if (e == cudaSuccess) e = cudaEventCreate(&h->stop[p]);
    if (e != cudaSuccess) {
      g_last_cuda_error = static_cast<int>(e);
      (void)cudaGetLastError();
      return fail(B200_ERR_CUDA);
    }
    // the fused gather stores into every other rank's copy of C: map them into this device
    for (int q = 0; q < world && gather; ++q) {
      if (h->device[q] == h->device[p]) continue;
      int can = 0;
      if (cudaDeviceCanAccessPeer(&can, h->device[p], h->device[q]) != cudaSuccess || !can) {
        return fail(B200_ERR_UNSUPPORTED_CFG);
      }
      e = cudaDeviceEnablePeerAccess(h->device[q], 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        g_last_cuda_error = static_cast<int>(e);
        (void)cudaGetLastError();
        return fail(B200_ERR_CUDA);
      }
      (void)cudaGetLastError();
    }
  }
  *out = h;
  return B200_OK;
}

int b200_mgemm_buffers(b200_mgemm* h, int rank, void** A, void** B, void** C) {
  if (h == nullptr || rank < 0 || rank >= h->world) return B200_ERR_INVALID_ARG;
  if (A) *A = h->A[rank];
  if (B) *B = h->B[rank];
  if (C) *C = h->C[rank];
  return B200_OK;
}

int b200_mgemm_run(b200_mgemm* h) {
  if (h == nullptr) return B200_ERR_INVALID_ARG;
  DeviceRestore restore;
  for (int p = 0; p < h->world; ++p) {
    B200_CUDA_TRY(cudaSetDevice(h->device[p]));
    B200_CUDA_TRY(cudaEventRecord(h->start[p], h->stream[p]));
    int rc;
    if (h->gather) {
      rc = b200_gemm_bf16_gather(h->M, h->N, h->K, h->A[p], h->B[p], h->C, h->world, p, nullptr, h->stream[p]);
    } else {
      rc = run_gemm(1, h->M, h->N, h->K, h->A[p], 0, h->B[p], 0, h->C[p], 0, 1.0f, 0.0f, nullptr, h->ws[p],
                    h->ws_bytes, h->stream[p]);
    }
    if (rc != B200_OK) return rc;
    B200_CUDA_TRY(cudaEventRecord(h->stop[p], h->stream[p]));
  }
  return B200_OK;
}

int b200_mgemm_sync(b200_mgemm* h, float* ms_max) {
  if (h == nullptr) return B200_ERR_INVALID_ARG;
  DeviceRestore restore;
  float worst = 0.0f;
  for (int p = 0; p < h->world; ++p) {
    B200_CUDA_TRY(cudaSetDevice(h->device[p]));
    B200_CUDA_TRY(cudaStreamSynchronize(h->stream[p]));
  }
  for (int p = 0; p < h->world; ++p) {  // every device is done: with gather = 1 every copy of C is complete
    float ms = 0.0f;
    B200_CUDA_TRY(cudaSetDevice(h->device[p]));
    if (cudaEventElapsedTime(&ms, h->start[p], h->stop[p]) == cudaSuccess) {
      worst = ms > worst ? ms : worst;
    } else {
      (void)cudaGetLastError();  // no run yet
    }
  }
  if (ms_max) *ms_max = worst;
  return B200_OK;
}

int b200_reference_gpu_gemm_bf16(int M, int N, int K, const void* A, const void* B, void* C,
                                 float alpha, float beta, void* stream) {
  int rc = validate(1, M, N, K, A, B, C);
  if (rc != B200_OK) return rc;
  dim3 block(128, 1);
  dim3 grid((N + 511) / 512, (M + 3) / 4);
  naive_gemm_kernel<__nv_bfloat16><<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
      M, N, K, static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B),
      static_cast<__nv_bfloat16*>(C), alpha, beta);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

int b200_reference_gpu_gemm_f16(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                                float beta, void* stream) {
  int rc = validate(1, M, N, K, A, B, C);
  if (rc != B200_OK) return rc;
  dim3 block(128, 1);
  dim3 grid((N + 511) / 512, (M + 3) / 4);
  naive_gemm_kernel<__half><<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
      M, N, K, static_cast<const __half*>(A), static_cast<const __half*>(B), static_cast<__half*>(C), alpha, beta);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

// The host-buffer call and its copy-only twin share one schedule. A is cut into row bands and B
// into row bands (column bands of C); the host -> device copies go A0, B0, B1, ..., then A1, A2, ...
// and block C[i][j] is multiplied as soon as A_i and B_j are on the device and copied out right after,
// so the first result leaves for the host after a quarter of B has arrived instead of all of it,
// and what nothing overlaps at the end is one small block's kernel and copy. The host link towards
// the device is the bottleneck of the whole call: everything else hides behind it.
static int host_schedule(int M, int N, int K, const void* hA, const void* hB, void* hC, float alpha, float beta,
                         const b200_gemm_cfg* cfg, bool launch) {
  int rc = validate(1, M, N, K, hA, hB, hC);
  if (rc != B200_OK) return rc;
  if (cfg != nullptr && cfg->c_col_major) return B200_ERR_UNSUPPORTED_CFG;
  int dev = 0;
  B200_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return B200_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  HostPath& h = g_host[dev];
  for (cudaStream_t* s : {&h.copy_in, &h.compute, &h.copy_out}) {
    if (*s == nullptr) B200_CUDA_TRY(cudaStreamCreateWithFlags(s, cudaStreamNonBlocking));
  }

  // Bands are multiples of 256 rows so every block tiles like a whole problem, and a block must be
  // worth a launch: at most 8 bands of A and 4 of B.
  const bool aligned = K % 8 == 0 && N % 8 == 0;
  int na = 1, nb = 1;
  if (aligned && M >= 2048) na = M >= 8192 ? 8 : 4;
  if (aligned && N >= 4096) nb = 4;
  const int a_rows = ((M + na - 1) / na + 255) / 256 * 256;
  const int b_rows = ((N + nb - 1) / nb + 255) / 256 * 256;
  na = (M + a_rows - 1) / a_rows;
  nb = (N + b_rows - 1) / b_rows;

  const size_t a_bytes = static_cast<size_t>(M) * K * 2;
  const size_t b_bytes = static_cast<size_t>(N) * K * 2;
  // C blocks are stored compactly on the device, block (i, j) at slot i * nb + j
  const size_t block_elems = static_cast<size_t>(a_rows) * b_rows;
  const size_t c_bytes = block_elems * na * nb * 2;
  if ((rc = grow(&h.dA, &h.a_cap, a_bytes)) != B200_OK) return rc;
  if ((rc = grow(&h.dB, &h.b_cap, b_bytes)) != B200_OK) return rc;
  if ((rc = grow(&h.dC, &h.c_cap, c_bytes)) != B200_OK) return rc;
  size_t ws_need = 0;
  for (int i = 0; i < na && launch; ++i) {
    for (int j = 0; j < nb; ++j) {
      ws_need = std::max(ws_need, b200_gemm_workspace_bytes(1, std::min(a_rows, M - i * a_rows),
                                                            std::min(b_rows, N - j * b_rows), K, cfg));
    }
  }
  if ((rc = grow(&h.ws, &h.ws_cap, ws_need)) != B200_OK) return rc;
  while (static_cast<int>(h.events.size()) < na + nb + na * nb) {
    cudaEvent_t e;
    B200_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    h.events.push_back(e);
  }
  cudaEvent_t* ev_a = h.events.data();           // A_i on the device
  cudaEvent_t* ev_b = ev_a + na;                 // B_j on the device
  cudaEvent_t* ev_c = ev_b + nb;                 // C block computed

  // Once the first copy is enqueued the caller's buffers are in use by the device: every way out
  // of the code below, failures included, waits for the three streams first.
  cudaError_t ce = cudaSuccess;
  auto copy_a = [&](int i) {
    const size_t off = static_cast<size_t>(i) * a_rows * K * 2;
    const size_t bytes = static_cast<size_t>(std::min(a_rows, M - i * a_rows)) * K * 2;
    ce = cudaMemcpyAsync(static_cast<uint8_t*>(h.dA) + off, static_cast<const uint8_t*>(hA) + off, bytes,
                         cudaMemcpyHostToDevice, h.copy_in);
    if (ce == cudaSuccess) ce = cudaEventRecord(ev_a[i], h.copy_in);
  };
  auto copy_b = [&](int j) {
    const size_t off = static_cast<size_t>(j) * b_rows * K * 2;
    const size_t bytes = static_cast<size_t>(std::min(b_rows, N - j * b_rows)) * K * 2;
    ce = cudaMemcpyAsync(static_cast<uint8_t*>(h.dB) + off, static_cast<const uint8_t*>(hB) + off, bytes,
                         cudaMemcpyHostToDevice, h.copy_in);
    if (ce == cudaSuccess) ce = cudaEventRecord(ev_b[j], h.copy_in);
  };
  auto block = [&](int i, int j) {  // multiply C[i][j] and send it to the host
    const int rows = std::min(a_rows, M - i * a_rows), cols = std::min(b_rows, N - j * b_rows);
    uint8_t* dc = static_cast<uint8_t*>(h.dC) + (static_cast<size_t>(i) * nb + j) * block_elems * 2;
    // the copy stream is in order: of the two operands, the one copied later is the one to wait for
    ce = cudaStreamWaitEvent(h.compute, i == 0 ? ev_b[j] : ev_a[i], 0);
    if (ce != cudaSuccess) return;
    if (launch) {
      rc = run_gemm(1, rows, cols, K, static_cast<uint8_t*>(h.dA) + static_cast<size_t>(i) * a_rows * K * 2, 0,
                    static_cast<uint8_t*>(h.dB) + static_cast<size_t>(j) * b_rows * K * 2, 0, dc, 0, alpha, beta, cfg,
                    h.ws, h.ws_cap, h.compute);
      if (rc != B200_OK) return;
    }
    ce = cudaEventRecord(ev_c[i * nb + j], h.compute);
    if (ce == cudaSuccess) ce = cudaStreamWaitEvent(h.copy_out, ev_c[i * nb + j], 0);
    if (ce == cudaSuccess) {
      ce = cudaMemcpy2DAsync(static_cast<uint8_t*>(hC) + (static_cast<size_t>(i) * a_rows * N + static_cast<size_t>(j) * b_rows) * 2,
                             static_cast<size_t>(N) * 2, dc, static_cast<size_t>(cols) * 2, static_cast<size_t>(cols) * 2,
                             static_cast<size_t>(rows), cudaMemcpyDeviceToHost, h.copy_out);
    }
  };
  auto ok = [&]() { return ce == cudaSuccess && rc == B200_OK; };

  copy_a(0);
  for (int j = 0; j < nb && ok(); ++j) {
    copy_b(j);
    if (ok()) block(0, j);
  }
  for (int i = 1; i < na && ok(); ++i) {
    copy_a(i);
    for (int j = 0; j < nb && ok(); ++j) block(i, j);
  }
  const cudaError_t s0 = cudaStreamSynchronize(h.copy_out);
  const cudaError_t s1 = cudaStreamSynchronize(h.compute);
  const cudaError_t s2 = cudaStreamSynchronize(h.copy_in);
  if (rc != B200_OK) return rc;
  for (cudaError_t e : {ce, s0, s1, s2}) B200_CUDA_TRY(e);
  return B200_OK;
}

int b200_gemm_bf16_host(int M, int N, int K, const void* hA, const void* hB, void* hC, float alpha,
                        float beta, const b200_gemm_cfg* cfg) {
  return host_schedule(M, N, K, hA, hB, hC, alpha, beta, cfg, /*launch=*/true);
}

int b200_gemm_bf16_host_copies_only(int M, int N, int K, const void* hA, const void* hB, void* hC) {
  return host_schedule(M, N, K, hA, hB, hC, 1.0f, 0.0f, nullptr, /*launch=*/false);
}

void b200_gemm_host_release(void) {
  std::lock_guard<std::mutex> lock(g_host_mutex);
  int current = 0;
  const bool have_device = cudaGetDevice(&current) == cudaSuccess;
  for (int dev = 0; dev < 64; ++dev) {
    HostPath& h = g_host[dev];
    if (h.copy_in == nullptr && h.dA == nullptr && h.dB == nullptr && h.dC == nullptr && h.ws == nullptr) continue;
    if (cudaSetDevice(dev) != cudaSuccess) continue;
    if (h.dA) cudaFree(h.dA);
    if (h.dB) cudaFree(h.dB);
    if (h.dC) cudaFree(h.dC);
    if (h.ws) cudaFree(h.ws);
    for (cudaEvent_t e : h.events) cudaEventDestroy(e);
    if (h.copy_in) cudaStreamDestroy(h.copy_in);
    if (h.compute) cudaStreamDestroy(h.compute);
    if (h.copy_out) cudaStreamDestroy(h.copy_out);
    h = HostPath();
  }
  if (have_device) cudaSetDevice(current);
  (void)cudaGetLastError();
}

int b200_gemm_last_device_status(unsigned int out[4]) {
  if (out == nullptr) return B200_ERR_INVALID_ARG;
  B200_CUDA_TRY(cudaDeviceSynchronize());
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200_OK) return rc;
  B200_CUDA_TRY(cudaMemcpy(out, st->status, sizeof(unsigned int) * 4, cudaMemcpyDeviceToHost));
  if (out[0] != 0) {
    B200_CUDA_TRY(cudaMemset(st->status, 0, sizeof(unsigned int) * 4));
    return B200_ERR_DEVICE_TIMEOUT;
  }
  return B200_OK;
}

int b200_gemm_set_profile_buffer(void* buffer, size_t bytes) {
  std::lock_guard<std::mutex> lock(g_mutex);
  g_profile = static_cast<long long*>(buffer);
  g_profile_bytes = buffer ? bytes : 0;
  return B200_OK;
}

int b200_gemm_selftest_bounded_wait(long long budget_cycles) {
  if (budget_cycles <= 0 || budget_cycles > (1ll << 31)) return B200_ERR_INVALID_ARG;
  std::lock_guard<std::mutex> lock(g_mutex);
  DeviceState* st = nullptr;
  int rc = get_device_state(&st);
  if (rc != B200_OK) return rc;
  bounded_wait_selftest_kernel<<<1, 32>>>(st->status, budget_cycles);
  B200_CUDA_TRY(cudaGetLastError());
  return B200_OK;
}

const char* b200_gemm_strerror(int status) {
  switch (status) {
    case B200_OK: return "success";
    case B200_ERR_INVALID_ARG: return "invalid argument";
    case B200_ERR_UNSUPPORTED_CFG: return "unsupported tile/cluster/stage configuration";
    case B200_ERR_SMEM: return "configuration exceeds shared memory";
    case B200_ERR_WORKSPACE: return "workspace missing or too small";
    case B200_ERR_CUDA: return "CUDA call failed";
    case B200_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    case B200_ERR_STATIC_SCRATCH:
      return "shape or alignment outside what the fixed scratch entry point covers (M <= 128, K % 8 == 0, "
             "16-byte aligned A and B)";
    default: return "unknown status";
  }
}

int b200_gemm_last_cuda_error(void) { return g_last_cuda_error; }

int b200_gemm_sm_count(void) {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return -1;
  }
  return v;
}

}  // extern "C"
