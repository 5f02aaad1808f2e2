// Bandwidth of TMA stores from shared memory into a peer GPU's memory over NVLink as a function of the
// contiguous segment size of a store — the question behind the fused GEMM + all-gather epilogue, whose
// stores are 32 x 64 boxes (32 segments of 128 bytes). One process, two devices, peer access; 148 CTAs
// of four warps, each warp streaming 4 or 8 KB stores from two alternating slabs:
//   tiled stores with 128-, 256- and 512-byte rows, fully contiguous 1-D bulk copies of 4 and 8 KB,
//   into the device's own memory (reference), into the peer's, and both devices storing at once.
// Stores only: nothing here loads from peer memory, and nothing uses multicast.
//
// Build: make -C h100_gemm_b200/bench peer_store_bw      Usage: bin/peer_store_bw   (needs two GPUs for the peer rows)
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1); } } while (0)

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// mode 0: 2D tiled store through `map` (box_cols x box_rows bf16), mode 1: 1-D bulk copy of `bytes` contiguous bytes
__global__ void __launch_bounds__(128, 1) store_kernel(const __grid_constant__ CUtensorMap map, uint8_t* dst, int mode,
                                                      int box_cols, int box_rows, int cols_total, int rows_total, int iters) {
  extern __shared__ __align__(1024) uint8_t smem[];
  const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
  const int bytes = box_cols * box_rows * 2;
  uint8_t* slab = smem + warp * 2 * 8192;  // two slabs of up to 8 KB per warp
  for (int i = lane; i < 2 * 8192 / 4; i += 32) reinterpret_cast<uint32_t*>(slab)[i] = blockIdx.x * 131 + i;
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  __syncwarp();
  const int boxes_x = cols_total / box_cols, boxes_y = rows_total / box_rows;
  const long long total_boxes = static_cast<long long>(boxes_x) * boxes_y;
  long long idx = (static_cast<long long>(blockIdx.x) * 4 + warp);
  const long long stride = static_cast<long long>(gridDim.x) * 4;
  if (lane == 0) {
    for (int it = 0; it < iters; ++it, idx += stride) {
      const long long b = idx % total_boxes;
      const int bx = static_cast<int>(b % boxes_x), by = static_cast<int>(b / boxes_x);
      const uint32_t src = smem_u32(slab + (it & 1) * 8192);
      asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
      if (mode == 0) {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                         reinterpret_cast<uint64_t>(&map)),
                     "r"(src), "r"(bx * box_cols), "r"(by * box_rows)
                     : "memory");
      } else {
        uint8_t* d = dst + b * bytes;
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(d), "r"(src), "r"(bytes) : "memory");
      }
      asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }
}

int main() {
  int ndev = 0;
  CK(cudaGetDeviceCount(&ndev));
  EncodeTiledFn encode = nullptr;
  {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    CK(cudaSetDevice(0));
    CK(cudaFree(0));
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    encode = reinterpret_cast<EncodeTiledFn>(fn);
  }
  const int rows_total = 65536, cols_total = 8192;  // 1 GiB of bf16, row pitch 16 KB
  const size_t bytes_total = static_cast<size_t>(rows_total) * cols_total * 2;
  for (int target = 0; target < (ndev >= 2 ? 2 : 1); ++target) {
    uint8_t* dst = nullptr;
    CK(cudaSetDevice(target));
    CK(cudaMalloc(&dst, bytes_total));
    CK(cudaSetDevice(0));
    if (target == 1) {
      cudaError_t e = cudaDeviceEnablePeerAccess(1, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { printf("no peer access\n"); return 1; }
      (void)cudaGetLastError();
    }
    struct Case { const char* name; int mode, cols, rows; CUtensorMapSwizzle sw; };
    const Case cases[] = {
        {"box 64 x 32 (128 B rows, 128B swizzle)", 0, 64, 32, CU_TENSOR_MAP_SWIZZLE_128B},
        {"box 64 x 64 (128 B rows, 8 KB)", 0, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B},
        {"box 128 x 32 (256 B rows)", 0, 128, 32, CU_TENSOR_MAP_SWIZZLE_NONE},
        {"box 256 x 16 (512 B rows)", 0, 256, 16, CU_TENSOR_MAP_SWIZZLE_NONE},
        {"box 256 x 8 (512 B rows, 4 KB)", 0, 256, 8, CU_TENSOR_MAP_SWIZZLE_NONE},
        {"1-D bulk 4 KB contiguous", 1, 64, 32, CU_TENSOR_MAP_SWIZZLE_NONE},
        {"1-D bulk 8 KB contiguous", 1, 128, 32, CU_TENSOR_MAP_SWIZZLE_NONE},
    };
    for (const Case& c : cases) {
      CUtensorMap map;
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols_total), static_cast<cuuint64_t>(rows_total)};
      cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols_total) * 2};
      cuuint32_t box[2] = {static_cast<cuuint32_t>(c.cols), static_cast<cuuint32_t>(c.rows)};
      cuuint32_t es[2] = {1, 1};
      CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dst, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          c.sw, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) { printf("%s: encode failed %d\n", c.name, (int)r); continue; }
      const int iters = 400;
      const size_t smem = 4 * 2 * 8192;
      CK(cudaFuncSetAttribute(store_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
      cudaEvent_t e0, e1;
      CK(cudaEventCreate(&e0));
      CK(cudaEventCreate(&e1));
      store_kernel<<<148, 128, smem>>>(map, dst, c.mode, c.cols, c.rows, cols_total, rows_total, 20);
      CK(cudaDeviceSynchronize());
      CK(cudaEventRecord(e0));
      store_kernel<<<148, 128, smem>>>(map, dst, c.mode, c.cols, c.rows, cols_total, rows_total, iters);
      CK(cudaEventRecord(e1));
      CK(cudaDeviceSynchronize());
      float ms = 0;
      CK(cudaEventElapsedTime(&ms, e0, e1));
      const double bytes = 148.0 * 4 * iters * c.cols * c.rows * 2;
      printf("%s -> %s: %.1f GB/s (%.3f ms, %.0f MB)\n", c.name, target == 0 ? "local HBM" : "peer GPU over NVLink", bytes / ms * 1e-6, ms,
             bytes * 1e-6);
    }
    CK(cudaSetDevice(target));
    CK(cudaFree(dst));
  }
  // both directions at once: device 0 stores to device 1 while device 1 stores to device 0
  if (ndev >= 2) {
    uint8_t* dst[2];
    CUtensorMap map[2];
    cudaEvent_t e0[2], e1[2];
    for (int d = 0; d < 2; ++d) {
      CK(cudaSetDevice(d));
      CK(cudaMalloc(&dst[d], bytes_total));
      cudaError_t e = cudaDeviceEnablePeerAccess(1 - d, 0);
      if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) { printf("no peer access\n"); return 1; }
      (void)cudaGetLastError();
      CK(cudaEventCreate(&e0[d]));
      CK(cudaEventCreate(&e1[d]));
      CK(cudaFuncSetAttribute(store_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 4 * 2 * 8192));
    }
    for (int d = 0; d < 2; ++d) {  // device d's map points at the OTHER device's buffer
      cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols_total), static_cast<cuuint64_t>(rows_total)};
      cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols_total) * 2};
      cuuint32_t box[2] = {64, 32};
      cuuint32_t es[2] = {1, 1};
      encode(&map[d], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, dst[1 - d], dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    }
    const int iters = 800;
    for (int rep = 0; rep < 2; ++rep) {
      for (int d = 0; d < 2; ++d) {
        CK(cudaSetDevice(d));
        CK(cudaEventRecord(e0[d]));
        store_kernel<<<148, 128, 4 * 2 * 8192>>>(map[d], dst[1 - d], 0, 64, 32, cols_total, rows_total, iters);
        CK(cudaEventRecord(e1[d]));
      }
      for (int d = 0; d < 2; ++d) {
        CK(cudaSetDevice(d));
        CK(cudaDeviceSynchronize());
      }
    }
    for (int d = 0; d < 2; ++d) {
      float ms = 0;
      CK(cudaSetDevice(d));
      CK(cudaEventElapsedTime(&ms, e0[d], e1[d]));
      const double bytes = 148.0 * 4 * iters * 64 * 32 * 2;
      printf("both directions at once, box 64 x 32: device %d -> device %d: %.1f GB/s (%.3f ms)\n", d, 1 - d, bytes / ms * 1e-6, ms);
    }
  }
  return 0;
}
