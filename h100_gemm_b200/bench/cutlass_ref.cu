// CUTLASS comparator for the sm_100a GEMM: a CUTLASS 4.x Blackwell collective-builder GEMM timed
// beside libb200gemm on the same buffers, with an exact-equality check between the two and against
// the library's plain SIMT GEMM.
//
// Counterpart of the reference's cutlass_ref/pingpong-gemm.cu (an Sm90 warp-specialised ping-pong
// GEMM checked for exact equality against CUTLASS's device reference, pingpong-gemm.cu:88-139,
// 328-358, 361-429). That file cannot be built for B200 (ArchTag Sm90, wgmma); this one asks the
// Sm100 builders for the closest equivalent: bf16 operands, fp32 accumulation, 256x256x64 tile
// computed by a CTA pair (cluster 2x1x1 — with that cluster shape the builders choose unicast
// two-CTA TMA loads, so the binary holds no TMA load with cluster multicast), automatic stage count
// and epilogue.
//
// Build (single-GPU harness; CUTLASS headers are not part of this repository):
//   make -C h100_gemm_b200/bench cutlass_ref CUTLASS_DIR=<dir holding include/ and tools/util/include/>
// Run:   bin/cutlass_ref --m=8192 --n=8192 --k=8192 --iterations=100
// Output lines follow the reference's: "Disposition: Passed|Failed", "Problem Size: MxNxK",
// "Avg runtime: <ms> ms", "GFLOPS: <f>" — once for CUTLASS, once for this library.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"
#include "cutlass/util/packed_stride.hpp"

#include "b200_gemm.h"

#define CHECK_CUDA(expr)                                                                        \
  do {                                                                                          \
    cudaError_t e__ = (expr);                                                                   \
    if (e__ != cudaSuccess) {                                                                   \
      std::fprintf(stderr, "%s:%d CUDA error %s\n", __FILE__, __LINE__, cudaGetErrorString(e__)); \
      std::exit(EXIT_FAILURE);                                                                  \
    }                                                                                           \
  } while (0)

namespace harness {

using cute::Shape;
using cute::_1;
using cute::_2;
using cute::_64;
using cute::_256;

// A is [M,K] with K contiguous (row-major); B is [N,K] with K contiguous, which CUTLASS names a
// column-major K x N operand; C and D are [M,N] row-major.
using ElementAB = cutlass::bfloat16_t;
using ElementCD = cutlass::bfloat16_t;
using ElementAcc = float;
using LayoutA = cutlass::layout::RowMajor;
using LayoutB = cutlass::layout::ColumnMajor;
using LayoutCD = cutlass::layout::RowMajor;
constexpr int kAlignAB = 128 / cutlass::sizeof_bits<ElementAB>::value;
constexpr int kAlignCD = 128 / cutlass::sizeof_bits<ElementCD>::value;

using MmaTile = Shape<_256, _256, _64>;  // per CTA pair
using Cluster = Shape<_2, _1, _1>;

using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, MmaTile, Cluster,
    cutlass::epilogue::collective::EpilogueTileAuto, ElementAcc, ElementAcc, ElementCD, LayoutCD, kAlignCD,
    ElementCD, LayoutCD, kAlignCD, cutlass::epilogue::collective::EpilogueScheduleAuto>::CollectiveOp;

using Mainloop = typename cutlass::gemm::collective::CollectiveBuilder<
    cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, ElementAB, LayoutA, kAlignAB, ElementAB, LayoutB,
    kAlignAB, ElementAcc, MmaTile, Cluster,
    cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
    cutlass::gemm::collective::KernelScheduleAuto>::CollectiveOp;

using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue, void>;
using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;

struct Options {
  int m = 5120, n = 5120, k = 4096, iterations = 100;
  float alpha = 1.0f, beta = 0.0f;
};

// --name=value, as the reference harness takes them (pingpong-gemm.cu:200-212)
bool parse(int argc, char** argv, Options* o) {
  for (int i = 1; i < argc; ++i) {
    const std::string arg = argv[i];
    const size_t eq = arg.find('=');
    if (arg == "--help" || arg.rfind("--", 0) != 0 || eq == std::string::npos) return false;
    const std::string key = arg.substr(2, eq - 2);
    const char* value = arg.c_str() + eq + 1;
    if (key == "m") o->m = std::atoi(value);
    else if (key == "n") o->n = std::atoi(value);
    else if (key == "k") o->k = std::atoi(value);
    else if (key == "iterations") o->iterations = std::atoi(value);
    else if (key == "alpha") o->alpha = static_cast<float>(std::atof(value));
    else if (key == "beta") o->beta = static_cast<float>(std::atof(value));
    else return false;
  }
  return o->m > 0 && o->n > 0 && o->k > 0 && o->iterations > 0;
}

// Integer-valued operands in [-4, 4]: every product and partial sum is exact in fp32 (for K up to
// 2^20), so two correct GEMMs agree bit for bit whatever their order of summation.
__global__ void fill_small_integers(__nv_bfloat16* p, size_t n, unsigned seed) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    unsigned x = static_cast<unsigned>(i) * 2654435761u + seed;
    x ^= x >> 15;
    x *= 2246822519u;
    x ^= x >> 13;
    p[i] = __float2bfloat16(static_cast<float>(static_cast<int>(x % 9u) - 4));
  }
}

__global__ void count_mismatches(const uint16_t* a, const uint16_t* b, size_t n, unsigned long long* out) {
  unsigned long long bad = 0;
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    bad += a[i] != b[i];
  }
  if (bad) atomicAdd(out, bad);
}

unsigned long long mismatches(const void* a, const void* b, size_t n) {
  unsigned long long* d = nullptr;
  unsigned long long h = 0;
  CHECK_CUDA(cudaMalloc(&d, sizeof h));
  CHECK_CUDA(cudaMemset(d, 0, sizeof h));
  count_mismatches<<<592, 256>>>(static_cast<const uint16_t*>(a), static_cast<const uint16_t*>(b), n, d);
  CHECK_CUDA(cudaMemcpy(&h, d, sizeof h, cudaMemcpyDeviceToHost));
  CHECK_CUDA(cudaFree(d));
  return h;
}

template <class F>
double average_ms(int iterations, F&& launch) {
  cudaEvent_t e0, e1;
  CHECK_CUDA(cudaEventCreate(&e0));
  CHECK_CUDA(cudaEventCreate(&e1));
  for (int i = 0; i < 3; ++i) launch();
  CHECK_CUDA(cudaEventRecord(e0));
  for (int i = 0; i < iterations; ++i) launch();
  CHECK_CUDA(cudaEventRecord(e1));
  CHECK_CUDA(cudaEventSynchronize(e1));
  float ms = 0.0f;
  CHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
  CHECK_CUDA(cudaEventDestroy(e0));
  CHECK_CUDA(cudaEventDestroy(e1));
  return static_cast<double>(ms) / iterations;
}

void report(const char* who, const Options& o, bool passed, double ms) {
  std::printf("%s\n", who);
  std::printf("  Disposition: %s\n", passed ? "Passed" : "Failed");
  std::printf("  Problem Size: %dx%dx%d\n", o.m, o.n, o.k);
  std::printf("  Avg runtime: %g ms\n", ms);
  std::printf("  GFLOPS: %g\n", 2.0 * o.m * o.n * o.k / (ms * 1e-3) / 1e9);
}

}  // namespace harness

int main(int argc, char** argv) {
  using namespace harness;
  Options o;
  if (!parse(argc, argv, &o)) {
    std::fprintf(stderr, "usage: %s [--m=<int>] [--n=<int>] [--k=<int>] [--alpha=<f>] [--beta=<f>] [--iterations=<int>]\n",
                 argv[0]);
    return EXIT_FAILURE;
  }
  if (o.k % kAlignAB != 0 || o.n % kAlignCD != 0) {
    std::fprintf(stderr, "K and N must be multiples of 8 (16-byte rows for TMA)\n");
    return EXIT_FAILURE;
  }
  const size_t na = static_cast<size_t>(o.m) * o.k, nb = static_cast<size_t>(o.n) * o.k;
  const size_t nc = static_cast<size_t>(o.m) * o.n;
  __nv_bfloat16 *A, *B, *C_cutlass, *C_ours, *C_simt;
  CHECK_CUDA(cudaMalloc(&A, na * 2));
  CHECK_CUDA(cudaMalloc(&B, nb * 2));
  CHECK_CUDA(cudaMalloc(&C_cutlass, nc * 2));
  CHECK_CUDA(cudaMalloc(&C_ours, nc * 2));
  CHECK_CUDA(cudaMalloc(&C_simt, nc * 2));
  fill_small_integers<<<592, 256>>>(A, na, 1u);
  fill_small_integers<<<592, 256>>>(B, nb, 2u);
  CHECK_CUDA(cudaMemset(C_cutlass, 0xff, nc * 2));
  CHECK_CUDA(cudaMemset(C_ours, 0xee, nc * 2));

  // ---- CUTLASS ----
  using StrideA = typename Gemm::GemmKernel::StrideA;
  using StrideB = typename Gemm::GemmKernel::StrideB;
  using StrideC = typename Gemm::GemmKernel::StrideC;
  using StrideD = typename Gemm::GemmKernel::StrideD;
  typename Gemm::Arguments args{
      cutlass::gemm::GemmUniversalMode::kGemm,
      {o.m, o.n, o.k, 1},
      {reinterpret_cast<ElementAB*>(A), cutlass::make_cute_packed_stride(StrideA{}, cute::make_shape(o.m, o.k, 1)),
       reinterpret_cast<ElementAB*>(B), cutlass::make_cute_packed_stride(StrideB{}, cute::make_shape(o.n, o.k, 1))},
      {{o.alpha, 0.0f},
       reinterpret_cast<ElementCD*>(C_cutlass),
       cutlass::make_cute_packed_stride(StrideC{}, cute::make_shape(o.m, o.n, 1)),
       reinterpret_cast<ElementCD*>(C_cutlass),
       cutlass::make_cute_packed_stride(StrideD{}, cute::make_shape(o.m, o.n, 1))}};
  Gemm gemm;
  if (gemm.can_implement(args) != cutlass::Status::kSuccess) {
    std::fprintf(stderr, "CUTLASS cannot implement this problem\n");
    return EXIT_FAILURE;
  }
  void* cutlass_ws = nullptr;
  const size_t cutlass_ws_bytes = Gemm::get_workspace_size(args);
  if (cutlass_ws_bytes) CHECK_CUDA(cudaMalloc(&cutlass_ws, cutlass_ws_bytes));
  if (gemm.initialize(args, cutlass_ws) != cutlass::Status::kSuccess) {
    std::fprintf(stderr, "CUTLASS initialize failed\n");
    return EXIT_FAILURE;
  }
  bool cutlass_ran = true;
  const double cutlass_ms = average_ms(o.iterations, [&] { cutlass_ran &= gemm.run() == cutlass::Status::kSuccess; });

  // ---- this library, same buffers ----
  const size_t ws_bytes = b200_gemm_workspace_bytes(1, o.m, o.n, o.k, nullptr);
  void* ws = nullptr;
  if (ws_bytes) CHECK_CUDA(cudaMalloc(&ws, ws_bytes));
  int rc = B200_OK;
  const double ours_ms = average_ms(o.iterations, [&] {
    const int r = b200_gemm_bf16(o.m, o.n, o.k, A, B, C_ours, o.alpha, 0.0f, nullptr, ws, ws_bytes, nullptr);
    if (r != B200_OK) rc = r;
  });
  if (rc != B200_OK) {
    std::fprintf(stderr, "b200_gemm_bf16: %s\n", b200_gemm_strerror(rc));
    return EXIT_FAILURE;
  }
  unsigned int status[4];
  if (b200_gemm_last_device_status(status) != B200_OK) {
    std::fprintf(stderr, "device status %u %u %u %u\n", status[0], status[1], status[2], status[3]);
    return EXIT_FAILURE;
  }

  // ---- exact equality: CUTLASS == SIMT reference == this library (beta is not compared: CUTLASS
  // reads a C matrix where this library adds a scalar, reference.h:40) ----
  rc = b200_reference_gpu_gemm_bf16(o.m, o.n, o.k, A, B, C_simt, o.alpha, 0.0f, nullptr);
  if (rc != B200_OK) {
    std::fprintf(stderr, "b200_reference_gpu_gemm_bf16: %s\n", b200_gemm_strerror(rc));
    return EXIT_FAILURE;
  }
  CHECK_CUDA(cudaDeviceSynchronize());
  const unsigned long long bad_cutlass = mismatches(C_cutlass, C_simt, nc);
  const unsigned long long bad_ours = mismatches(C_ours, C_simt, nc);
  report("CUTLASS Sm100 builder GEMM (bf16, 256x256x64 pair tile, cluster 2x1x1)", o, cutlass_ran && bad_cutlass == 0,
         cutlass_ms);
  report("libb200gemm (cfg = NULL)", o, bad_ours == 0, ours_ms);
  std::printf("mismatching elements against the SIMT GEMM: CUTLASS %llu, libb200gemm %llu of %zu\n", bad_cutlass,
              bad_ours, nc);
  return (cutlass_ran && bad_cutlass == 0 && bad_ours == 0) ? EXIT_SUCCESS : EXIT_FAILURE;
}
