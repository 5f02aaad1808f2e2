// Fixed-shape comparison harness: cuBLAS against this project's kernel through runKernel(), the
// counterpart of the reference's matmul_h100_optimal.cu (main, :115-229): bf16, N(0,1) inputs from
// default_random_engine(69), column-major C, kernel 0 = cuBLAS, kernel 1 = runKernel, `repeat`
// timed launches each, TFLOPS printed per kernel. Unlike the reference (whose check is dead code,
// :177) the two results ARE compared here, with the reference's own bound (abs diff <= 0.1
// relative to the magnitude scale, :101).
//
// Build: see Makefile in this directory.   Usage: ./matmul_b200_optimal [size=8192] [repeat=8]
#include <cublas_v2.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#include "b200_gemm_shim.hpp"

extern "C" int b200_baseline_cublas_gemm_bf16(int M, int N, int K, const void* A, const void* B, void* C,
                                              int c_col_major, void* stream);

static void run_kernel(int kernel_num, int M, int N, int K, bf16* A, bf16* B, bf16* C, int* DB = nullptr) {
  if (kernel_num == 0) {
    if (b200_baseline_cublas_gemm_bf16(M, N, K, A, B, C, /*c_col_major=*/1, nullptr) != 0) {
      std::printf("CUBLAS error\n");
      std::exit(1);
    }
  } else {
    runKernel(M, N, K, A, B, C, DB);
  }
}

int main(int argc, char** argv) {
  const int size = argc > 1 ? std::atoi(argv[1]) : 8192;
  const int repeat = argc > 2 ? std::atoi(argv[2]) : 8;
  const int M = size, N = size, K = size;
  std::default_random_engine generator(69);
  std::normal_distribution<float> dist(0.f, 1.f);
  std::vector<bf16> hA(static_cast<size_t>(M) * K), hB(static_cast<size_t>(N) * K);
  for (auto& v : hA) v = __float2bfloat16(dist(generator));
  for (auto& v : hB) v = __float2bfloat16(dist(generator));
  bf16 *dA, *dB, *dC, *dC_ref;
  cudaMalloc(&dA, hA.size() * 2);
  cudaMalloc(&dB, hB.size() * 2);
  cudaMalloc(&dC, static_cast<size_t>(M) * N * 2);
  cudaMalloc(&dC_ref, static_cast<size_t>(M) * N * 2);
  cudaMemcpy(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice);

  run_kernel(0, M, N, K, dA, dB, dC_ref);
  run_kernel(1, M, N, K, dA, dB, dC);
  cudaDeviceSynchronize();
  std::vector<bf16> hC(static_cast<size_t>(M) * N), hC_ref(static_cast<size_t>(M) * N);
  cudaMemcpy(hC.data(), dC, hC.size() * 2, cudaMemcpyDeviceToHost);
  cudaMemcpy(hC_ref.data(), dC_ref, hC.size() * 2, cudaMemcpyDeviceToHost);
  const float scale = std::sqrt(static_cast<float>(K));  // |C| ~ sqrt(K) for N(0,1) inputs
  for (size_t i = 0; i < hC.size(); ++i) {
    const float d = std::fabs(__bfloat162float(hC[i]) - __bfloat162float(hC_ref[i]));
    if (d > 0.1f * scale / 8.f + 0.1f) {
      std::printf("Divergence! Should %5.2f, Is %5.2f (Diff %5.2f) at %zu\n", __bfloat162float(hC_ref[i]),
                  __bfloat162float(hC[i]), d, i);
      return 1;
    }
  }
  std::printf("Verified against cuBLAS\n");

  cudaEvent_t start, stop;
  cudaEventCreate(&start);
  cudaEventCreate(&stop);
  for (int kernel_num = 0; kernel_num < 2; ++kernel_num) {
    for (int i = 0; i < 3; ++i) run_kernel(kernel_num, M, N, K, dA, dB, dC);
    cudaDeviceSynchronize();
    cudaEventRecord(start);
    for (int i = 0; i < repeat; ++i) run_kernel(kernel_num, M, N, K, dA, dB, dC);
    cudaEventRecord(stop);
    cudaEventSynchronize(stop);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, start, stop);
    const double flops = 2.0 * M * N * K * repeat;
    std::printf("Average elapsed time: (%7.6f) s, performance: (%7.1f) TFLOPS. size: (%d). kernel %d (%s)\n",
                ms / 1000.0 / repeat, flops * 1e-9 / ms, size, kernel_num, kernel_num == 0 ? "cuBLAS" : "b200 runKernel");
  }
  return 0;
}
