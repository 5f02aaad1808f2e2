// Stand-alone cuBLAS / cuBLASLt bf16 benchmark on K-major operands: the counterpart of the
// reference's cublas_ref/spmm_test.cu (dense part only; its sparsity argument and structured-
// sparsity initialisation belong to an unrelated SpMM project and are left out).
// Usage: ./cublas_ref M K N [iters]      (argument order of spmm_test.cu:21-28)
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

extern "C" int b200_baseline_cublas_gemm_bf16(int, int, int, const void*, const void*, void*, int, void*);
extern "C" int b200_baseline_cublaslt_gemm_bf16(int, int, int, const void*, const void*, void*, void*);

int main(int argc, char** argv) {
  if (argc < 4) {
    std::printf("Usage: %s M K N [iters]\n", argv[0]);
    return 2;
  }
  const int M = std::atoi(argv[1]), K = std::atoi(argv[2]), N = std::atoi(argv[3]);
  const int iters = argc > 4 ? std::atoi(argv[4]) : 100;
  std::vector<__nv_bfloat16> hA(static_cast<size_t>(M) * K), hB(static_cast<size_t>(N) * K);
  std::srand(1);
  for (auto& v : hA) v = __float2bfloat16(static_cast<float>(std::rand() % 5) - 2.f);
  for (auto& v : hB) v = __float2bfloat16(static_cast<float>(std::rand() % 5) - 2.f);
  void *dA, *dB, *dC;
  cudaMalloc(&dA, hA.size() * 2);
  cudaMalloc(&dB, hB.size() * 2);
  cudaMalloc(&dC, static_cast<size_t>(M) * N * 2);
  cudaMemcpy(dA, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(dB, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice);
  cudaEvent_t start, stop;
  cudaEventCreate(&start);
  cudaEventCreate(&stop);
  for (int which = 0; which < 2; ++which) {
    auto call = [&]() {
      return which == 0 ? b200_baseline_cublas_gemm_bf16(M, N, K, dA, dB, dC, 0, nullptr)
                        : b200_baseline_cublaslt_gemm_bf16(M, N, K, dA, dB, dC, nullptr);
    };
    for (int i = 0; i < 10; ++i)
      if (call() != 0) return 1;
    cudaDeviceSynchronize();
    cudaEventRecord(start);
    for (int i = 0; i < iters; ++i) call();
    cudaEventRecord(stop);
    cudaEventSynchronize(stop);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, start, stop);
    ms /= iters;
    std::printf("******************************************Problem Size******************************************\n");
    std::printf("M: %d N: %d K: %d\n", M, N, K);
    std::printf("%s -> Time/ms: %5.3f\t Performance/TFLOPs: %4.2f\n", which == 0 ? "CuBlas_TC" : "CuBlasLt",
                ms, 2.0 * M * N * K / (ms / 1000.0) / 1e12);
  }
  return 0;
}
