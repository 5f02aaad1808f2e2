// TEST INFRASTRUCTURE — NOT A PRODUCT PATH.
//
// C-ABI wrapper around the REAL reference oracle: it #includes reference.h from the reference
// checkout where it lies (the include directory is given on the compiler command line by
// oracle/Makefile; no reference source is copied into this repository) and instantiates
// reference_cpu_gemm<bf16,bf16,bf16,float> (reference.h:5-46). The resulting shared object,
// oracle/_ref/libref_gemm.so, needs no GPU and no libcuda: nvcc is used only because
// reference.h also defines a __global__ kernel and common.h includes CUDA headers.
//
// Used to (1) pin oracle/cpu_gemm.c bit for bit, (2) generate tests/golden/, and (3) time the
// reference's own CPU GEMM as the benchmark's reference arm.
#include <cuda_bf16.h>
#include <omp.h>

#include "reference.h"

// Number of OpenMP threads reference_cpu_gemm's `omp parallel for` uses from now on (launchers
// such as torchrun export OMP_NUM_THREADS=1).
extern "C" void ref_set_threads(int n) {
  if (n > 0) omp_set_num_threads(n);
}

extern "C" void ref_cpu_gemm_f16(int M, int N, int K, const void* A, const void* B, void* C, float alpha,
                                 float beta) {
  GemmParams<half_t, half_t, half_t, float> params(M, N, K, static_cast<const half_t*>(A),
                                                   static_cast<const half_t*>(B), static_cast<half_t*>(C), alpha,
                                                   beta);
  reference_cpu_gemm(params);
}

extern "C" void ref_cpu_gemm_bf16(int M, int N, int K, const void* A, const void* B, void* C,
                                  float alpha, float beta) {
  GemmParams<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, float> params(
      M, N, K, static_cast<const __nv_bfloat16*>(A), static_cast<const __nv_bfloat16*>(B),
      static_cast<__nv_bfloat16*>(C), alpha, beta);
  reference_cpu_gemm(params);
}
