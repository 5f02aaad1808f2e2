// C++ shim that re-creates the reference's host-side names on top of the C ABI (b200_gemm.h), so
// a harness written against Faraz9877/H100_GEMM compiles unchanged apart from its includes:
//
//   GemmParams<A,B,C,Acc>                                   common.h:206-221
//   gpu_gemm<A,B,C,Acc,CLUSTER_M,CLUSTER_N,BLOCKM,BLOCKN,BLOCKK,STAGES>(GemmParams)
//                                                           matmul_h100.cu.jinja:927-985
//   reference_gpu_gemm(GemmParams)                          reference.h:78-90
//   runKernel(M,N,K,A,B,C,DB)                               matmul_h100_optimal.cu:32-59
//   get_sm_count(), ceil_div()                              common.h:43-60,67
//
// Error behaviour follows the reference's CUDA_CHECK (common.h:29-37): print and exit.
// gpu_gemm and reference_gpu_gemm accept bf16 or half_t operands (the reference's template path is
// half_t only, its bf16 path is the fixed-configuration runKernel; both types go through both
// entry points here). Accumulation is float.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdio>
#include <cstdlib>
#include <type_traits>

#include "b200_gemm.h"

using bf16 = __nv_bfloat16;
using half_t = __half;  // common.h:27

constexpr int ceil_div(int a, int b) { return (a + (b - 1)) / b; }

inline int get_sm_count() {
  const int n = b200_gemm_sm_count();
  return n > 0 ? n : 1;
}

template <class AType, class BType, class CType, class AccumType>
struct GemmParams {
  const int M;
  const int N;
  const int K;
  const AType* A;
  const BType* B;
  CType* C;
  const AccumType alpha;
  const AccumType beta;

  GemmParams(const int M, const int N, const int K, const AType* A, const BType* B, CType* C,
             const AccumType alpha, const AccumType beta)
      : M(M), N(N), K(K), A(A), B(B), C(C), alpha(alpha), beta(beta) {}
};

inline void b200_check(int status, const char* what) {
  if (status != B200_OK) {
    std::fprintf(stderr, "%s failed: %s (cuda error %d)\n", what, b200_gemm_strerror(status),
                 b200_gemm_last_cuda_error());
    std::exit(EXIT_FAILURE);
  }
}

// The reference's kernels ignore alpha and beta (matmul_h100.cu.jinja:696 stores (CType)accum);
// its oracles apply them as acc * alpha + beta (reference.h:40,72). `apply_alpha_beta` selects
// between the two so that both of the reference's behaviours can be reproduced.
template <class AType, class BType, class CType, class AccumType, int CLUSTER_M, int CLUSTER_N,
          int BLOCKM, int BLOCKN, int BLOCKK, int STAGES>
void gpu_gemm(GemmParams<AType, BType, CType, AccumType> p, bool apply_alpha_beta = false) {
  constexpr bool is_bf16 = std::is_same<AType, bf16>::value;
  static_assert((is_bf16 || std::is_same<AType, half_t>::value) && std::is_same<BType, AType>::value &&
                    std::is_same<CType, AType>::value && std::is_same<AccumType, float>::value,
                "gpu_gemm is built for bf16 or fp16 inputs and outputs with float accumulation");
  b200_gemm_cfg cfg = {};
  cfg.block_m = BLOCKM;
  cfg.block_n = BLOCKN;
  cfg.block_k = BLOCKK;
  cfg.stages = STAGES;
  cfg.cluster_m = CLUSTER_M;
  cfg.cluster_n = CLUSTER_N;
  const float alpha = apply_alpha_beta ? p.alpha : 1.0f;
  const float beta = apply_alpha_beta ? p.beta : 0.0f;
  b200_check(is_bf16 ? b200_gemm_bf16(p.M, p.N, p.K, p.A, p.B, p.C, alpha, beta, &cfg, nullptr, 0, nullptr)
                     : b200_gemm_f16(p.M, p.N, p.K, p.A, p.B, p.C, alpha, beta, &cfg, nullptr, 0, nullptr),
             "gpu_gemm");
}

template <class AType, class BType, class CType, class AccumType>
void reference_gpu_gemm(GemmParams<AType, BType, CType, AccumType> p) {
  constexpr bool is_bf16 = std::is_same<AType, bf16>::value;
  static_assert(is_bf16 || std::is_same<AType, half_t>::value, "bf16 or fp16");
  b200_check(is_bf16 ? b200_reference_gpu_gemm_bf16(p.M, p.N, p.K, p.A, p.B, p.C, p.alpha, p.beta, nullptr)
                     : b200_reference_gpu_gemm_f16(p.M, p.N, p.K, p.A, p.B, p.C, p.alpha, p.beta, nullptr),
             "reference_gpu_gemm");
}

inline void runKernel(int M, int N, int K, bf16* A, bf16* B, bf16* C, int* DB) {
  b200_check(b200_run_kernel(M, N, K, A, B, C, DB), "runKernel");
}
