// Multi-GPU harness of the row-sharded GEMM, one process driving every GPU of the node through
// the C ABI (b200_mgemm_*). The counterpart, for several devices, of the reference's fixed-shape
// main (matmul_h100_optimal.cu:115-229: fill, launch `repeat` times, print TFLOPS); the reference
// itself stops at one GPU.
//
// Problem: C[P * rows, N] = A[P * rows, K] * B[N, K]^T, `rows` rows of A per GPU, B on every GPU.
// For each P in 1, 2, 4, ... up to the devices present it prints the box throughput of
//   compute only   every GPU fills its own rows of C, nothing is exchanged, and
//   fused gather   every GPU's epilogue also stores its tiles into all other GPUs' copies of C,
// timed as the slowest device's CUDA events around `repeat` launches, and checks rank 0's first and
// last rows of the gathered C against the on-device SIMT GEMM.
//
// Build: see Makefile in this directory.   Usage: ./matmul_b200_multi [rows=8192] [N=8192] [K=8192] [repeat=10]
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "b200_gemm.h"

static void check(int status, const char* what) {
  if (status != B200_OK) {
    std::fprintf(stderr, "%s failed: %s (cuda error %d)\n", what, b200_gemm_strerror(status), b200_gemm_last_cuda_error());
    std::exit(EXIT_FAILURE);
  }
}

static void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) {
    std::fprintf(stderr, "%s failed: %s\n", what, cudaGetErrorString(e));
    std::exit(EXIT_FAILURE);
  }
}

// values in [-4, 4], a function of (seed, index) only: any GPU regenerates any part of the matrices
static void fill(std::vector<__nv_bfloat16>& v, unsigned seed) {
  unsigned x = seed * 2654435761u + 12345u;
  for (auto& e : v) {
    x = x * 1664525u + 1013904223u;
    e = __float2bfloat16(static_cast<float>(static_cast<int>((x >> 24) % 9) - 4));
  }
}

static double run(int P, int rows, int N, int K, int repeat, int gather, const std::vector<__nv_bfloat16>& hB,
                  bool* ok) {
  b200_mgemm* h = nullptr;
  check(b200_mgemm_create(&h, P, nullptr, rows, N, K, gather), "b200_mgemm_create");
  std::vector<__nv_bfloat16> hA(static_cast<size_t>(rows) * K);
  for (int p = 0; p < P; ++p) {
    void *A, *B, *C;
    check(b200_mgemm_buffers(h, p, &A, &B, &C), "b200_mgemm_buffers");
    fill(hA, 100u + p);
    cuda_check(cudaSetDevice(p), "cudaSetDevice");
    cuda_check(cudaMemcpy(A, hA.data(), hA.size() * 2, cudaMemcpyHostToDevice), "copy A");
    cuda_check(cudaMemcpy(B, hB.data(), hB.size() * 2, cudaMemcpyHostToDevice), "copy B");
  }
  float ms = 0.f;
  for (int i = 0; i < 3; ++i) check(b200_mgemm_run(h), "b200_mgemm_run");  // warm-up
  check(b200_mgemm_sync(h, &ms), "b200_mgemm_sync");
  double total_ms = 0.0;
  for (int i = 0; i < repeat; ++i) {
    check(b200_mgemm_run(h), "b200_mgemm_run");
    check(b200_mgemm_sync(h, &ms), "b200_mgemm_sync");  // slowest device of this launch
    total_ms += ms;
  }
  // rank 0's copy: the rows of the LAST rank (written over NVLink when gather = 1) against the SIMT GEMM
  {
    const int last = gather ? P - 1 : 0;
    void *A0, *B0, *C0, *Al, *Bl, *Cl;
    check(b200_mgemm_buffers(h, 0, &A0, &B0, &C0), "buffers");
    check(b200_mgemm_buffers(h, last, &Al, &Bl, &Cl), "buffers");
    const int sample = rows < 256 ? rows : 256;
    std::vector<__nv_bfloat16> got(static_cast<size_t>(sample) * N), want(got.size());
    cuda_check(cudaSetDevice(last), "cudaSetDevice");
    __nv_bfloat16* ref = nullptr;
    cuda_check(cudaMalloc(&ref, got.size() * 2), "cudaMalloc");
    check(b200_reference_gpu_gemm_bf16(sample, N, K, Al, Bl, ref, 1.0f, 0.0f, nullptr), "reference");
    cuda_check(cudaMemcpy(want.data(), ref, want.size() * 2, cudaMemcpyDeviceToHost), "copy ref");
    cuda_check(cudaFree(ref), "cudaFree");
    cuda_check(cudaSetDevice(0), "cudaSetDevice");
    const __nv_bfloat16* src = static_cast<const __nv_bfloat16*>(C0) + static_cast<size_t>(gather ? last : 0) * rows * N;
    cuda_check(cudaMemcpy(got.data(), src, got.size() * 2, cudaMemcpyDeviceToHost), "copy C");
    size_t bad = 0;
    for (size_t i = 0; i < got.size(); ++i) bad += __bfloat162float(got[i]) != __bfloat162float(want[i]);
    if (bad) {
      std::printf("Wrong answer! %zu of %zu sampled elements differ (P=%d, gather=%d)\n", bad, got.size(), P, gather);
      *ok = false;
    }
  }
  unsigned int status[4];
  for (int p = 0; p < P; ++p) {
    cuda_check(cudaSetDevice(p), "cudaSetDevice");
    if (b200_gemm_last_device_status(status) != B200_OK) {
      std::printf("Device %d status %u block %u tile %u\n", p, status[0], status[1], status[2]);
      *ok = false;
    }
  }
  check(b200_mgemm_destroy(h), "b200_mgemm_destroy");
  return total_ms / repeat;
}

int main(int argc, char** argv) {
  const int rows = argc > 1 ? std::atoi(argv[1]) : 8192;
  const int N = argc > 2 ? std::atoi(argv[2]) : 8192;
  const int K = argc > 3 ? std::atoi(argv[3]) : 8192;
  const int repeat = argc > 4 ? std::atoi(argv[4]) : 10;
  int devices = 0;
  cuda_check(cudaGetDeviceCount(&devices), "cudaGetDeviceCount");
  std::printf("Shape per GPU M=%d, N=%d, K=%d; %d device(s)\n", rows, N, K, devices);
  std::vector<__nv_bfloat16> hB(static_cast<size_t>(N) * K);
  fill(hB, 7u);
  bool ok = true;
  for (int P = 1; P <= devices && P <= 8; P *= 2) {
    const double flops = 2.0 * P * rows * static_cast<double>(N) * K;
    const double t_plain = run(P, rows, N, K, repeat, 0, hB, &ok);
    const double t_gather = run(P, rows, N, K, repeat, 1, hB, &ok);
    std::printf("P=%d  compute only: %.4f ms, %.1f TFLOPS (box)   fused gather: %.4f ms, %.1f TFLOPS (box)\n", P,
                t_plain, flops / t_plain * 1e-9, t_gather, flops / t_gather * 1e-9);
  }
  if (ok) std::printf("Correct!\n");
  return ok ? 0 : 1;
}
