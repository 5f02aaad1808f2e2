/* TEST INFRASTRUCTURE — NOT A PRODUCT PATH.
 *
 * CPU restatement of the reference's oracle GEMM, reference_cpu_gemm<bf16,bf16,bf16,float>
 * (reference.h:5-46 of Faraz9877/H100_GEMM), in plain C. Only tests, the smoke check and the
 * benchmark's CPU-baseline leg may call it; the library never does.
 *
 * What it follows, line by line:
 *   reference.h:20     one fp32 accumulator per output element, starting at 0
 *   reference.h:21-34  k ascending from 0 to K-1; accum += (float)A[i*K+k] * (float)B[j*K+k]
 *                      (A is [M,K], B is [N,K], both K-contiguous, so C = A * B^T)
 *   reference.h:40     C[i*N+j] = (bf16)(accum * alpha + beta)   -- beta is a SCALAR addend
 * The reference walks 64x64 output blocks and wraps tail loads with % M / % N
 * (reference.h:15-31); neither changes any stored element, because each element's own sum is
 * formed in the same k order and wrapped elements are never stored (reference.h:39). This file
 * is free to block differently for speed.
 *
 * bf16 <-> fp32 follows cuda_bf16.h's host path, which the reference's casts resolve to:
 * widening is a 16-bit shift; narrowing rounds to nearest even and maps NaN to 0x7FFF.
 * The product of two bf16 values is exact in fp32 (8+8 significand bits), so a fused
 * multiply-add and a separate multiply and add give the same sum; the file is nevertheless
 * meant to be compiled with -ffp-contract=off so the alpha/beta line is a multiply then an add.
 *
 * Parity status: PINNED. tests/test_oracle.py compares this file bit for bit with the real
 * reference.h compiled from the reference checkout (oracle/_ref), and with committed golden
 * vectors that oracle/_ref produced (tests/golden/).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* Number of OpenMP threads later calls use (launchers such as torchrun export OMP_NUM_THREADS=1). */
void oracle_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

static inline float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

static inline uint16_t f32_to_bf16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFFu; /* NaN */
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* IEEE binary16 <-> fp32, as cuda_fp16.h's host path does: widening is exact; narrowing rounds to
 * nearest even, produces subnormals, overflows to infinity, and maps NaN to 0x7FFF. */
static inline float f16_to_f32(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else { /* subnormal: normalise */
      int e = -1;
      do {
        ++e;
        man <<= 1;
      } while ((man & 0x400u) == 0);
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7F800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, sizeof f);
  return f;
}

static inline uint16_t f32_to_f16_rne(float f) {
  uint32_t u;
  memcpy(&u, &f, sizeof u);
  const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
  const uint32_t abs = u & 0x7FFFFFFFu;
  if (abs > 0x7F800000u) return 0x7FFFu;                    /* NaN */
  if (abs >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u); /* rounds to >= 65520: infinity */
  if (abs < 0x33000001u) return sign;                        /* below half the smallest subnormal */
  int exp = (int)(abs >> 23) - 127;
  uint32_t man = (abs & 0x7FFFFFu) | 0x800000u;
  int shift;
  uint32_t base;
  if (exp < -14) { /* subnormal result */
    shift = 13 + (-14 - exp);
    base = 0;
  } else {
    shift = 13;
    base = (uint32_t)(exp + 15) << 10;
    man &= 0x7FFFFFu;
  }
  uint32_t q = man >> shift;
  const uint32_t rem = man & ((1u << shift) - 1u);
  const uint32_t half = 1u << (shift - 1);
  if (rem > half || (rem == half && (q & 1u))) ++q; /* carries into the exponent correctly */
  return (uint16_t)(sign | (base + q));
}

uint16_t oracle_f32_to_f16(float f) { return f32_to_f16_rne(f); }
float oracle_f16_to_f32(uint16_t h) { return f16_to_f32(h); }

uint16_t oracle_f32_to_bf16(float f) { return f32_to_bf16_rne(f); }
float oracle_bf16_to_f32(uint16_t h) { return bf16_to_f32(h); }

/* Rows [row_begin, row_end) of C. Threads (OpenMP, when compiled with it) split row blocks, as
 * the reference's outer `omp parallel for` does (reference.h:14). */
void oracle_cpu_gemm_bf16_rows(int M, int N, int K, const uint16_t* A, const uint16_t* B,
                               uint16_t* C, float alpha, float beta, int row_begin, int row_end) {
  enum { BI = 16, BJ = 64 };
  (void)M;
#pragma omp parallel
  {
    float* a_f = (float*)malloc(sizeof(float) * (size_t)BI * (size_t)K);
    float* b_f = (float*)malloc(sizeof(float) * (size_t)BJ * (size_t)K);
#pragma omp for schedule(dynamic, 1)
    for (int i0 = row_begin; i0 < row_end; i0 += BI) {
      const int bi = row_end - i0 < BI ? row_end - i0 : BI;
      for (int ii = 0; ii < bi; ++ii)
        for (int k = 0; k < K; ++k) a_f[(size_t)ii * K + k] = bf16_to_f32(A[(size_t)(i0 + ii) * K + k]);
      for (int j0 = 0; j0 < N; j0 += BJ) {
        const int bj = N - j0 < BJ ? N - j0 : BJ;
        /* b_f is stored k-major ([k][jj]) so the inner loop runs over independent outputs. */
        for (int jj = 0; jj < bj; ++jj)
          for (int k = 0; k < K; ++k) b_f[(size_t)k * BJ + jj] = bf16_to_f32(B[(size_t)(j0 + jj) * K + k]);
        for (int ii = 0; ii < bi; ++ii) {
          float acc[BJ];
          for (int jj = 0; jj < BJ; ++jj) acc[jj] = 0.0f;
          const float* a_row = a_f + (size_t)ii * K;
          for (int k = 0; k < K; ++k) {
            const float a = a_row[k];
            const float* b_row = b_f + (size_t)k * BJ;
            for (int jj = 0; jj < bj; ++jj) acc[jj] += a * b_row[jj];
          }
          for (int jj = 0; jj < bj; ++jj)
            C[(size_t)(i0 + ii) * N + j0 + jj] = f32_to_bf16_rne(acc[jj] * alpha + beta);
        }
      }
    }
    free(a_f);
    free(b_f);
  }
}

/* reference_cpu_gemm<half_t, half_t, half_t, float>: the instantiation the reference's template
 * path uses (matmul_h100.cu.jinja:1010-1013). Same loop; only the conversions differ. The product
 * of two fp16 values has at most 22 significant bits, so it too is exact in fp32. */
void oracle_cpu_gemm_f16(int M, int N, int K, const uint16_t* A, const uint16_t* B, uint16_t* C,
                         float alpha, float beta) {
#pragma omp parallel
  {
    float* a_f = (float*)malloc(sizeof(float) * (size_t)K);
    float* acc = (float*)malloc(sizeof(float) * (size_t)N);
#pragma omp for schedule(dynamic, 4)
    for (int i = 0; i < M; ++i) {
      for (int k = 0; k < K; ++k) a_f[k] = f16_to_f32(A[(size_t)i * K + k]);
      for (int j = 0; j < N; ++j) {
        const uint16_t* b = B + (size_t)j * K;
        float s = 0.0f;
        for (int k = 0; k < K; ++k) s += a_f[k] * f16_to_f32(b[k]);
        acc[j] = s;
      }
      for (int j = 0; j < N; ++j) C[(size_t)i * N + j] = f32_to_f16_rne(acc[j] * alpha + beta);
    }
    free(a_f);
    free(acc);
  }
}

void oracle_cpu_gemm_bf16(int M, int N, int K, const uint16_t* A, const uint16_t* B, uint16_t* C,
                          float alpha, float beta) {
  oracle_cpu_gemm_bf16_rows(M, N, K, A, B, C, alpha, beta, 0, M);
}

/* Selected rows only (rows[i] indexes A and C); output is written densely: Cs[i*N + j]. Used to
 * spot-check shapes whose full product would take minutes on a CPU. */
void oracle_cpu_gemm_bf16_sampled_rows(int N, int K, const uint16_t* A, const uint16_t* B,
                                       uint16_t* Cs, float alpha, float beta, const int* rows,
                                       int nrows) {
#pragma omp parallel for schedule(dynamic, 1)
  for (int r = 0; r < nrows; ++r) {
    const uint16_t* a = A + (size_t)rows[r] * K;
    for (int j = 0; j < N; ++j) {
      const uint16_t* b = B + (size_t)j * K;
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) acc += bf16_to_f32(a[k]) * bf16_to_f32(b[k]);
      Cs[(size_t)r * N + j] = f32_to_bf16_rne(acc * alpha + beta);
    }
  }
}
