// UMMA (tcgen05.mma) operand descriptors for sm_100a.
//
// Replaces the reference's Hopper GMMA descriptor (header.cuh:8-71, matmul_utils.cuh:4-12): on
// Blackwell the 64-bit shared-memory matrix descriptor gains a version field and a 3-bit layout
// field, and the instruction shape / data types move into a separate 32-bit instruction
// descriptor. All functions are constexpr and host-compilable so the bit layouts are unit-tested
// without a GPU.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#define B200_HD __host__ __device__ __forceinline__
#else
#define B200_HD inline
#endif

namespace b200 {

enum class InFormat : uint32_t { F16 = 0, BF16 = 1 };

// 32-bit instruction descriptor of tcgen05.mma.kind::f16:
//   [4,6)   accumulator format (1 = fp32)
//   [7,10)  A format, [10,13) B format (0 = fp16, 1 = bf16)
//   [15]    A major (0 = K-major), [16] B major (0 = K-major)
//   [17,23) N >> 3
//   [24,29) M >> 4   (M = 256 for a CTA pair, 128 or 64 for one CTA)
B200_HD constexpr uint32_t make_instr_desc(uint32_t umma_m, uint32_t umma_n, InFormat fmt) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         ((umma_n >> 3) << 17) | ((umma_m >> 4) << 24);
}

// 64-bit shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes
// (64 16-bit elements) with the 128-byte swizzle a TMA tile load produces:
//   [0,14)  start address >> 4
//   [16,30) leading byte offset >> 4 (unused for a single 128-byte swizzle atom along K: 0)
//   [32,46) stride byte offset >> 4 = 1024 B between consecutive 8-row groups
//   [46,48) descriptor version = 1
//   [61,64) layout type: 2 = SWIZZLE_128B
// The tile base must be 1024-byte aligned (base_offset field = 0). Advancing by one MMA K-step
// (16 elements = 32 bytes) inside the swizzle atom adds 32 B to the start address.
B200_HD constexpr uint64_t make_smem_desc_sw128(uint32_t smem_addr) {
  return static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4) |
         (static_cast<uint64_t>(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}

// Descriptor increment for one 16-element K-step inside a 128-byte swizzle row.
static constexpr uint64_t kDescKStep = (16u * 2u) >> 4;

// Byte offset, inside a 128B-swizzled tile whose rows are 128 bytes, of 16-byte chunk `chunk`
// (0..7) of row `row`. This is the layout both TMA (SWIZZLE_128B) and the UMMA descriptor above
// assume; the epilogue writes its staging tile with it.
B200_HD constexpr uint32_t sw128_offset(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

}  // namespace b200
