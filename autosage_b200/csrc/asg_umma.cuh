// 5th-generation tensor-core primitives (tcgen05, sm_100a) as thin inline-PTX wrappers: tensor-memory
// allocation, the shared-memory and instruction descriptors of a bf16 x bf16 -> f32 MMA with K-major,
// 128-byte-swizzled operands, the MMA issue and commit, tensor-memory loads, and the split of a
// float32 value into three bfloat16 pieces whose sum reproduces it to 2^-24.
//
// One CTA per SM, cta_group::1 throughout: nothing here names a cluster, a peer CTA or multicast.
#pragma once

#include <cuda_bf16.h>

#include "asg_common.cuh"

namespace asg {
namespace umma {

constexpr int kSwizzleRowBytes = 128;   // one row of a K-major operand block: 64 bf16 of K
constexpr int kBlockK = 64;             // bf16 elements of K per swizzled row
constexpr int kInstrK = 16;             // K of one tcgen05.mma.kind::f16 instruction
constexpr int kAtomBytes = 1024;        // 8 rows x 128 bytes: the swizzle repeats every 1024 bytes

// Byte offset of element (row, k) of a K-major [rows x 64] bf16 block stored in the canonical
// 128-byte-swizzle layout: row r occupies bytes [128 r, 128 r + 128), and inside it the 16-byte
// chunk index is XORed with (r mod 8).  The block must start on a 1024-byte boundary.
__host__ __device__ __forceinline__ uint32_t swizzled_offset(uint32_t row, uint32_t k) {
  const uint32_t chunk = (k >> 3) ^ (row & 7u);
  return row * kSwizzleRowBytes + chunk * 16u + (k & 7u) * 2u;
}

#ifdef __CUDACC__

// Shared-memory matrix descriptor of a K-major, 128-byte-swizzled operand block whose first byte is
// at shared address `addr` (16-byte units in bits 0-13), leading byte offset 1 (unused by swizzled
// K-major layouts), stride byte offset 1024 (between groups of 8 rows), descriptor version 1
// (sm_100), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t smem_descriptor(uint32_t addr) {
  return static_cast<uint64_t>((addr >> 4) & 0x3FFFu) | (1ull << 16) | (static_cast<uint64_t>(kAtomBytes >> 4) << 32) |
         (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: dense, f32 accumulator (bits 4-5 = 1), bf16 A and B (bits 7-9, 10-12 = 1),
// both K-major (bits 15, 16 = 0), N/8 in bits 17-22, M/16 in bits 24-28.
__host__ __device__ __forceinline__ uint32_t instruction_descriptor(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// ---- tensor memory ----------------------------------------------------------------------------
// Allocation and release are warp-wide (all 32 lanes of ONE warp of the CTA, the same warp for both).
__device__ __forceinline__ void tmem_alloc(uint32_t* result_in_smem, uint32_t columns) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(result_in_smem)),
               "r"(columns)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_alloc_permit() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t address, uint32_t columns) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(address), "r"(columns) : "memory");
}

__device__ __forceinline__ void fence_before_thread_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_thread_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]^T, issued by ONE thread.  accumulate = 0 overwrites D.
__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Makes `bar` receive one arrival once every MMA this thread has issued so far has completed (and
// with it the reads of their shared-memory operands).  Implies fence::before_thread_sync.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive columns of 32-bit values: thread t of the warp receives row
// (lane base + t), columns [column, column + 32).  A warp may only touch the 32 lanes
// 32 * (warp index mod 4) ... + 31.  `address` = (lane << 16) | column.
__device__ __forceinline__ void tmem_load_32x32(uint32_t address, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(address)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- mbarrier helpers beyond asg_common.cuh ------------------------------------------------------
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait that also gives up as soon as the CTA-wide abort flag is set.  `limit_ns` of wall time.
__device__ __forceinline__ bool mbar_wait_or_abort(uint64_t* bar, unsigned parity, volatile int* abort_flag,
                                                   unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = global_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 32; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (*abort_flag != 0) return false;
    if (global_ns() - start > limit_ns) return false;
  }
}

// ---- float32 -> three bfloat16 pieces ------------------------------------------------------------
// x = hi + mid + lo + r with |r| <= 2^-24 |x|: hi = bf16(x), mid = bf16(x - hi), lo = bf16(x - hi - mid)
// (round to nearest each time; the two subtractions are exact in float32).
struct Pieces2 {
  uint32_t hi, mid, lo;  // two bf16 each: element 0 in the low half
};
__device__ __forceinline__ Pieces2 split_pair(float a, float b) {
  Pieces2 p;
  const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  const float2 hf = __bfloat1622float2(h);
  const float ra = a - hf.x, rb = b - hf.y;
  const __nv_bfloat162 m = __floats2bfloat162_rn(ra, rb);
  const float2 mf = __bfloat1622float2(m);
  const __nv_bfloat162 l = __floats2bfloat162_rn(ra - mf.x, rb - mf.y);
  p.hi = *reinterpret_cast<const uint32_t*>(&h);
  p.mid = *reinterpret_cast<const uint32_t*>(&m);
  p.lo = *reinterpret_cast<const uint32_t*>(&l);
  return p;
}

#endif  // __CUDACC__

}  // namespace umma
}  // namespace asg
