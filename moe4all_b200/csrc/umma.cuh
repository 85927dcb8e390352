// tcgen05 (5th-generation tensor core) helpers for sm_100a: tensor-memory allocation, shared-memory
// matrix descriptors for K-major 128-byte-swizzled f16 tiles, MMA issue, commit, accumulator loads.
// Single-CTA group only (cta_group::1); nothing here multicasts.
#pragma once
#include "common.cuh"

namespace infr {
namespace umma {

// ---- tensor memory ----------------------------------------------------------------------------
// Executed by one full warp.  `slot` (shared memory) receives the base address; columns are a
// power of two >= 32.
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Generic-proxy writes to shared memory (st.shared) become visible to the tensor core's reads.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- operand tiles in shared memory -------------------------------------------------------------
// A K-major tile of `rows` x 64 f16 (128 bytes per row), 128-byte swizzle: row r lives at byte
// r*128, its 16-byte chunk c at chunk position c ^ (r & 7).  Eight rows form one 1024-byte
// swizzle atom; the tile base must be 1024-byte aligned.
__device__ __forceinline__ uint32_t swz128_offset(int row, int chunk) {
  return (uint32_t)row * 128u + (uint32_t)((chunk ^ (row & 7)) << 4);
}

// 64-bit matrix descriptor for such a tile (start address, leading/stride byte offsets in units
// of 16 bytes, descriptor version 1, swizzle mode 128B).  `k16` selects the 16-element K slice
// inside the 64-element row (32 bytes each).
__device__ __forceinline__ uint64_t smem_desc_k_major_swz128(const void* tile, int k16) {
  const uint32_t addr = smem_u32(tile) + (uint32_t)k16 * 32u;
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFFu) >> 4);        // bits  0-13: start address
  d |= (uint64_t)1 << 16;                          // bits 16-29: leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024u >> 4) << 32;               // bits 32-45: stride byte offset = 8 rows * 128 B
  d |= (uint64_t)1 << 46;                          // bits 46-47: descriptor version (sm_100)
  d |= (uint64_t)2 << 61;                          // bits 61-63: swizzle mode 128 B
  return d;
}

// 32-bit instruction descriptor for kind::f16: f16 x f16 -> f32, both operands K-major.
__device__ __forceinline__ uint32_t idesc_f16_f32(int m, int n) {
  uint32_t d = 0;
  d |= 1u << 4;                      // D format: f32
  d |= 0u << 7;                      // A format: f16
  d |= 0u << 10;                     // B format: f16
  d |= 0u << 15;                     // A major: K
  d |= 0u << 16;                     // B major: K
  d |= (uint32_t)(n >> 3) << 17;     // N / 8
  d |= (uint32_t)(m >> 4) << 24;     // M / 16
  return d;
}

// D[tmem] (+)= A[smem] * B[smem]^T for one K = 16 slice.  Issued by ONE thread.
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

// The accumulating form without the predicate set-up.
__device__ __forceinline__ void mma_f16_acc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.eq.b32 p, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc)
      : "memory");
}

// All MMAs issued so far by this thread arrive on `bar` when they have completed.
__device__ __forceinline__ void commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive columns of f32 accumulators -> 32 registers per thread (thread i of
// the warp reads TMEM lane base+i).  The warp may only touch lanes 32*(warp%4) .. +31.
__device__ __forceinline__ void ld_32x32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// Two such loads in flight, one wait: 32 columns at `ta` into a, 32 columns at `tb` into b.  One
// asm statement, so that no use of the outputs can be scheduled ahead of the wait.
__device__ __forceinline__ void ld_32x32_pair(uint32_t ta, uint32_t tb, float (&a)[32], float (&b)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%64];\n\t"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%65];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=f"(a[0]), "=f"(a[1]), "=f"(a[2]), "=f"(a[3]), "=f"(a[4]), "=f"(a[5]), "=f"(a[6]), "=f"(a[7]), "=f"(a[8]), "=f"(a[9]), "=f"(a[10]), "=f"(a[11]), "=f"(a[12]), "=f"(a[13]), "=f"(a[14]), "=f"(a[15]), "=f"(a[16]), "=f"(a[17]), "=f"(a[18]), "=f"(a[19]), "=f"(a[20]), "=f"(a[21]), "=f"(a[22]), "=f"(a[23]), "=f"(a[24]), "=f"(a[25]), "=f"(a[26]), "=f"(a[27]), "=f"(a[28]), "=f"(a[29]), "=f"(a[30]), "=f"(a[31]),
        "=f"(b[0]), "=f"(b[1]), "=f"(b[2]), "=f"(b[3]), "=f"(b[4]), "=f"(b[5]), "=f"(b[6]), "=f"(b[7]), "=f"(b[8]), "=f"(b[9]), "=f"(b[10]), "=f"(b[11]), "=f"(b[12]), "=f"(b[13]), "=f"(b[14]), "=f"(b[15]), "=f"(b[16]), "=f"(b[17]), "=f"(b[18]), "=f"(b[19]), "=f"(b[20]), "=f"(b[21]), "=f"(b[22]), "=f"(b[23]), "=f"(b[24]), "=f"(b[25]), "=f"(b[26]), "=f"(b[27]), "=f"(b[28]), "=f"(b[29]), "=f"(b[30]), "=f"(b[31])
      : "r"(ta), "r"(tb)
      : "memory");
}

}  // namespace umma
}  // namespace infr
