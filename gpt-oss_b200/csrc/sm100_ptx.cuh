// Thin inline-PTX wrappers for the sm_100a features the expert GEMM uses:
// mbarrier, TMA (cp.async.bulk[.tensor], never with cluster multicast), tensor
// memory (tcgen05.alloc/ld/st), and the tcgen05.mma instruction with its A operand
// in tensor memory.  Every wait is bounded: a wait that runs out records a code
// in a status word and returns false so the kernel can unwind (free its tensor
// memory, leave) instead of hanging the device.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sm100 {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  `abort_flag` is a CTA-shared word that any role sets when it
// gives up; `status` is the global status word the host reads.  About one
// second of polling at most, and it leaves early once another role aborted.
constexpr long long kWaitCycles = 2000000000LL;
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                          unsigned int *status, unsigned int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spin & 63u) == 63u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) break;
    }
  }
  *abort_flag = 1u;
  atomicOr(status, code);
  return false;
}

// The same wait for a whole converged warp.  Every decision is taken by a vote, so the 32 lanes leave
// together (success or give-up) and may go on to warp-wide instructions (elect.sync).  The roles that
// issue tcgen05.mma or TMA keep their warp converged and elect one lane per instruction group: the
// operands of those instructions (descriptors, tensor-memory addresses) are then computed once per warp in
// uniform registers; a lone diverged lane has to move every one of them there, which on this part costs
// the issuing thread more than the instructions themselves.
__device__ __forceinline__ bool mbar_wait_warp(uint32_t bar, uint32_t parity, volatile uint32_t *abort_flag,
                                               unsigned int *status, unsigned int code) {
  if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
  const long long t0 = clock64();
  bool timed_out = false;
  for (uint32_t spin = 0;; ++spin) {
    if (__all_sync(0xffffffffu, mbar_try_wait(bar, parity))) return true;
    if ((spin & 63u) == 63u) {
      timed_out = __any_sync(0xffffffffu, clock64() - t0 > kWaitCycles);
      if (timed_out || __any_sync(0xffffffffu, *abort_flag != 0u)) break;
    }
  }
  if (timed_out && (threadIdx.x & 31u) == 0u) {
    *abort_flag = 1u;
    atomicOr(status, code);
  }
  return false;
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap *m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
// 2-D tile load, global -> shared, completion on an mbarrier (no multicast).
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *m, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *m, int x, int y, int z,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z)
      : "memory");
}
// L2 policy for data that is streamed once: its lines are the first to go when L2 needs room.
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void tma_load_3d_hint(uint32_t dst, const CUtensorMap *m, int x, int y, int z, uint32_t bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_load_hint(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar,
                                               uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
// Untiled bulk copy: both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}

// ---------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// One warp, 32 lanes x 16 consecutive 32-bit columns; lane i <-> TMEM lane
// (taddr.lane + i).  A warp may only touch lanes 32*(warp_id % 4) .. +31.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
      "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}

// ---------------------------------------------------------------- tcgen05.mma
// D[tmem] (+)= A[tmem] * B[smem]^T, kind::f16 (fp16 operands, fp32 accumulate),
// M = 128, K = 16 per instruction, issued by ONE thread.
__device__ __forceinline__ void mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives (count 1) on an mbarrier once every MMA issued so far by this thread
// has completed.  Implies tcgen05.fence::before_thread_sync.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}

// Instruction descriptor, kind::f16: fp32 accumulator, fp16 A and B, both
// K-major, M = 128, N = n (multiple of 16, 16..256).
__host__ __device__ constexpr uint32_t idesc_f16_m128(uint32_t n) {
  return (1u << 4)            // D format  = F32
         | (0u << 7)          // A format  = F16
         | (0u << 10)         // B format  = F16
         | ((n >> 3) << 17)   // N >> 3
         | ((128u >> 4) << 24);  // M >> 4
}

// Shared-memory matrix descriptor of a K-major operand stored as rows of 128
// bytes with the 128-byte swizzle (what a TMA box of 64 fp16 x rows with
// CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                  // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;          // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                  // descriptor version of sm_100
  d |= static_cast<uint64_t>(2) << 61;                  // SWIZZLE_128B
  return d;
}

// D[tmem] (+)= (A * SFA) * (B * SFB)^T, kind::mxf8f6f4 with one UE8M0 scale per 32
// elements of K for every row of A and of B; A and B from shared memory, scale
// factors from tensor memory, M = 128, K = 32 per instruction.
__device__ __forceinline__ void mma_mxf8f6f4_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                uint32_t accumulate, uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// Instruction descriptor, kind::mxf8f6f4 block scaled: A = e4m3, B = e2m1 (4-bit
// codes in 8-bit containers as the 16U4_ALIGN16B tensor map writes them), both
// K-major, UE8M0 scales, M = 128, N = n.  sf_id selects which of the four scale
// bytes of a tensor-memory column (which 32-wide k block of a 128-wide slice)
// the instruction applies, for A and for B.
__host__ __device__ constexpr uint32_t idesc_mxf8f6f4_m128(uint32_t n, uint32_t sf_id) {
  return (sf_id << 4)          // B scale-factor id
         | (0u << 7)           // A format = E4M3
         | (5u << 10)          // B format = E2M1
         | ((n >> 3) << 17)    // N >> 3
         | (1u << 23)          // scale format = UE8M0
         | ((128u >> 4) << 24) // M >> 4
         | (sf_id << 29);      // A scale-factor id
}

// Copies one 512-byte scale-factor atom (32 rows x 16 bytes, no swizzle) from
// shared memory into 4 tensor-memory columns, replicated into all four 32-lane
// quadrants.  Byte (r % 32) * 16 + (r / 32) * 4 + kb of the atom is the scale of
// row r, k block kb.  Issued by one thread; ordered before later tcgen05.mma of
// the same thread.
__device__ __forceinline__ void tmem_cp_sf_atom(uint32_t taddr, uint32_t saddr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);  // start address
  d |= static_cast<uint64_t>(128 >> 4) << 32;           // stride between 8-row groups: 8 x 16 bytes
  d |= static_cast<uint64_t>(1) << 46;                  // descriptor version of sm_100
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(d) : "memory");
}

// ---------------------------------------------------------------- MXFP4 decode
// Four bytes = eight e2m1 codes (low nibble = even element) -> four packed
// fp16 pairs, element order preserved (pair i = elements 2i, 2i+1).
__device__ __forceinline__ void cvt_e2m1x8_f16(uint32_t w, uint32_t (&h)[4]) {
  asm volatile(
      "{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
      : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
      : "r"(w));
}

// fp16x2 splat of 2^(e8m0 - 127).  Exact for exponents -24..15; below that the
// scale flushes to zero, above it saturates to 2^15 (the loader rejects tensors
// whose scaled values would leave the fp16 range, so neither branch is reached
// by accepted weights).
__device__ __forceinline__ uint32_t e8m0_to_f16x2(uint32_t sbyte) {
  const int e = static_cast<int>(sbyte) - 127;
  uint32_t bits;
  if (e >= -14) bits = static_cast<uint32_t>(min(e, 15) + 15) << 10;
  else if (e >= -24) bits = 1u << (e + 24);
  else bits = 0u;
  return bits | (bits << 16);
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

// 16 bytes of codes (32 elements, one scale block) -> 16 packed fp16 pairs.
__device__ __forceinline__ void dequant_block32(const uint4 &codes, uint32_t scale_f16x2, uint32_t (&out)[16]) {
  uint32_t h[4];
  cvt_e2m1x8_f16(codes.x, h);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[i] = hmul2_u32(h[i], scale_f16x2);
  cvt_e2m1x8_f16(codes.y, h);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[4 + i] = hmul2_u32(h[i], scale_f16x2);
  cvt_e2m1x8_f16(codes.z, h);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[8 + i] = hmul2_u32(h[i], scale_f16x2);
  cvt_e2m1x8_f16(codes.w, h);
#pragma unroll
  for (int i = 0; i < 4; ++i) out[12 + i] = hmul2_u32(h[i], scale_f16x2);
}

}  // namespace sm100
