// Device-side building blocks shared by the tensor-core kernels: mbarrier / TMA / tcgen05 wrappers,
// shared-memory descriptors, the swizzled staging panel, and the packed requantisation.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "common.cuh"

namespace cvmk {
namespace tc {

constexpr int BLOCK_M = 128;
constexpr uint32_t SPIN_LIMIT = 1u << 19;  // x 2 us per hardware wait
#ifdef CVMK_CONV_TIMING
__device__ uint32_t g_wait_hint = 2000u;  // development builds: suspend-time hint of the waits, settable
#endif

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// True on exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "elect.sync _|p, 0xffffffff;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One bounded hardware wait: returns true once the phase with `parity` has completed, false if
// the barrier is still pending after about `ns` nanoseconds.
__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Non-blocking: true if the phase with `parity` has completed.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait (about a second in all).  Returns false when it gave up, or when another role of
// this CTA already did.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int code, uint32_t limit = SPIN_LIMIT) {
  for (uint32_t i = 0; i < limit; ++i) {
#ifdef CVMK_CONV_TIMING
    if (mbar_try(bar, parity, g_wait_hint)) return true;
#else
    if (mbar_try(bar, parity, 2000u)) return true;
#endif
    if (*abort_flag) return false;
  }
  *abort_flag = code;
  return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_im2col_4d(void* dst, const CUtensorMap* map, uint64_t* bar,
                                                   int c, int w, int h, int n, uint16_t off_w,
                                                   uint16_t off_h) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.im2col.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], {%7, %8};" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c), "r"(w), "r"(h), "r"(n),
      "h"(off_w), "h"(off_h)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(slot)),
               "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// NK back-to-back instructions over K slices 32 bytes apart (descriptor address units of 16
// bytes: +2 each).  The descriptors come as 32-bit halves: only the low word (start address)
// changes from instruction to instruction, so the issuing thread spends one 32-bit add per
// operand and instruction.  That matters: the issuing warp shares its scheduler with epilogue
// warps, and every instruction of its loop waits its turn.
template <int NK>
__device__ __forceinline__ void mma_i8_k(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                         uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 da, db;\n"
      "setp.ne.b32 p, %6, 0;\n"
      "mov.b64 da, {%1, %2};\n"
      "mov.b64 db, {%3, %4};\n"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
#pragma unroll
  for (int j = 1; j < NK; ++j) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        ".reg .b64 da, db;\n"
        "setp.eq.b32 p, 0, 0;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n"
        "}\n" ::"r"(d_tmem),
        "r"(a_lo + 2u * (uint32_t)j), "r"(a_hi), "r"(b_lo + 2u * (uint32_t)j), "r"(b_hi), "r"(idesc)
        : "memory");
  }
}
// Arrive on `bar` once every tcgen05.mma issued so far by this thread has finished.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, int32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]),
        "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]),
        "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]),
        "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
        "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Two adjacent 32-column chunks with one wait: both loads are in flight together, so a row of the
// epilogue pays the TMEM latency once per 64 columns.
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, int32_t (&a)[32], int32_t (&b)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%64];\n"
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, %48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%65];\n"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]), "=r"(a[4]), "=r"(a[5]), "=r"(a[6]), "=r"(a[7]), "=r"(a[8]), "=r"(a[9]), "=r"(a[10]), "=r"(a[11]), "=r"(a[12]), "=r"(a[13]), "=r"(a[14]), "=r"(a[15]), "=r"(a[16]), "=r"(a[17]), "=r"(a[18]), "=r"(a[19]), "=r"(a[20]), "=r"(a[21]), "=r"(a[22]), "=r"(a[23]), "=r"(a[24]), "=r"(a[25]), "=r"(a[26]), "=r"(a[27]), "=r"(a[28]), "=r"(a[29]), "=r"(a[30]), "=r"(a[31]),
        "=r"(b[0]), "=r"(b[1]), "=r"(b[2]), "=r"(b[3]), "=r"(b[4]), "=r"(b[5]), "=r"(b[6]), "=r"(b[7]), "=r"(b[8]), "=r"(b[9]), "=r"(b[10]), "=r"(b[11]), "=r"(b[12]), "=r"(b[13]), "=r"(b[14]), "=r"(b[15]), "=r"(b[16]), "=r"(b[17]), "=r"(b[18]), "=r"(b[19]), "=r"(b[20]), "=r"(b[21]), "=r"(b[22]), "=r"(b[23]), "=r"(b[24]), "=r"(b[25]), "=r"(b[26]), "=r"(b[27]), "=r"(b[28]), "=r"(b[29]), "=r"(b[30]), "=r"(b[31])
      : "r"(taddr), "r"(taddr + 32u)
      : "memory");
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are `row_bytes` long
// (32, 64 or 128) and stored with the matching TMA swizzle: 8-row groups are 8 * row_bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, int row_bytes) {
  const uint64_t layout = row_bytes == 128 ? 2 : (row_bytes == 64 ? 4 : 6);
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)1 << 16;                                  // leading byte offset (unused) = 16 B
  d |= (uint64_t)((8u * (uint32_t)row_bytes) >> 4) << 32;  // stride byte offset
  d |= (uint64_t)1 << 46;                                  // descriptor version (sm_100)
  d |= layout << 61;
  return d;
}
// Instruction descriptor: s8 x s8 -> s32, both operands K-major, M = 128, N = block_n.
__device__ __forceinline__ uint32_t umma_idesc_i8(int n) {
  return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(BLOCK_M >> 4) << 24);
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* src, int c0, int c1,
                                             int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Byte offset of 16-byte chunk `j` of row `row` inside a staging panel whose rows are `pw` bytes
// long and stored with the TMA swizzle of that width (address bits [4,7) ^= bits [7,10), cut to
// the width).
__device__ __forceinline__ uint32_t panel_offset(int row, int j, int pw) {
  const uint32_t lin = (uint32_t)row * (uint32_t)pw + (uint32_t)j * 16u;
  const uint32_t mask = ((uint32_t)pw - 1u) >> 4;  // 7, 3 or 1 chunks
  return lin ^ (((lin >> 7) & mask) << 4);
}

// Byte permute with the full selector semantics of the instruction: a selector nibble with its top
// bit set replicates the sign of the chosen byte (the __byte_perm() intrinsic documents only the low
// three bits of each nibble).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

// Clamp bounds of the packed requantisation, each replicated into both halves of an s16x2 word.
struct FastQ {
  uint32_t f_lo1, f_hi1;  // first clamp
  uint32_t f_lo2, f_hi2;  // clamp after the tensor step
};

// Requantisation of 32 accumulators to int8 when the caller has proven that the biased sums cannot
// overflow and fit 16 bits after the shift:  t = (acc + bias + 2^(s-1)) >> s  is computed in 32
// bits, then pairs are packed into s16x2 words and everything else runs two elements per
// instruction: clamp, the add / subtract of the int8 tensor operand (sign-extended by a byte
// permute), the final clamp (one fused add-min-relu when its lower bound is 0), and the pack to
// bytes.  Same values as the step-by-step chain: every clamp commutes with the monotone shift, and
// all intermediate values are exact in 16 bits.
// RELU1: the first clamp has lower bound 0.  KIND: 0 no tensor step, 1 add with a final clamp whose
// lower bound is 0, 2 add with a general clamp, 3 subtract with a general clamp.  All of it is
// resolved at compile time so that the 32 columns form one straight-line block.
template <int RELU1, int KIND>
__device__ __forceinline__ void fast_requant(const FastQ& p, const int32_t (&v)[32], const uint4& r0,
                                             const uint4& r1, uint4* o0, uint4* o1) {
  uint32_t h[16];
  const uint32_t hi1 = p.f_hi1, lo1 = p.f_lo1, hi2 = p.f_hi2, lo2 = p.f_lo2;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    h[j] = __byte_perm((uint32_t)v[2 * j], (uint32_t)v[2 * j + 1], 0x7632);  // the two upper halves
    if (RELU1) h[j] = __vimin_s16x2_relu(h[j], hi1);
    else h[j] = __vmaxs2(__vmins2(h[j], hi1), lo1);
  }
  if (KIND != 0) {
    const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const uint32_t ra = prmt(rw[q], 0, 0x9180);  // bytes 0,1 sign-extended to 16 bits
      const uint32_t rb = prmt(rw[q], 0, 0xB3A2);  // bytes 2,3
      if (KIND == 1) {
        h[2 * q] = __viaddmin_s16x2_relu(h[2 * q], ra, hi2);
        h[2 * q + 1] = __viaddmin_s16x2_relu(h[2 * q + 1], rb, hi2);
      } else {
        const uint32_t xa = KIND == 3 ? __vsub2(h[2 * q], ra) : __vadd2(h[2 * q], ra);
        const uint32_t xb = KIND == 3 ? __vsub2(h[2 * q + 1], rb) : __vadd2(h[2 * q + 1], rb);
        h[2 * q] = __vmaxs2(__vmins2(xa, hi2), lo2);
        h[2 * q + 1] = __vmaxs2(__vmins2(xb, hi2), lo2);
      }
    }
  }
  uint32_t w[8];
#pragma unroll
  for (int q = 0; q < 8; ++q) w[q] = __byte_perm(h[2 * q], h[2 * q + 1], 0x6420);
  *o0 = make_uint4(w[0], w[1], w[2], w[3]);
  *o1 = make_uint4(w[4], w[5], w[6], w[7]);
}

}  // namespace tc
}  // namespace cvmk
