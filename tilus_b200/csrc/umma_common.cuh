// Helpers shared by the tcgen05 kernels: bounded mbarrier waits with a CTA-wide abort flag,
// shared-memory / instruction descriptors of tcgen05.mma, tensor-memory loads and stores.
#pragma once
#include "common.cuh"

namespace b200q {

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait (about a quarter of a second); also gives up as soon as another thread raised the abort flag
__device__ __forceinline__ bool mbar_wait_abortable(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  uint64_t t0 = 0;
  for (int it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 0x10000;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    if (*abort_flag) return false;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (it == 0) t0 = now;
    else if (now - t0 > 250000000ull) { *abort_flag = 1; return false; }
  }
}

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 64 fp16
// (128 bytes), 8-row groups 1024 bytes apart (stride byte offset), descriptor version 1
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= (uint64_t)1 << 46;                        // version
  d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
  return d;
}
// instruction descriptor of kind::f16: D fp32 (bit 4), A and B formats (bits 7-9 and 10-12: 0 fp16,
// 1 bf16), both K-major, N = n (bits 17-22, in units of 8), M = 128 (bits 24-28, in units of 16)
template <int ACT>
__device__ __forceinline__ uint32_t umma_idesc(int n) {
  return (1u << 4) | ((uint32_t)ACT << 7) | ((uint32_t)ACT << 10) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(128 >> 4) << 24);
}

// the 2*B words of two consecutive units, from a shared-memory byte address (8-byte aligned;
// 16-byte aligned when B is even)
template <int B>
__device__ __forceinline__ void lds_two_units(uint32_t addr, uint32_t (&w)[2 * B]) {
  if constexpr (B % 2 == 0) {
#pragma unroll
    for (int q = 0; q < B / 2; ++q) {
      const uint4 v = lds_u4(addr + q * 16);
      w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
    }
  } else {
#pragma unroll
    for (int q = 0; q < B; ++q)
      asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[2 * q]), "=r"(w[2 * q + 1]) : "r"(addr + q * 8));
  }
}

// 32 consecutive tensor-memory columns of this thread's lane -> 32 registers (waits for the data)
__device__ __forceinline__ void tmem_ld_32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
        "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
        "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
        "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 16 consecutive tensor-memory columns of this thread's lane -> 16 registers (waits for the data)
__device__ __forceinline__ void tmem_ld_16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// 32 registers -> 32 consecutive tensor-memory columns of this thread's lane
__device__ __forceinline__ void tmem_st_32(uint32_t taddr, const uint32_t (&out)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(out[0]), "r"(out[1]), "r"(out[2]), "r"(out[3]), "r"(out[4]), "r"(out[5]), "r"(out[6]), "r"(out[7]),
      "r"(out[8]), "r"(out[9]), "r"(out[10]), "r"(out[11]), "r"(out[12]), "r"(out[13]), "r"(out[14]),
      "r"(out[15]), "r"(out[16]), "r"(out[17]), "r"(out[18]), "r"(out[19]), "r"(out[20]), "r"(out[21]),
      "r"(out[22]), "r"(out[23]), "r"(out[24]), "r"(out[25]), "r"(out[26]), "r"(out[27]), "r"(out[28]),
      "r"(out[29]), "r"(out[30]), "r"(out[31])
      : "memory");
}
}  // namespace b200q
