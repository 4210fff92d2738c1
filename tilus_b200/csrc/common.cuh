// Shared definitions of the b200q kernels: status codes, workspace layout, launch
// parameter blocks and small PTX helpers.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "decode.cuh"

namespace b200q {

// ---- status codes (also returned through the C ABI) -------------------------------------
enum : int {
  ST_OK = 0,
  ST_INVALID_ARG = 1,     // null pointer, non-positive size, misaligned pointer
  ST_UNSUPPORTED = 2,     // shape / dtype / group size outside what the kernels cover
  ST_WORKSPACE = 3,       // workspace missing or too small
  ST_CUDA = 4,            // a CUDA runtime call failed (see b200q_last_cuda_error)
  ST_DEVICE_TIMEOUT = 5,  // a bounded device-side wait ran out (see b200q_device_status)
};

// ---- weight layout constants (tilus_b200/packing.py) --------------------------------------
constexpr int BLOCK_N = 16;
constexpr int BLOCK_K = 512;

// ---- workspace -----------------------------------------------------------------------------
// [0, 256)                    : status header, int32[64]; word 0 = device error code,
//                               words 1..3 = where it was raised
// [256, 256 + cnt_bytes)      : int32 arrival counters, one per 16-column tile
// [256 + cnt_bytes, ...)      : fp32 split-K partial sums [M][N]
// Everything past the header must be zero when a GEMM starts; the kernels leave it zero.
constexpr size_t WS_HEADER_BYTES = 256;
inline size_t ws_counter_bytes(int N) { return (((size_t)(N / BLOCK_N) * 4) + 255) / 256 * 256; }

// ---- skinny (M <= 16 per launch) split-K kernel ---------------------------------------------
struct SkinnyParams {
  const __half* a;       // [M, K] row-major, leading dimension lda
  const uint4* bq;       // b200 layout
  const __half* scales;  // [K/group, N]
  __half* c;             // [M, N], leading dimension ldc
  float* partial;        // [M, N] fp32, zero on entry, zero on exit
  int* counters;         // [N/16], zero on entry, zero on exit
  int M, N, K, group;
  int gshift;            // log2(group / 128), or -1 when there is one group per column (group == K)
  int lda, ldc;
  int KB, NT;            // K/512, N/16
  int GS, CS, P, KBc;    // global k splits, cluster size (k splits inside a cluster), column ranges,
                         // k-blocks per CTA (K/512 / (GS*CS))
  int tiles_max;         // most column tiles any cluster owns: ceil(NT / P)
  int pitch;             // shared-memory row pitch of the activation chunk, in halfs
  int stages;            // items in flight per warp (<= 8)
  int* status;           // workspace status header
  int debug_skip;        // diagnosis: 1 stream the weights but skip the math, 2 skip the loop, 3 and the staging
  int pdl;               // launch with programmatic stream serialization
};

// ---- tcgen05 kernel (any M; used for M > 16) ---------------------------------------------------
struct UmmaParams {
  const uint4* bq;       // b200 layout
  const __half* scales;  // [K/group, N]
  __half* c;             // [M, N], leading dimension ldc
  float* partial;        // [M, N] fp32 split-K scratch, zero on entry and on exit
  int* counters;         // [n_tiles * m_tiles], zero on entry and on exit
  int* status;           // workspace status header
  int M, N, K, KB;       // KB = K / 512
  int ldc;
  int gshift;            // log2(group / 128), or -1 when group == K
  int tm;                // activation rows per CTA tile = N extent of the MMA (32, 64, 128 or 256)
  int m_tiles, n_tiles;  // ceil(M / tm), ceil(N / 128)
  int splits;            // split-K factor
  int kblocks_per_split; // 64-row k blocks per CTA
};

// ---- dequantize kernel -----------------------------------------------------------------------
struct DequantParams {
  const uint4* bq;
  const __half* scales;
  __half* w;  // [K, N] row-major
  int N, K, group, KB, NT;
};

__device__ __forceinline__ uint4 ld_stream_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

__device__ __forceinline__ uint32_t u4_comp(const uint4& v, int c) {
  return c == 0 ? v.x : c == 1 ? v.y : c == 2 ? v.z : v.w;
}

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// same, first step of a chain: the accumulator input is zero
__device__ __forceinline__ void mma_m16n8k16_init(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

}  // namespace b200q
