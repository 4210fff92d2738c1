// Shared definitions of the b200q kernels: status codes, workspace layout, launch
// parameter blocks and small PTX helpers.
#pragma once
#include <cuda_bf16.h>
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
//                               words 1..3 = where it was raised; word 8 = arrival counter of a
//                               gather launch's CTAs; words 16, 17 = the counters of a launch that
//                               fetches its activations from host memory (all zero between launches)
// [256, 256 + cnt_bytes)      : int32 arrival counters, one per 16-column tile
// [256 + cnt_bytes, ...)      : fp32 split-K partial sums [M][N]
// Everything past the header must be zero when a GEMM starts; the kernels leave it zero.
constexpr size_t WS_HEADER_BYTES = 256;
inline size_t ws_counter_bytes(int N) { return (((size_t)(N / BLOCK_N) * 4) + 255) / 256 * 256; }

// ---- stream kernel (up to 16 rows per launch, the kernel for M <= 16): item-balanced, ring-fed --
// warps per CTA.  Up to 8 rows (MT = 1) two CTAs share an SM: 12 warps each leave up to 85 registers per
// thread (the loop uses 72), which keeps it out of local memory (16 warps at 64 registers spilled and
// measured 5-10 % slower; 10 and 14 warps were no better).  9..16 rows (MT = 2): one CTA has the SM.
constexpr int stream_warps(int mt) { return mt == 1 ? 12 : 16; }
// bytes of mbarriers in front of the rings: 8 slots of 8 bytes per warp, rounded up to 1 KB
constexpr int stream_header_bytes(int mt) { return (stream_warps(mt) * 64 + 1023) / 1024 * 1024; }
constexpr int STREAM_SC_GROUPS = 16;  // groups per warp in the shared-memory scale cache (32 bytes each)
// 128-row groups per ring item: items of 1..2 KB for every bit width
constexpr int stream_gi(int bits) { return bits <= 2 ? 4 : bits <= 5 ? 2 : 1; }
// Fused all-gather of a column-sharded GEMV (G == 0: none).  Every rank's launch stores its
// columns into the full output row of every rank and then raises its flag on every rank; the
// next launch waits for all flags before it reads its activations.  The call counter lives on
// the device (`epoch`), so a launch carries no per-call state and can be replayed from a graph.
//
// mode 1, tagged words: no flags.  The row buffers hold 8-byte words {two 16-bit outputs, call
// number}, three buffers per rank used in turn; a launch stores its columns as such words (one
// 64-bit store each: value and tag arrive together) into buffer (E + 1) % 3 of every rank, and the
// next launch polls the words it stages until each carries tag E + 1.  Nothing waits for a whole
// grid: the hand-over costs one store's flight time.  `out[g]` then points at 64-bit words and
// `buf_elems` counts words.
constexpr int GATHER_TAG_BUFFERS = 3;
struct GatherArgs {
  int G, rank;             // ranks, this rank
  int col_off;             // first column of this rank's shard in the full row
  int mode;                // 0: dense rows + flags; 1: tagged words (see above)
  __half* out[8];          // row buffer 0 of every rank (peer-mapped); buffer 1 is buf_elems further
  unsigned* flag_slot[8];  // this rank's slot in every rank's flag array (peer-mapped)
  const unsigned* flags;   // this rank's own flag array [G]
  unsigned* epoch;         // this rank's count of completed fused calls
  unsigned* done;          // arrival counter of this launch's CTAs (zero on entry, zero on exit)
  long long buf_elems;     // elements between a rank's two row buffers
  long long a_prev_off;    // >= 0: the activations are this rank's previous gathered output, from this element on
};

struct StreamParams {
  const __half* a;       // [M, K] row-major, leading dimension lda (16-bit elements: fp16 or bf16, see act)
  const void* bq;        // b200 layout
  const __half* scales;  // [K/group, N], 16-byte aligned
  __half* c;             // [M, N], leading dimension ldc
  float* partial;        // [N][8*MT] fp32, zero on entry, zero on exit
  int* counters;         // [N/16] arrived items per column tile, zero on entry, zero on exit
  int* status;           // workspace status header
  int M, N, K;
  int lda, ldc;
  int KB, NT;            // K/512, N/16
  int gshift, gdiv;      // scale row of 128-row group i: i >> gshift when gdiv = group / 128 is a power of two, else i / gdiv
  int S, KBc, CPC;       // k chunks, k blocks per chunk, CTAs per chunk; grid = S * CPC
  int T_own;             // whole column tiles per CTA (<= NT / CPC); the rest is shared item-wise
  int pitch;             // shared-memory row pitch of the activation chunk, in halfs
  int stages;            // ring slots per warp (<= 8)
  int pdl;               // launch with programmatic stream serialization
  int ipt_shift;         // log2 of the items per column tile inside a k chunk when that is a power of two, else -1
  int act;               // activation / scale / output dtype: 0 fp16, 1 bf16
  int trig;              // 1: CTA 0 lets the next kernel of the stream launch only after its own griddepcontrol.wait
  // Activations in pinned host memory (template value HOSTA of the kernel): the first `fetch_ctas` CTAs
  // read A from `a_host` (device-side address of the host rows, row stride lda) before they wait for the
  // previous kernel, store it to `a` (dense [M, K] staging on the device) afterwards and count themselves
  // in on `fetch_flag`; every CTA stages from `a` once the count is complete.  `fetch_flag[1]` counts the
  // CTAs that have seen it complete; the last of them puts both words back to zero.
  // Such a launch reads nothing the previous kernel of the stream wrote.  With one K chunk and no column
  // tiles shared between CTAs (`nowait`) it therefore does not wait for that kernel before its main loop,
  // only before it writes its outputs (so that outputs of consecutive calls land in order); and it lets
  // its own successor launch once all of its CTAs have staged their activations, i.e. once the staging
  // buffer is free again.  Consecutive host calls then overlap: the next one streams weights while this
  // one's results drain to the host.
  const __half* a_host;
  unsigned* fetch_flag;
  int fetch_ctas;
  int nowait;
  GatherArgs ga;
};

// ---- tcgen05 kernel with the weights in tensor memory (any M; used for M > 128) ----------------
struct UmmaParams {
  const uint4* bq;       // b200 layout
  const __half* scales;  // [K/group, N]
  __half* c;             // [M, N], leading dimension ldc
  float* partial;        // fp32 split-K scratch [tile slot][tm rows][128 columns], zero on entry and on exit
  int* counters;         // one per tile slot, zero on entry and on exit
  int* status;           // workspace status header
  int M, N, K, G;        // G = K / 128
  int ldc;
  int group;             // rows per scale: 32, 64 or a multiple of 128
  int rpg;               // scale rows per 128-row group: 128 / group for group < 128, else 1
  int tm;                // activation rows per CTA tile = N extent of the MMA (32, 64, 128 or 256)
  int m_tiles, n_tiles;  // ceil(M / tm), ceil(N / 128)
  int splits;            // split-K factor
  int kblocks_per_split; // 64-row k blocks per tile (even)
  int tail_tiles;        // the last tail_tiles tiles (raster order) are cut into tail_splits K ranges of
  int tail_splits;       // tail_kblocks 64-row blocks each (0 / 1 / all of K: no tail)
  int tail_kblocks;
  int a_stages;          // activation stages in shared memory
  int grid;              // persistent CTAs: min(tiles, SMs)
  int m_group;           // row tiles per raster group: tiles of m_group row tiles x all column tiles run together
  int act;               // activation / scale / output dtype: 0 fp16, 1 bf16
};

// ---- wide tcgen05 kernel (a few dozen rows): weights on the 256-column side of the MMA ---------
struct WideParams {
  const void* bq;        // b200 layout
  const __half* scales;  // [K/group, N]
  __half* c;             // [M, N], leading dimension ldc (multiple of 8)
  float* partial;        // [M, N] fp32 split-K scratch, zero on entry and on exit
  int* counters;         // [n_tiles * m_tiles], zero on entry and on exit
  int* status;           // workspace status header
  int M, N, K, G;        // G = K / 128
  int ldc;
  int group;             // rows per scale: 32, 64 or a multiple of 128
  int rpg;               // scale rows per 128-row group: 128 / group for group < 128, else 1
  int m_tiles, n_tiles;  // ceil(M / 128), ceil(N / 256)
  int splits;            // split-K factor
  int kblocks_per_split; // 64-row k blocks per work item (even)
  int wg_stages;         // packed 128-row weight groups in the shared-memory ring
  int a_rows;            // rows per activation copy: 32, 64 or 128
  int grid;              // persistent CTAs: min(work items, SMs)
  int act;               // activation / scale / output dtype: 0 fp16, 1 bf16
};

// ---- dequantize kernel -----------------------------------------------------------------------
struct DequantParams {
  const uint4* bq;
  const __half* scales;
  __half* w;  // [K, N] row-major (16-bit elements of the activation dtype)
  int N, K, group, G, NT;  // G = K / 128
  int act;    // 0 fp16, 1 bf16
};

// ---- per-token FP8 cast kernels ------------------------------------------------------------------
struct CastParams {
  const unsigned short* x;   // [T, H] (cast) or [T, 2H] (SwiGLU), row stride ldx elements, fp16 or bf16
  unsigned char* out;        // e4m3 [T, H], row stride ldo bytes
  float* out_sf;             // [T, H / group]
  int T, H, ldx, ldo, group;
  const int* pos_to_token_topk;  // [T] or null
  const float* topk_weights;     // flat, or null
  const int* pos_to_expert;      // [T] or null
  float clamp;
  int use_clamp;
};

// two fp32 values rounded to the activation dtype (ACT 0: fp16, 1: bf16), low half first
template <int ACT>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (ACT == 0) {
    return bits_from_h2(__floats2half2_rn(lo, hi));
  } else {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&b);
  }
}

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
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// same, first step of a chain: the accumulator input is zero
__device__ __forceinline__ void mma_m16n8k16_init(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ void red_add_v2(float* addr, float x, float y) {
  asm volatile("red.global.add.v2.f32 [%0], {%1, %2};" ::"l"(addr), "f"(x), "f"(y) : "memory");
}

// ---- shared-memory and mbarrier helpers of the mma.sync kernels ----------------------------------
// Waits on an mbarrier phase for at most about a quarter of a second; false when that ran out.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  uint64_t t0 = 0;
  for (int it = 0;; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 0x100000;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    if (ok) return true;
    uint64_t now;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
    if (it == 0) t0 = now;
    else if (now - t0 > 250000000ull) return false;
  }
}

__device__ __forceinline__ uint4 lds_u4(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
// the B words of one unit, from a shared-memory byte address
template <int B>
__device__ __forceinline__ void lds_unit_words(uint32_t addr, uint32_t (&w)[B]) {
  if constexpr (B % 4 == 0) {
#pragma unroll
    for (int q = 0; q < B / 4; ++q) {
      const uint4 v = lds_u4(addr + q * 16);
      w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
    }
  } else if constexpr (B % 2 == 0) {
#pragma unroll
    for (int q = 0; q < B / 2; ++q)
      asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(w[2 * q]), "=r"(w[2 * q + 1]) : "r"(addr + q * 8));
  } else {
#pragma unroll
    for (int q = 0; q < B; ++q) asm volatile("ld.shared.u32 %0, [%1];" : "=r"(w[q]) : "r"(addr + q * 4));
  }
}

}  // namespace b200q
