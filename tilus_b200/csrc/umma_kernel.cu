// Compute-bound path: C[M, N] = A[M, K] x dequant(Bq[K, N]) on the sm_100a tensor cores.
//
// The product is computed transposed, D[n, m] = sum_k W[k, n] * A[m, k], so that the
// dequantized weights are the operand that lives in tensor memory and the activations are
// the operand that TMA brings to shared memory.  A CTA is persistent: it walks over output
// tiles of 128 weight columns x TM activation rows (TM = 32 .. 256, the N extent of the MMA),
// each over all of K (or one of S splits of it), with the pipelines running across tile
// boundaries.  Warp roles:
//
//   * warp 17, weight producer: per 128-row group it brings the packed weights of the tile's
//     128 columns (eight 16-column pieces of 256*b contiguous bytes, cp.async.bulk) and their
//     128 fp16 scales into a 4-deep shared-memory ring;
//   * warps 0-7 dequantize.  Thread t of warp w is lane n = 32 * (w % 4) + t of tensor
//     memory.  For a block of 64 k it reads its column's 2 units (64 codes, 16*b contiguous
//     bytes) from the ring, decodes and scales them in registers with the unit decoder
//     (decode.cuh; the weights are fp16_rn(value * scale), exactly the values the reference
//     multiplies by, examples/quantization/matmul_a16wx.py:316-320) and writes the 32 half2
//     results to 32 columns of tensor memory with one tcgen05.st.  Warps 0-3 take the even
//     64-blocks, warps 4-7 the odd ones;
//   * warp 16, activation producer: one 2-D tiled TMA copy (128-byte swizzle) per 64-block
//     brings A[m0 : m0+TM, k : k+64] into a shared-memory ring; rows past M read as zero;
//   * warp 18 owns tensor memory (alloc / dealloc) and issues the MMAs: per 64-block four
//     tcgen05.mma.cta_group::1.kind::f16 (K = 16 each) with the weight operand in tensor
//     memory, the activation operand through a shared-memory descriptor and the fp32
//     accumulator D (128 lanes x TM columns) in tensor memory; tcgen05.commit releases the
//     activation stage and the weight stage when the MMAs have read them;
//   * warps 8-15, epilogue (two per lane quadrant, alternate 32-column chunks): when a tile's last
//     MMA has completed they read D with
//     tcgen05.ld, convert to fp16 and store C[m, n] (or add into the fp32 split-K scratch),
//     then hand D back.  Meanwhile the producers and the dequantizers are already working on
//     the next tile, so the tensor pipe restarts as soon as D is free.
//
// Every mbarrier wait is bounded in time; a wait that runs out raises a CTA-wide abort flag,
// all loops leave, tensor memory is still freed and the status word of the workspace reports
// it (the host reads it with b200q_device_status).
#include <cuda.h>

#include "common.cuh"
#include "umma_common.cuh"

#ifndef B200Q_PART
#define B200Q_PART 0
#endif
#ifndef B200Q_NPARTS
#define B200Q_NPARTS 1
#endif

namespace b200q {

constexpr int UMMA_THREADS = 608;   // 8 dequant warps, 8 epilogue warps, 2 producers, MMA warp
constexpr int UMMA_SA_MAX = 6;      // activation stages (most)
constexpr int UMMA_SW = 8;          // weight stages in tensor memory (32 columns each)
constexpr int UMMA_WG = 4;          // 128-row weight groups in the shared-memory ring
constexpr int UMMA_WCOL0 = 256;     // first tensor-memory column of the weight stages
constexpr int UMMA_TMEM_COLS = 512;

struct UmmaBarriers {
  uint64_t a_full[UMMA_SA_MAX], a_empty[UMMA_SA_MAX];
  uint64_t w_full[UMMA_SW], w_empty[UMMA_SW];
  uint64_t g_full[UMMA_WG], g_empty[UMMA_WG];
  uint64_t d_full, d_empty;
  uint32_t tmem_base;
  volatile int abort_flag;
  int last_flag;
};

// a ring stage: the packed weights of 128 columns x 128 rows, then rpg (1, 2 or 4) rows of 128 scales
__host__ __device__ constexpr int umma_wstage_bytes(int bits, int rpg) { return 2048 * bits + 256 * rpg; }

template <int VAR, int ACT>
__global__ void __launch_bounds__(UMMA_THREADS, 1)
umma_kernel(const UmmaParams p, const __grid_constant__ CUtensorMap tmap_a) {
  constexpr int B = var_bits(VAR);
  const uint32_t WSTAGE = (uint32_t)umma_wstage_bytes(B, p.rpg);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // [0, SA * TM * 128): activation stages (1024-byte aligned for the 128-byte swizzle: aligned
  // by hand), then the weight ring, then the barriers
  const uint32_t smem_unaligned = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t smem_base = (smem_unaligned + 1023u) & ~1023u;
  unsigned char* smem_al = smem_raw + (smem_base - smem_unaligned);
  const int TM = p.tm;
  const int SA = p.a_stages;
  const uint32_t stage_bytes = (uint32_t)TM * 128u;
  const uint32_t wring_s = smem_base + (uint32_t)SA * stage_bytes;
  const uint32_t bars_off = (uint32_t)SA * stage_bytes + UMMA_WG * WSTAGE;
  UmmaBarriers* bars = reinterpret_cast<UmmaBarriers*>(smem_al + bars_off);
  const uint32_t bars_s = smem_base + bars_off;
#define BAR_ADDR(field, i) (bars_s + (uint32_t)offsetof(UmmaBarriers, field) + (uint32_t)(i) * 8u)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // Work items.  The first splits * main_tiles items are the tiles 0 .. main_tiles-1 (raster order),
  // each over 1/splits of K.  The last tail_tiles tiles - what would be a thinly filled last round of
  // the persistent CTAs - are cut into tail_splits K ranges each, so that the round takes a fraction
  // of a tile's time; their partial sums meet in the fp32 scratch like any split-K tile.
  const int main_tiles = p.m_tiles * p.n_tiles - p.tail_tiles;
  const int main_items = p.splits * main_tiles;
  const int total_tiles = main_items + p.tail_splits * p.tail_tiles;  // work items of the launch
  volatile int* abort_flag = &bars->abort_flag;

  if (tid == 0) {
    for (int i = 0; i < UMMA_SA_MAX; ++i) { mbar_init(BAR_ADDR(a_full, i), 1); mbar_init(BAR_ADDR(a_empty, i), 1); }
    for (int i = 0; i < UMMA_SW; ++i) { mbar_init(BAR_ADDR(w_full, i), 4); mbar_init(BAR_ADDR(w_empty, i), 1); }
    for (int i = 0; i < UMMA_WG; ++i) { mbar_init(BAR_ADDR(g_full, i), 1); mbar_init(BAR_ADDR(g_empty, i), 8); }
    mbar_init(BAR_ADDR(d_full, 0), 1);
    mbar_init(BAR_ADDR(d_empty, 0), 8);
    bars->abort_flag = 0;
    bars->last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 18) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     bars_s + (uint32_t)offsetof(UmmaBarriers, tmem_base)),
                 "r"(UMMA_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = bars->tmem_base;

  // tile t -> (split, n_tile, m_tile).  Inside a split the row tiles are taken in groups of MG: all
  // column tiles of one group (row tile fastest) before the next group, so that the CTAs running
  // together share weight columns and the activation rows of one group stay in L2 while the weights
  // stream past them.  The last group holds the m_tiles % MG left-over row tiles.
  const int MG = p.m_group;
  const int full_group_tiles = (p.m_tiles / MG) * MG * p.n_tiles;
#define TILE_COORDS(t)                                                        \
  const bool in_tail = (t) >= main_items;                                     \
  const int t_rel = in_tail ? (t) - main_items : (t);                         \
  const int per = in_tail ? p.tail_tiles : main_tiles;                        \
  const int split = t_rel / per;                                              \
  const int t_in = t_rel - split * per + (in_tail ? main_tiles : 0);          \
  const int nkk = in_tail ? p.tail_kblocks : p.kblocks_per_split;             \
  const int ngrp = nkk >> 1;                                                  \
  const bool splitk = in_tail || p.splits > 1;                                \
  const bool in_full = t_in < full_group_tiles;                               \
  const int gsz = in_full ? MG : p.m_tiles % MG;                              \
  const int t_g = in_full ? t_in : t_in - full_group_tiles;                   \
  const int grp_i = in_full ? t_g / (MG * p.n_tiles) : p.m_tiles / MG;        \
  const int t_w = in_full ? t_g - grp_i * (MG * p.n_tiles) : t_g;             \
  const int n_tile = t_w / gsz;                                               \
  const int m_tile = grp_i * MG + (t_w - n_tile * gsz);                       \
  const int slot = in_tail ? t_in - main_tiles : n_tile * p.m_tiles + m_tile; \
  const int kk0 = split * nkk;                                                \
  const int m0 = m_tile * TM;                                                 \
  (void)m_tile; (void)n_tile; (void)split; (void)kk0; (void)m0; (void)ngrp; (void)splitk; (void)slot;

  if (warp < 8) {
    // ================= dequantize: shared-memory ring -> registers -> tensor memory =================
    const int grp = warp >> 2;              // 0: even 64-blocks, 1: odd ones
    const int nl = (warp & 3) * 32 + lane;  // lane of tensor memory = column inside the tile
    // this column inside a ring stage: 16-column piece nl / 16, then unit (half*32 + r*4 + j)
    const uint32_t lane_off = (uint32_t)((nl >> 4) * (256 * B) + (((nl >> 3) & 1) * 32 + (nl & 7) * 4 + grp * 2) * (B * 4));
    const uint32_t taddr_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + UMMA_WCOL0;
    int g_run = 0;  // groups consumed so far (all tiles)
    bool good = true;
    for (int t = blockIdx.x; t < total_tiles && good; t += gridDim.x) {
      TILE_COORDS(t)
      const bool nvalid = n_tile * 128 + nl < p.N;
      for (int g = 0; g < ngrp; ++g, ++g_run) {
        const int gs = g_run % UMMA_WG;
        if (!mbar_wait_abortable(BAR_ADDR(g_full, gs), (uint32_t)(g_run / UMMA_WG) & 1u, abort_flag)) { good = false; break; }
        uint32_t w[2 * B];
        const uint32_t st = wring_s + (uint32_t)gs * WSTAGE;
        lds_two_units<B>(st + lane_off, w);
        // the scales of this thread's two 32-row units: scale row (unit * rpg) / 4 of the stage
        unsigned short sb0, sb1;
        const uint32_t sc_s = st + 2048u * B + (uint32_t)nl * 2u;
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sb0) : "r"(sc_s + (uint32_t)(((2 * grp) * p.rpg) >> 2) * 256u));
        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sb1) : "r"(sc_s + (uint32_t)(((2 * grp + 1) * p.rpg) >> 2) * 256u));
        if (!nvalid) {
#pragma unroll
          for (int q = 0; q < 2 * B; ++q) w[q] = 0u;
          sb0 = 0; sb1 = 0;
        }
        uint32_t out[32];
        unit_decode_scaled<VAR, ACT>(w, (uint32_t)sb0 * 0x00010001u, out);  // the 16-bit scale in both halves
        unit_decode_scaled<VAR, ACT>(w + B, (uint32_t)sb1 * 0x00010001u, out + 16);
        // the ring stage has been read (its values fed the arithmetic above)
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_ADDR(g_empty, gs));
        const int wi = 2 * g_run + grp;  // running 64-block index
        const int sw = wi % UMMA_SW;
        if (!mbar_wait_abortable(BAR_ADDR(w_empty, sw), ((uint32_t)(wi / UMMA_SW) & 1u) ^ 1u, abort_flag)) { good = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t taddr = taddr_lane + (uint32_t)(sw * 32);
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
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_ADDR(w_full, sw));
      }
    }
  } else if (warp < 16) {
    // ================= epilogue: read D, write C (or add into the split-K scratch) =================
    // two warps per lane quadrant of tensor memory; they take alternate 32-column chunks of D
    const int ew = warp & 3;            // lane quadrant this warp may read
    const int chunk0 = (warp - 8) >> 2; // first chunk of this warp
    const int nl = ew * 32 + lane;
    const uint32_t daddr = tmem + ((uint32_t)(ew * 32) << 16);
    int tile_it = 0;
    bool good = true;
    // with several tiles per CTA the accumulator is handed back before the stores (the next tile's
    // MMAs run under them); a CTA with a single tile has nothing to overlap and takes the shorter path
    const bool many_items = total_tiles > (int)gridDim.x;
    for (int t = blockIdx.x; t < total_tiles && good; t += gridDim.x, ++tile_it) {
      TILE_COORDS(t)
      const int n = n_tile * 128 + nl;
      const bool nvalid = n < p.N;
      if (!mbar_wait_abortable(BAR_ADDR(d_full, 0), (uint32_t)tile_it & 1u, abort_flag)) { good = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (!splitk && many_items) {
        // Lane l holds column n of the tile, one accumulator row per tensor-memory column.  All of this
        // warp's 32-row chunks are read and rounded to the output dtype first (two rows per register)
        // and D is handed back at once, so that the next tile's MMAs run under the transposition and
        // the stores below.
        uint32_t hb[4][16];  // chunk ci, rows (2i, 2i+1) of column n
#pragma unroll
        for (int ci = 0; ci < 4; ++ci) {
          const int c0 = chunk0 * 32 + ci * 64;
          if (c0 < TM) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {  // 16 columns at a time: few registers live next to hb
              uint32_t v[16];
              tmem_ld_16(daddr + (uint32_t)(c0 + 16 * hh), v);
#pragma unroll
              for (int i = 0; i < 8; ++i)
                hb[ci][8 * hh + i] = pack2<ACT>(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            }
          }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(BAR_ADDR(d_empty, 0));
        // Three exchange rounds (lanes l ^ 1, l ^ 2, l ^ 4) transpose 8 x 8 blocks, so that a lane ends
        // with 8 consecutive columns of 4 rows and writes each as one 16-byte store.
        const bool b0 = lane & 1, b1 = lane & 2, b2 = lane & 4;
        const int n8 = n_tile * 128 + (nl & ~7);
#pragma unroll
        for (int ci = 0; ci < 4; ++ci) {
          const int c0 = chunk0 * 32 + ci * 64;
          if (c0 < TM && m0 + c0 < p.M) {
            uint32_t h[16];  // exchange 1: columns (n & ~1, +1), row 2 i + b0
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t got = __shfl_xor_sync(0xffffffffu, hb[ci][i], 1);
              // even lane: (own row 2i, partner's row 2i); odd lane: (partner's row 2i+1, own row 2i+1)
              h[i] = b0 ? __byte_perm(hb[ci][i], got, 0x3276) : __byte_perm(hb[ci][i], got, 0x5410);
            }
            uint32_t w2[8][2];  // exchange 2: columns (n & ~3 .. +3), row 4 j + 2 b1 + b0
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t mine = b1 ? h[2 * j + 1] : h[2 * j];
              const uint32_t give = b1 ? h[2 * j] : h[2 * j + 1];
              const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 2);
              w2[j][0] = b1 ? got : mine;
              w2[j][1] = b1 ? mine : got;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // exchange 3: columns (n & ~7 .. +7), row 8 k + (lane & 7)
              const uint32_t m0r = b2 ? w2[2 * k + 1][0] : w2[2 * k][0], m1r = b2 ? w2[2 * k + 1][1] : w2[2 * k][1];
              const uint32_t g0r = b2 ? w2[2 * k][0] : w2[2 * k + 1][0], g1r = b2 ? w2[2 * k][1] : w2[2 * k + 1][1];
              const uint32_t r0 = __shfl_xor_sync(0xffffffffu, g0r, 4), r1 = __shfl_xor_sync(0xffffffffu, g1r, 4);
              const int m = m0 + c0 + 8 * k + (lane & 7);
              if (m < p.M && n8 < p.N) {
                uint4 o;
                o.x = b2 ? r0 : m0r; o.y = b2 ? r1 : m1r; o.z = b2 ? m0r : r0; o.w = b2 ? m1r : r1;
                *reinterpret_cast<uint4*>(p.c + (size_t)m * p.ldc + n8) = o;
              }
            }
          }
        }
      } else {
        if (chunk0 * 32 >= TM) {  // nothing of this tile is this warp's (TM = 32): hand D back at once
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR_ADDR(d_empty, 0));
        }
        for (int c0 = chunk0 * 32; c0 < TM; c0 += 64) {
          uint32_t v[32];
          tmem_ld_32(daddr + (uint32_t)c0, v);
          if (c0 + 64 >= TM) {
            // this warp's last chunk of D is in registers: the next tile's MMAs may overwrite it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(BAR_ADDR(d_empty, 0));
          }
          if (m0 + c0 < p.M && !splitk) {
            const bool b0 = lane & 1, b1 = lane & 2, b2 = lane & 4;
            uint32_t h[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const uint32_t mine = b0 ? v[2 * i + 1] : v[2 * i];
              const uint32_t give = b0 ? v[2 * i] : v[2 * i + 1];
              const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 1);
              h[i] = pack2<ACT>(__uint_as_float(b0 ? got : mine), __uint_as_float(b0 ? mine : got));
            }
            uint32_t w2[8][2];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const uint32_t mine = b1 ? h[2 * j + 1] : h[2 * j];
              const uint32_t give = b1 ? h[2 * j] : h[2 * j + 1];
              const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 2);
              w2[j][0] = b1 ? got : mine;
              w2[j][1] = b1 ? mine : got;
            }
            const int n8 = n_tile * 128 + (nl & ~7);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const uint32_t m0r = b2 ? w2[2 * k + 1][0] : w2[2 * k][0], m1r = b2 ? w2[2 * k + 1][1] : w2[2 * k][1];
              const uint32_t g0r = b2 ? w2[2 * k][0] : w2[2 * k + 1][0], g1r = b2 ? w2[2 * k][1] : w2[2 * k + 1][1];
              const uint32_t r0 = __shfl_xor_sync(0xffffffffu, g0r, 4), r1 = __shfl_xor_sync(0xffffffffu, g1r, 4);
              const int m = m0 + c0 + 8 * k + (lane & 7);
              if (m < p.M && n8 < p.N) {
                uint4 o;
                o.x = b2 ? r0 : m0r; o.y = b2 ? r1 : m1r; o.z = b2 ? m0r : r0; o.w = b2 ? m1r : r1;
                *reinterpret_cast<uint4*>(p.c + (size_t)m * p.ldc + n8) = o;
              }
            }
          } else if (m0 + c0 < p.M) {
            // split-K: lanes 2i and 2i+1 exchange so that each adds two columns (8 bytes) of a row
            const bool odd = lane & 1;
#pragma unroll
            for (int q = 0; q < 32; q += 2) {
              const uint32_t mine = odd ? v[q + 1] : v[q];      // row q + odd, own column
              const uint32_t give = odd ? v[q] : v[q + 1];      // row q + !odd, own column
              const uint32_t got = __shfl_xor_sync(0xffffffffu, give, 1);  // row q + odd, the other column
              const float lo = __uint_as_float(odd ? got : mine), hi = __uint_as_float(odd ? mine : got);
              const int mr = c0 + q + (odd ? 1 : 0);  // row inside the tile
              const int ne = n & ~1;
              if (m0 + mr < p.M && ne < p.N)
                red_add_v2(p.partial + ((size_t)slot * TM + mr) * 128 + (nl & ~1), lo, hi);
            }
          }
        }
      }
      (void)nvalid;
      if (splitk) {
        // the last K range to arrive converts the tile's fp32 sums (kept per tile slot: [slot][row][128
        // columns]) and restores the zeros
        const int nsplit = in_tail ? p.tail_splits : p.splits;
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (warp == 8 && lane == 0) {
          __threadfence();
          const int old = atomicAdd(p.counters + slot, 1);
          const int last = (old + 1 == nsplit) ? 1 : 0;
          if (last) __threadfence();
          bars->last_flag = last;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");
        if (bars->last_flag) {
          // eight independent loads per thread in flight: one L2 round trip per batch, not per load
          float* tile_sums = p.partial + (size_t)slot * TM * 128;
          for (int base = tid - 256; base < 64 * TM; base += 8 * 256) {
            float2 x[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int idx = base + u * 256;
              const int nn = n_tile * 128 + (idx & 63) * 2, m = m0 + (idx >> 6);
              if (idx < 64 * TM && nn < p.N && m < p.M)
                x[u] = __ldcg(reinterpret_cast<const float2*>(tile_sums + (size_t)idx * 2));
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int idx = base + u * 256;
              const int nn = n_tile * 128 + (idx & 63) * 2, m = m0 + (idx >> 6);
              if (idx < 64 * TM && nn < p.N && m < p.M) {
                *reinterpret_cast<uint32_t*>(p.c + (size_t)m * p.ldc + nn) = pack2<ACT>(x[u].x, x[u].y);
                __stcg(reinterpret_cast<float2*>(tile_sums + (size_t)idx * 2), make_float2(0.f, 0.f));
              }
            }
          }
          if (warp == 8 && lane == 0) p.counters[slot] = 0;
        }
        asm volatile("bar.sync 1, 256;" ::: "memory");  // last_flag may be rewritten by the next item
      }
    }
  } else if (warp == 16) {
    // ================= TMA producer: activations =================
    if (lane == 0) {
      int ai = 0;
      bool good = true;
      for (int t = blockIdx.x; t < total_tiles && good; t += gridDim.x) {
        TILE_COORDS(t)
        for (int i = 0; i < nkk; ++i, ++ai) {
          const int sa = ai % SA;
          if (!mbar_wait_abortable(BAR_ADDR(a_empty, sa), ((uint32_t)(ai / SA) & 1u) ^ 1u, abort_flag)) { good = false; break; }
          const uint32_t bar = BAR_ADDR(a_full, sa);
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(stage_bytes)
                       : "memory");
          const int kx = (kk0 + i) * 64;
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
              ::"r"(smem_base + (uint32_t)sa * stage_bytes), "l"(&tmap_a), "r"(bar), "r"(kx), "r"(m0)
              : "memory");
        }
      }
    }
  } else if (warp == 17) {
    // ================= bulk-copy producer: packed weights and scales =================
    int g_run = 0;
    bool good = true;
    const unsigned char* bq = reinterpret_cast<const unsigned char*>(p.bq);
    for (int t = blockIdx.x; t < total_tiles && good; t += gridDim.x) {
      TILE_COORDS(t)
      const int nt0 = n_tile * 8;
      const int pieces = min(8, p.N / BLOCK_N - nt0);  // 16-column pieces of this tile that exist
      for (int g = 0; g < ngrp; ++g, ++g_run) {
        const int gs = g_run % UMMA_WG;
        int ok = 1;
        if (lane == 0) ok = mbar_wait_abortable(BAR_ADDR(g_empty, gs), ((uint32_t)(g_run / UMMA_WG) & 1u) ^ 1u, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { good = false; break; }
        const uint32_t bar = BAR_ADDR(g_full, gs);
        const uint32_t dst = wring_s + (uint32_t)gs * WSTAGE;
        if (lane == 0)
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                       "r"((uint32_t)pieces * (256u * B + 32u * (uint32_t)p.rpg))
                       : "memory");
        __syncwarp();
        const int G = (kk0 >> 1) + g;  // 128-row group of K
        if (lane < pieces) {
          const unsigned char* src = bq + ((size_t)(nt0 + lane) * p.G + G) * (size_t)(256 * B);
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                  dst + (uint32_t)lane * (256u * B)),
              "l"(src), "r"(256u * B), "r"(bar)
              : "memory");
        } else if (lane >= 8 && lane < 8 + p.rpg) {
          // scale row(s) of the group: one per 128 / rpg rows
          const int row = p.rpg == 1 ? (G * 128) / p.group : G * p.rpg + (lane - 8);
          const __half* src = p.scales + (size_t)row * p.N + n_tile * 128;
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                  dst + 2048u * B + (uint32_t)(lane - 8) * 256u),
              "l"(src), "r"((uint32_t)pieces * 32u), "r"(bar)
              : "memory");
        }
      }
    }
  } else {
    // ================= MMA issuer =================
    if (lane == 0) {
      const uint32_t idesc = umma_idesc<ACT>(TM);
      bool good = true;
      int ai = 0, tile_it = 0;
      for (int t = blockIdx.x; t < total_tiles && good; t += gridDim.x, ++tile_it) {
        TILE_COORDS(t)
        // D must have been read out by the epilogue of the previous tile
        if (!mbar_wait_abortable(BAR_ADDR(d_empty, 0), ((uint32_t)tile_it & 1u) ^ 1u, abort_flag)) { good = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        for (int i = 0; i < nkk; ++i, ++ai) {
          const int sa = ai % SA, sw = ai % UMMA_SW;
          good = mbar_wait_abortable(BAR_ADDR(a_full, sa), (uint32_t)(ai / SA) & 1u, abort_flag) &&
                 mbar_wait_abortable(BAR_ADDR(w_full, sw), (uint32_t)(ai / UMMA_SW) & 1u, abort_flag);
          if (!good) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t bdesc = umma_smem_desc(smem_base + (uint32_t)sa * stage_bytes);
          const uint32_t a_tmem = tmem + UMMA_WCOL0 + (uint32_t)(sw * 32);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t accumulate = (i > 0 || ks > 0) ? 1u : 0u;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "setp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                ::"r"(tmem), "r"(a_tmem + (uint32_t)(ks * 8)), "l"(bdesc + (uint64_t)(ks * 2)), "r"(idesc),
                "r"(accumulate)
                : "memory");
          }
          // the stages may be overwritten once these MMAs have read them
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           BAR_ADDR(a_empty, sa))
                       : "memory");
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           BAR_ADDR(w_empty, sw))
                       : "memory");
        }
        if (good)
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           BAR_ADDR(d_full, 0))
                       : "memory");
      }
    }
  }

  // ================= teardown =================
  __syncwarp();
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag && tid == 0) {
    atomicExch(p.status, ST_DEVICE_TIMEOUT);
    p.status[1] = 2;  // where: tcgen05 kernel pipeline
    p.status[2] = blockIdx.x;
    p.status[3] = 0;
  }
  if (warp == 18) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(UMMA_TMEM_COLS) : "memory");
  }
#undef BAR_ADDR
#undef TILE_COORDS
}

template <int VAR, int ACT>
static cudaError_t umma_launch_one(const UmmaParams& p, const CUtensorMap& tmap, int smem_bytes,
                                   cudaStream_t stream) {
  auto kern = umma_kernel<VAR, ACT>;
  static int configured_smem[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || configured_smem[dev] < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 16) configured_smem[dev] = smem_bytes;
  }
  kern<<<p.grid, UMMA_THREADS, smem_bytes, stream>>>(p, tmap);
  return cudaGetLastError();
}

template <int VAR>
static cudaError_t umma_launch_var(int var, const UmmaParams& p, const CUtensorMap& tmap, int smem_bytes,
                                   cudaStream_t stream) {
  if constexpr (VAR % B200Q_NPARTS == B200Q_PART) {
    if (var == VAR)
      return p.act == 0 ? umma_launch_one<VAR, 0>(p, tmap, smem_bytes, stream)
                        : umma_launch_one<VAR, 1>(p, tmap, smem_bytes, stream);
  }
  if constexpr (VAR + 1 < VAR_COUNT) return umma_launch_var<VAR + 1>(var, p, tmap, smem_bytes, stream);
  else return cudaErrorInvalidValue;
}

#define B200Q_CAT2(a, b) a##b
#define B200Q_CAT(a, b) B200Q_CAT2(a, b)

// One of these per compiled part; api.cu picks the part as var % B200Q_NPARTS.
cudaError_t B200Q_CAT(umma_launch_part, B200Q_PART)(int var, const UmmaParams& p, const void* tmap, int smem_bytes,
                                                    cudaStream_t stream) {
  return umma_launch_var<0>(var, p, *reinterpret_cast<const CUtensorMap*>(tmap), smem_bytes, stream);
}

#if B200Q_PART == 0
// dynamic shared memory: alignment slack + activation stages + weight ring + barriers
int umma_smem_bytes(int tm, int bits, int a_stages, int rpg) {
  return 1024 + a_stages * tm * 128 + UMMA_WG * umma_wstage_bytes(bits, rpg) + (int)sizeof(UmmaBarriers) + 64;
}
// most activation stages (<= UMMA_SA_MAX) that fit next to the weight ring
int umma_a_stages(int tm, int bits, int max_smem, int rpg) {
  int sa = UMMA_SA_MAX;
  while (sa > 2 && umma_smem_bytes(tm, bits, sa, rpg) > max_smem) --sa;
  return sa;
}
#endif

}  // namespace b200q
