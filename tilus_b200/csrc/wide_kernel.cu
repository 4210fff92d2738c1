// Batches of a few dozen rows: C[M<=128 per tile, N] = A[M, K] x dequant(Bq[K, N]) on tcgen05 with
// the weights on the wide side of the instruction.
//
// A tcgen05.mma with 128 rows costs about 170 cycles whatever its column count (measured for N = 16,
// 64 and 256), so for small M the product is bound by the number of instructions per weight.  This
// kernel therefore computes D[m, n] = sum_k A[m, k] * W[k, n] with M = 128 activation rows (rows
// past the batch are zero-filled by TMA and cost nothing to fetch) and N = 256 weight columns per
// instruction - twice the weights per instruction of the transposed form used for prefill
// (umma_kernel.cu), and one decode per weight shared by all rows of the batch:
//
//   * warp 21 brings the packed weights of the tile's 256 columns, one 128-row group at a time
//     (sixteen 16-column pieces of 256*b contiguous bytes, cp.async.bulk) and their 256 fp16
//     scales into a shared-memory ring;
//   * warps 0-15 dequantize, in two sets of eight that take alternate 128-row groups: thread t is
//     column n = t % 256 of the tile; per 64-row block it reads its column's 2 units (64 codes) from the
//     ring, decodes and scales them in registers
//     (decode.cuh, unit_decode_scaled: fp16_rn(value * scale), exactly the values the reference
//     multiplies by, examples/quantization/matmul_a16wx.py:316-320) and stores the 64 halfs as
//     row n of the K-major, 128-byte-swizzled B operand tile in shared memory (8 x 16 bytes);
//   * warp 20 brings A[m0 : m0+128, k : k+64] with one 2-D tiled TMA copy per block;
//   * warp 22 owns tensor memory and issues 4 x tcgen05.mma.cta_group::1.kind::f16 per block
//     (M = 128, N = 256, K = 16, both operands through shared-memory descriptors), fp32
//     accumulators 128 lanes x 256 columns, two of them so that the epilogue of one tile runs
//     under the MMAs of the next;
//   * warps 16-19 read the accumulator (lane = activation row, 32 columns = 32 consecutive output
//     columns per tcgen05.ld) and store 64-byte row segments of C, or add into the fp32 split-K
//     scratch (red.global.add.v4.f32); the last split to arrive converts and restores the zeros.
//
// Persistent CTAs walk over (split, column tile, row tile) work items.  Every mbarrier wait is
// bounded in time; a wait that runs out raises a CTA-wide abort flag, all loops leave, tensor
// memory is still freed and the status word of the workspace reports it.
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

constexpr int WIDE_THREADS = 736;   // 16 dequant warps, 4 epilogue warps, 2 producers, MMA warp
constexpr int WIDE_SA = 4;          // activation stages (a_rows * 128 bytes apart; the MMA reads 16 KB from each)
constexpr int WIDE_SB = 3;          // dequantized weight stages (32 KB each)
constexpr int WIDE_WG_MAX = 8;      // packed 128-row weight groups in the ring (4096*b + 512 bytes each)
#ifndef WIDE_FINALIZE_BATCH
#define WIDE_FINALIZE_BATCH 3
#endif
constexpr int WIDE_TMEM_COLS = 512; // two accumulators of 256 columns

// rows of the tcgen05.mma instruction: the 64-row form for batches of up to 64 rows
__host__ __device__ constexpr int wide_umma_rows(int a_rows) { return a_rows <= 64 ? 64 : 128; }

struct WideBarriers {
  uint64_t a_full[WIDE_SA], a_empty[WIDE_SA];
  uint64_t b_full[WIDE_SB], b_empty[WIDE_SB];
  uint64_t g_full[WIDE_WG_MAX], g_empty[WIDE_WG_MAX];
  uint64_t d_full[2], d_empty[2];
  uint32_t tmem_base;
  volatile int abort_flag;
  int last_flag;
  int fin_pending, fin_n_tile, fin_m_tile;  // a finalize left for the whole CTA (see the teardown)
};

// a ring stage: the packed weights of 256 columns x 128 rows, then rpg (1, 2 or 4) rows of 256 scales
__host__ __device__ constexpr int wide_wstage_bytes(int bits, int rpg) { return 4096 * bits + 512 * rpg; }

template <int VAR, int ACT>
__global__ void __launch_bounds__(WIDE_THREADS, 1)
wide_kernel(const WideParams p, const __grid_constant__ CUtensorMap tmap_a) {
  constexpr int B = var_bits(VAR);
  const uint32_t WSTAGE = (uint32_t)wide_wstage_bytes(B, p.rpg);
  constexpr uint32_t BSTAGE = 256u * 128u;
  // Activation stages: the copy fills a_rows rows (32, 64 or 128: the batch rounded up); the MMA
  // always reads 128 rows, i.e. 16 KB, from the stage's base.  Rows beyond the batch only feed
  // accumulator rows that nobody reads, so for small batches the stages are laid a_rows * 128 bytes
  // apart and the MMA's surplus rows alias the following stages: what is saved goes to the packed ring.
  const uint32_t ASTAGE = (uint32_t)p.a_rows * 128u;
  // Batches of up to 64 rows use the 64-row form of the instruction: it reads half the activation bytes
  // from shared memory, whose bandwidth is what the MMAs of this kernel wait for.
  const int UM = wide_umma_rows(p.a_rows);
  const uint32_t AREGION = (WIDE_SA - 1) * ASTAGE + (uint32_t)UM * 128u;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t smem_unaligned = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t smem_base = (smem_unaligned + 1023u) & ~1023u;
  unsigned char* smem_al = smem_raw + (smem_base - smem_unaligned);
  const int WG = p.wg_stages;
  const uint32_t a_s = smem_base;
  const uint32_t b_s = a_s + AREGION;
  const uint32_t w_s = b_s + WIDE_SB * BSTAGE;
  const uint32_t bars_off = AREGION + WIDE_SB * BSTAGE + (uint32_t)WG * WSTAGE;
  WideBarriers* bars = reinterpret_cast<WideBarriers*>(smem_al + bars_off);
  const uint32_t bars_s = smem_base + bars_off;
#define BAR_ADDR(field, i) (bars_s + (uint32_t)offsetof(WideBarriers, field) + (uint32_t)(i) * 8u)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int total_items = p.splits * p.n_tiles * p.m_tiles;
  const int nkk = p.kblocks_per_split;  // 64-blocks per work item (even)
  const int ngrp = nkk >> 1;
  volatile int* abort_flag = &bars->abort_flag;

  if (tid == 0) {
    for (int i = 0; i < WIDE_SA; ++i) { mbar_init(BAR_ADDR(a_full, i), 1); mbar_init(BAR_ADDR(a_empty, i), 1); }
    for (int i = 0; i < WIDE_SB; ++i) { mbar_init(BAR_ADDR(b_full, i), 8); mbar_init(BAR_ADDR(b_empty, i), 1); }
    for (int i = 0; i < WIDE_WG_MAX; ++i) { mbar_init(BAR_ADDR(g_full, i), 1); mbar_init(BAR_ADDR(g_empty, i), 8); }
    for (int i = 0; i < 2; ++i) { mbar_init(BAR_ADDR(d_full, i), 1); mbar_init(BAR_ADDR(d_empty, i), 4); }
    bars->abort_flag = 0;
    bars->last_flag = 0;
    bars->fin_pending = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // programmatic dependent launch: the next kernel of the stream may become resident when there is
  // room; this one reads activations / writes C only after its predecessor has completed (the two
  // roles that do so wait below), while the packed weights - constants - stream in right away
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (warp == 22) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     bars_s + (uint32_t)offsetof(WideBarriers, tmem_base)),
                 "r"(WIDE_TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = bars->tmem_base;

  // work item w -> (split, n_tile, m_tile), m fastest
#define ITEM_COORDS(w)                                         \
  const int m_tile = (w) % p.m_tiles;                          \
  const int n_tile = ((w) / p.m_tiles) % p.n_tiles;            \
  const int split = (w) / (p.m_tiles * p.n_tiles);             \
  const int kk0 = split * nkk;                                 \
  const int m0 = m_tile * 128;                                 \
  (void)m_tile; (void)n_tile; (void)split; (void)kk0; (void)m0;

  if (warp < 16) {
    // ================= dequantize: packed ring -> registers -> swizzled B operand tile =================
    // Two sets of eight warps take alternate 128-row groups, so that one set's loads and decode run
    // under the other set's stores and hand-over instead of all warps moving in lockstep.
    const int set = warp >> 3;
    const int nl = tid & 255;  // column inside the tile = row of the B operand
    // this column inside a ring stage: 16-column piece nl / 16, then unit (half*32 + r*4 + j)
    const uint32_t lane_off = (uint32_t)((nl >> 4) * (256 * B) + (((nl >> 3) & 1) * 32 + (nl & 7) * 4) * (B * 4));
    // row nl of a K-major 128-byte-swizzled tile: 8-row atoms of 1024 bytes, 16-byte chunk c at c ^ (row % 8)
    const uint32_t row_off = (uint32_t)((nl >> 3) * 1024 + (nl & 7) * 128);
    const uint32_t sw = (uint32_t)(nl & 7);
    // lanes that take the second unit of a block first (see the loads below): every other pair of
    // columns for 4-bit types (columns 64 bytes apart), every other column for 8-bit types (128 bytes)
    const uint32_t usw = B == 4 ? (uint32_t)((nl >> 1) & 1) : (B == 8 ? (uint32_t)(nl & 1) : 0u);
    int g_run = 0;  // groups passed so far (all work items)
    bool good = true;
    for (int w = blockIdx.x; w < total_items && good; w += gridDim.x) {
      ITEM_COORDS(w)
      const bool nvalid = n_tile * 256 + nl < p.N;
      for (int g = 0; g < ngrp && good; ++g, ++g_run) {
        if ((g_run & 1) != set) continue;  // the other set's group
        const int gs = g_run % WG;
        if (!mbar_wait_abortable(BAR_ADDR(g_full, gs), (uint32_t)(g_run / WG) & 1u, abort_flag)) { good = false; break; }
        const uint32_t st = w_s + (uint32_t)gs * WSTAGE;
        // the scales of this column's four 32-row units: scale row (unit * rpg) / 4 of the stage
        uint32_t s2u[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          unsigned short sbits;
          asm volatile("ld.shared.u16 %0, [%1];"
                       : "=h"(sbits)
                       : "r"(st + 4096u * B + (uint32_t)((u * p.rpg) >> 2) * 512u + (uint32_t)nl * 2u));
          s2u[u] = nvalid ? (uint32_t)sbits * 0x00010001u : 0u;  // the 16-bit scale in both halves
        }
        // all of this column's codes of the group go to registers first, so that the ring stage is
        // free for the next copy while the decode and the stores below run
        // Adjacent columns lie 16 * B bytes apart in the ring stage, so lanes reading the same unit of
        // their columns collide on the shared-memory banks.  Half of the lanes (usw = 1) therefore
        // read and process the two units of a block in the opposite order: wq[h][0] is unit usw of
        // block h, wq[h][1] unit usw ^ 1 (halves the conflicts; the decode does not care which unit it gets).
        uint32_t wq[2][2][B];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t blk = st + lane_off + (uint32_t)(2 * h * B * 4);
          if constexpr (B == 4 || B == 8) {
            lds_unit_words<B>(blk + usw * (uint32_t)(B * 4), wq[h][0]);
            lds_unit_words<B>(blk + (usw ^ 1u) * (uint32_t)(B * 4), wq[h][1]);
          } else {  // usw = 0: both units with the widest loads
            uint32_t two[2 * B];
            lds_two_units<B>(blk, two);
#pragma unroll
            for (int q = 0; q < B; ++q) { wq[h][0][q] = two[q]; wq[h][1][q] = two[B + q]; }
          }
        }
        if (!nvalid) {
#pragma unroll
          for (int q = 0; q < B; ++q) { wq[0][0][q] = 0u; wq[0][1][q] = 0u; wq[1][0][q] = 0u; wq[1][1][q] = 0u; }
        }
        // order the arrive after the loads have returned: make it depend on the loaded values
        {
          uint32_t dep = wq[0][0][0] ^ wq[1][1][B - 1];
          asm volatile("" : "+r"(dep));
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR_ADDR(g_empty, gs));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {  // the two 64-row blocks of the group
          uint32_t out[32];
          // wq[h][0] is unit usw of block h, wq[h][1] unit usw ^ 1
          unit_decode_scaled<VAR, ACT>(wq[h][0], usw ? s2u[2 * h + 1] : s2u[2 * h], out);
          unit_decode_scaled<VAR, ACT>(wq[h][1], usw ? s2u[2 * h] : s2u[2 * h + 1], out + 16);
          const int bi = 2 * g_run + h;  // running 64-block index
          const int sb = bi % WIDE_SB;
          if (!mbar_wait_abortable(BAR_ADDR(b_empty, sb), ((uint32_t)(bi / WIDE_SB) & 1u) ^ 1u, abort_flag)) { good = false; break; }
          const uint32_t dst = b_s + (uint32_t)sb * BSTAGE + row_off;
#pragma unroll
          for (int c = 0; c < 8; ++c)  // out[0..15] is unit usw (chunks 4 * usw ..), out[16..31] the other one
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst + (((uint32_t)c ^ sw ^ (usw << 2)) << 4)),
                         "r"(out[4 * c]), "r"(out[4 * c + 1]), "r"(out[4 * c + 2]), "r"(out[4 * c + 3])
                         : "memory");
          // generic-proxy writes must be visible to the tensor core's (async proxy) reads
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) mbar_arrive(BAR_ADDR(b_full, sb));
        }
      }
    }
  } else if (warp < 20) {
    // ================= epilogue: read D, write C (or add into the split-K scratch) =================
    asm volatile("griddepcontrol.wait;" ::: "memory");  // writes C and the split-K scratch
    const int ew = warp - 16;  // lane quadrant of tensor memory
    int it = 0;
    bool good = true;
    for (int w = blockIdx.x; w < total_items && good; w += gridDim.x, ++it) {
      ITEM_COORDS(w)
      const int buf = it & 1;
      // accumulator row r lives in lane r (128-row instruction) or in lane 32 * (r / 16) + r % 16 (64-row
      // instruction: sixteen rows at the start of each 32-lane quadrant)
      const bool lane_has_row = UM == 128 || lane < 16;
      const int m = m0 + (UM == 128 ? ew * 32 + lane : ew * 16 + lane);
      if (!mbar_wait_abortable(BAR_ADDR(d_full, buf), (uint32_t)(it >> 1) & 1u, abort_flag)) { good = false; break; }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t daddr = tmem + ((uint32_t)(ew * 32) << 16) + (uint32_t)(buf * 256);
      const bool rows_here = m0 + (UM == 128 ? ew * 32 : ew * 16) < p.M;  // any row of this warp inside the batch
      for (int c0 = 0; c0 < 256; c0 += 32) {
        const int n = n_tile * 256 + c0;
        if (!rows_here || n >= p.N) continue;  // warp-uniform
        uint32_t v[32];
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
            "%14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
              "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
              "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
              "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(daddr + (uint32_t)c0)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (m < p.M && lane_has_row) {
          const int ncols = min(32, p.N - n);  // multiple of 16
          if (p.splits == 1) {
            __half* dst = p.c + (size_t)m * p.ldc + n;
#pragma unroll
            for (int q = 0; q < 32; q += 8) {
              if (q < ncols) {
                uint4 o;
                o.x = pack2<ACT>(__uint_as_float(v[q]), __uint_as_float(v[q + 1]));
                o.y = pack2<ACT>(__uint_as_float(v[q + 2]), __uint_as_float(v[q + 3]));
                o.z = pack2<ACT>(__uint_as_float(v[q + 4]), __uint_as_float(v[q + 5]));
                o.w = pack2<ACT>(__uint_as_float(v[q + 6]), __uint_as_float(v[q + 7]));
                *reinterpret_cast<uint4*>(dst + q) = o;
              }
            }
          } else {
            float* dst = p.partial + (size_t)m * p.N + n;
#pragma unroll
            for (int q = 0; q < 32; q += 4)
              if (q < ncols)
                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + q), "f"(__uint_as_float(v[q])),
                             "f"(__uint_as_float(v[q + 1])), "f"(__uint_as_float(v[q + 2])),
                             "f"(__uint_as_float(v[q + 3]))
                             : "memory");
          }
        }
      }
      // the accumulator has been read: the MMAs of the tile after next may overwrite it
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(BAR_ADDR(d_empty, buf));
      if (p.splits > 1) {
        // the last split to arrive converts the fp32 sums and restores the zeros
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (warp == 16 && lane == 0) {
          __threadfence();
          const int old = atomicAdd(p.counters + n_tile * p.m_tiles + m_tile, 1);
          const int last = (old + 1 == p.splits) ? 1 : 0;
          if (last) __threadfence();
          // The CTA's last item: every role is done by then, so all 23 warps convert the tile after the
          // roles have left their loops (four warps alone need a dozen L2 round trips for it, and the next
          // kernel of the stream waits for the slowest CTA).
          const bool defer = w + (int)gridDim.x >= total_items;
          bars->last_flag = (last && !defer) ? 1 : 0;
          if (last && defer) {
            bars->fin_n_tile = n_tile;
            bars->fin_m_tile = m_tile;
            bars->fin_pending = 1;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (bars->last_flag) {
          const int rows = min(128, p.M - m0), cols = min(256, p.N - n_tile * 256);
          // FB independent 32-byte loads per thread in flight: one L2 round trip per batch, not per load
          constexpr int FB = WIDE_FINALIZE_BATCH;
          const int per_row = cols / 8, total = rows * per_row;
          for (int base = tid - 512; base < total; base += FB * 128) {
            float4 x[FB][2];
#pragma unroll
            for (int u = 0; u < FB; ++u) {
              const int idx = base + u * 128;
              if (idx < total) {
                const float4* src = reinterpret_cast<const float4*>(
                    p.partial + (size_t)(m0 + idx / per_row) * p.N + n_tile * 256 + (idx % per_row) * 8);
                x[u][0] = __ldcg(src);
                x[u][1] = __ldcg(src + 1);
              }
            }
#pragma unroll
            for (int u = 0; u < FB; ++u) {
              const int idx = base + u * 128;
              if (idx < total) {
                const int mm = m0 + idx / per_row, nn = n_tile * 256 + (idx % per_row) * 8;
                float4* src = reinterpret_cast<float4*>(p.partial + (size_t)mm * p.N + nn);
                uint4 o;
                o.x = pack2<ACT>(x[u][0].x, x[u][0].y);
                o.y = pack2<ACT>(x[u][0].z, x[u][0].w);
                o.z = pack2<ACT>(x[u][1].x, x[u][1].y);
                o.w = pack2<ACT>(x[u][1].z, x[u][1].w);
                *reinterpret_cast<uint4*>(p.c + (size_t)mm * p.ldc + nn) = o;
                __stcg(src, make_float4(0.f, 0.f, 0.f, 0.f));
                __stcg(src + 1, make_float4(0.f, 0.f, 0.f, 0.f));
              }
            }
          }
          if (warp == 16 && lane == 0) p.counters[n_tile * p.m_tiles + m_tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");  // last_flag may be rewritten by the next item
      }
    }
  } else if (warp == 20) {
    // ================= TMA producer: activations =================
    if (lane == 0) {
      asm volatile("griddepcontrol.wait;" ::: "memory");  // reads A
      int ai = 0;
      bool good = true;
      for (int w = blockIdx.x; w < total_items && good; w += gridDim.x) {
        ITEM_COORDS(w)
        for (int i = 0; i < nkk; ++i, ++ai) {
          const int sa = ai % WIDE_SA;
          if (!mbar_wait_abortable(BAR_ADDR(a_empty, sa), ((uint32_t)(ai / WIDE_SA) & 1u) ^ 1u, abort_flag)) { good = false; break; }
          const uint32_t bar = BAR_ADDR(a_full, sa);
          asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar),
                       "r"(ASTAGE)
                       : "memory");
          const int kx = (kk0 + i) * 64;
          asm volatile(
              "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
              ::"r"(a_s + (uint32_t)sa * ASTAGE), "l"(&tmap_a), "r"(bar), "r"(kx), "r"(m0)
              : "memory");
        }
      }
    }
  } else if (warp == 21) {
    // ================= bulk-copy producer: packed weights and scales =================
    int g_run = 0;
    bool good = true;
    const unsigned char* bq = reinterpret_cast<const unsigned char*>(p.bq);
    for (int w = blockIdx.x; w < total_items && good; w += gridDim.x) {
      ITEM_COORDS(w)
      const int nt0 = n_tile * 16;
      const int pieces = min(16, p.N / BLOCK_N - nt0);  // 16-column pieces of this tile that exist
      for (int g = 0; g < ngrp; ++g, ++g_run) {
        const int gs = g_run % WG;
        int ok = 1;
        if (lane == 0)
          ok = mbar_wait_abortable(BAR_ADDR(g_empty, gs), ((uint32_t)(g_run / WG) & 1u) ^ 1u, abort_flag) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) { good = false; break; }
        const uint32_t bar = BAR_ADDR(g_full, gs);
        const uint32_t dst = w_s + (uint32_t)gs * WSTAGE;
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
        }
        if (lane >= 16 && lane < 16 + p.rpg) {
          // scale row(s) of the group: one per 128 / rpg rows
          const int row = p.rpg == 1 ? (G * 128) / p.group : G * p.rpg + (lane - 16);
          const __half* src = p.scales + (size_t)row * p.N + n_tile * 256;
          asm volatile(
              "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                  dst + 4096u * B + (uint32_t)(lane - 16) * 512u),
              "l"(src), "r"((uint32_t)pieces * 32u), "r"(bar)
              : "memory");
        }
      }
    }
  } else {
    // ================= MMA issuer =================
    if (lane == 0) {
      const uint32_t idesc = (umma_idesc<ACT>(256) & ~(31u << 24)) | ((uint32_t)(UM >> 4) << 24);  // M = UM, N = 256
      bool good = true;
      int bi = 0, it = 0;
      for (int w = blockIdx.x; w < total_items && good; w += gridDim.x, ++it) {
        const int buf = it & 1;
        // the accumulator must have been read out by the epilogue two items ago
        if (!mbar_wait_abortable(BAR_ADDR(d_empty, buf), ((uint32_t)(it >> 1) & 1u) ^ 1u, abort_flag)) { good = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d_tmem = tmem + (uint32_t)(buf * 256);
        for (int i = 0; i < nkk; ++i, ++bi) {
          const int sa = bi % WIDE_SA, sb = bi % WIDE_SB;
          good = mbar_wait_abortable(BAR_ADDR(a_full, sa), (uint32_t)(bi / WIDE_SA) & 1u, abort_flag) &&
                 mbar_wait_abortable(BAR_ADDR(b_full, sb), (uint32_t)(bi / WIDE_SB) & 1u, abort_flag);
          if (!good) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t adesc = umma_smem_desc(a_s + (uint32_t)sa * ASTAGE);
          const uint64_t bdesc = umma_smem_desc(b_s + (uint32_t)sb * BSTAGE);
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            const uint32_t accumulate = (i > 0 || ks > 0) ? 1u : 0u;
            asm volatile(
                "{\n\t.reg .pred p;\n\t"
                "setp.ne.b32 p, %4, 0;\n\t"
                "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                ::"r"(d_tmem), "l"(adesc + (uint64_t)(ks * 2)), "l"(bdesc + (uint64_t)(ks * 2)), "r"(idesc),
                "r"(accumulate)
                : "memory");
          }
          // the stages may be overwritten once these MMAs have read them
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           BAR_ADDR(a_empty, sa))
                       : "memory");
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           BAR_ADDR(b_empty, sb))
                       : "memory");
        }
        if (good)
          asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                           BAR_ADDR(d_full, buf))
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
    p.status[1] = 6;  // where: wide tcgen05 kernel pipeline
    p.status[2] = blockIdx.x;
    p.status[3] = 0;
  }
  if (warp == 22) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(WIDE_TMEM_COLS) : "memory");
  }
  if (bars->fin_pending && !*abort_flag) {
    // the last K range of the CTA's last tile arrived here: all threads convert the fp32 sums and
    // restore the zeros (the counting thread's fence above ordered the other CTAs' additions before this)
    const int n_tile = bars->fin_n_tile, m_tile = bars->fin_m_tile, m0 = m_tile * 128;
    const int rows = min(128, p.M - m0), cols = min(256, p.N - n_tile * 256);
    constexpr int FB = WIDE_FINALIZE_BATCH;
    const int per_row = cols / 8, total = rows * per_row;
    for (int base = tid; base < total; base += FB * WIDE_THREADS) {
      float4 x[FB][2];
#pragma unroll
      for (int u = 0; u < FB; ++u) {
        const int idx = base + u * WIDE_THREADS;
        if (idx < total) {
          const float4* src = reinterpret_cast<const float4*>(
              p.partial + (size_t)(m0 + idx / per_row) * p.N + n_tile * 256 + (idx % per_row) * 8);
          x[u][0] = __ldcg(src);
          x[u][1] = __ldcg(src + 1);
        }
      }
#pragma unroll
      for (int u = 0; u < FB; ++u) {
        const int idx = base + u * WIDE_THREADS;
        if (idx < total) {
          const int mm = m0 + idx / per_row, nn = n_tile * 256 + (idx % per_row) * 8;
          float4* src = reinterpret_cast<float4*>(p.partial + (size_t)mm * p.N + nn);
          uint4 o;
          o.x = pack2<ACT>(x[u][0].x, x[u][0].y);
          o.y = pack2<ACT>(x[u][0].z, x[u][0].w);
          o.z = pack2<ACT>(x[u][1].x, x[u][1].y);
          o.w = pack2<ACT>(x[u][1].z, x[u][1].w);
          *reinterpret_cast<uint4*>(p.c + (size_t)mm * p.ldc + nn) = o;
          __stcg(src, make_float4(0.f, 0.f, 0.f, 0.f));
          __stcg(src + 1, make_float4(0.f, 0.f, 0.f, 0.f));
        }
      }
    }
    if (tid == 0) p.counters[n_tile * p.m_tiles + m_tile] = 0;
  }
#undef BAR_ADDR
#undef ITEM_COORDS
}

template <int VAR, int ACT>
static cudaError_t wide_launch_one(const WideParams& p, const CUtensorMap& tmap, int smem_bytes, cudaStream_t stream) {
  auto kern = wide_kernel<VAR, ACT>;
  static int configured_smem[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || configured_smem[dev] < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 16) configured_smem[dev] = smem_bytes;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)p.grid, 1, 1);
  cfg.blockDim = dim3(WIDE_THREADS, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, p, tmap);
}

template <int VAR>
static cudaError_t wide_launch_var(int var, const WideParams& p, const CUtensorMap& tmap, int smem_bytes,
                                   cudaStream_t stream) {
  if constexpr (VAR % B200Q_NPARTS == B200Q_PART) {
    if (var == VAR)
      return p.act == 0 ? wide_launch_one<VAR, 0>(p, tmap, smem_bytes, stream)
                        : wide_launch_one<VAR, 1>(p, tmap, smem_bytes, stream);
  }
  if constexpr (VAR + 1 < VAR_COUNT) return wide_launch_var<VAR + 1>(var, p, tmap, smem_bytes, stream);
  else return cudaErrorInvalidValue;
}

#define B200Q_CAT2(a, b) a##b
#define B200Q_CAT(a, b) B200Q_CAT2(a, b)

// One of these per compiled part; api.cu picks the part as var % B200Q_NPARTS.
cudaError_t B200Q_CAT(wide_launch_part, B200Q_PART)(int var, const WideParams& p, const void* tmap, int smem_bytes,
                                                    cudaStream_t stream) {
  return wide_launch_var<0>(var, p, *reinterpret_cast<const CUtensorMap*>(tmap), smem_bytes, stream);
}

#if B200Q_PART == 0
// dynamic shared memory: alignment slack + activation stages + B operand stages + packed ring + barriers
int wide_smem_bytes(int bits, int wg_stages, int a_rows, int rpg) {
  return 1024 + (WIDE_SA - 1) * a_rows * 128 + wide_umma_rows(a_rows) * 128 + WIDE_SB * 256 * 128 + wg_stages * wide_wstage_bytes(bits, rpg) +
         (int)sizeof(WideBarriers) + 64;
}
// rows one activation copy fills: the batch rounded up to 32, 64 or 128
int wide_a_rows(int M) { return M <= 32 ? 32 : (M <= 64 ? 64 : 128); }
// most packed weight groups in the ring (<= WIDE_WG_MAX) that fit
int wide_wg_stages(int bits, int max_smem, int a_rows, int rpg) {
  int wg = WIDE_WG_MAX;
  while (wg > 1 && wide_smem_bytes(bits, wg, a_rows, rpg) > max_smem) --wg;
  return wg;
}
#endif

}  // namespace b200q
