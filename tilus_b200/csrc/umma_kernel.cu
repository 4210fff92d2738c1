// Compute-bound path: C[M, N] = A[M, K] x dequant(Bq[K, N]) on the sm_100a tensor cores.
//
// The product is computed transposed, D[n, m] = sum_k W[k, n] * A[m, k], so that the
// dequantized weights are the operand that lives in tensor memory and the activations are
// the operand that TMA brings to shared memory:
//
//   * the 128 lanes of tensor memory are 128 weight columns n; a CTA owns a tile of
//     128 columns x TM activation rows (TM = 32 .. 256, the N extent of the MMA) and all of
//     K (or one of S splits of it);
//   * warps 0-7 dequantize.  Thread t of warp w is lane n = 32 * (w % 4) + t.  For a block
//     of 64 k it reads its column's 2 units (64 codes, 16*b contiguous bytes) from global
//     memory, decodes and scales them in registers with the unit decoder (decode.cuh; the
//     weights are fp16_rn(value * scale), exactly the values the reference multiplies by,
//     examples/quantization/matmul_a16wx.py:316-320) and writes the 32 half2 results to 32
//     columns of tensor memory with one tcgen05.st.  Warps 0-3 take the even 64-blocks,
//     warps 4-7 the odd ones;
//   * warp 8 is the TMA producer: one 2-D tiled copy (128-byte swizzle) per 64-block brings
//     A[m0 : m0+TM, k : k+64] into a 4-deep shared-memory ring; rows past M read as zero;
//   * warp 9 owns tensor memory (alloc / dealloc) and issues the MMAs: per 64-block four
//     tcgen05.mma.cta_group::1.kind::f16 (K = 16 each) with the weight operand in tensor
//     memory, the activation operand through a shared-memory descriptor and the fp32
//     accumulator D (128 lanes x TM columns) in tensor memory; tcgen05.commit releases the
//     activation stage and the weight stage when the MMAs have read them;
//   * after the last block warps 0-3 read D with tcgen05.ld, convert to fp16 and store
//     C[m, n] (64-byte row segments), or add into the fp32 split-K scratch.
//
// Every mbarrier wait is bounded in time; a wait that runs out raises a CTA-wide abort flag,
// all loops leave, tensor memory is still freed and the status word of the workspace reports
// it (the host reads it with b200q_device_status).
#include <cuda.h>

#include "common.cuh"

#ifndef B200Q_PART
#define B200Q_PART 0
#endif
#ifndef B200Q_NPARTS
#define B200Q_NPARTS 1
#endif

namespace b200q {

constexpr int UMMA_THREADS = 320;   // 8 dequant warps + TMA warp + MMA warp
constexpr int UMMA_SA = 4;          // activation stages
constexpr int UMMA_SW = 8;          // weight stages (32 tensor-memory columns each)
constexpr int UMMA_WCOL0 = 256;     // first tensor-memory column of the weight stages
constexpr int UMMA_TMEM_COLS = 512;

struct UmmaBarriers {
  uint64_t a_full[UMMA_SA], a_empty[UMMA_SA];
  uint64_t w_full[UMMA_SW], w_empty[UMMA_SW];
  uint64_t d_full;
  uint32_t tmem_base;
  volatile int abort_flag;
};

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// bounded wait (about two seconds); also gives up as soon as another thread raised the abort flag
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
    else if (now - t0 > 2000000000ull) { *abort_flag = 1; return false; }
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
// instruction descriptor: D fp32, A/B fp16, both K-major, M = 128, N = tm
__device__ __forceinline__ uint32_t umma_idesc(int tm) {
  return (1u << 4) | ((uint32_t)(tm >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

template <int VAR>
__global__ void __launch_bounds__(UMMA_THREADS, 1)
umma_kernel(const UmmaParams p, const __grid_constant__ CUtensorMap tmap_a) {
  constexpr int B = var_bits(VAR);
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  // [0, SA * TM * 128): activation stages (1024-byte aligned), then the barriers
  // (the 128-byte swizzle wants the stages on 1024-byte boundaries: align by hand)
  const uint32_t smem_unaligned = (uint32_t)__cvta_generic_to_shared(smem_raw);
  const uint32_t smem_base = (smem_unaligned + 1023u) & ~1023u;
  unsigned char* smem_al = smem_raw + (smem_base - smem_unaligned);
  const int TM = p.tm;
  const uint32_t stage_bytes = (uint32_t)TM * 128u;
  UmmaBarriers* bars = reinterpret_cast<UmmaBarriers*>(smem_al + (size_t)UMMA_SA * stage_bytes);
  const uint32_t bars_s = smem_base + UMMA_SA * stage_bytes;
#define BAR_ADDR(field, i) (bars_s + (uint32_t)offsetof(UmmaBarriers, field) + (uint32_t)(i) * 8u)

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // blockIdx.x = (split * n_tiles + n_tile) * m_tiles + m_tile: CTAs that run together share weights
  const int m_tile = blockIdx.x % p.m_tiles;
  const int n_tile = (blockIdx.x / p.m_tiles) % p.n_tiles;
  const int split = blockIdx.x / (p.m_tiles * p.n_tiles);
  const int kk0 = split * p.kblocks_per_split;  // first 64-block of this CTA
  const int nkk = p.kblocks_per_split;
  const int m0 = m_tile * TM;
  volatile int* abort_flag = &bars->abort_flag;

  if (tid == 0) {
    for (int i = 0; i < UMMA_SA; ++i) { mbar_init(BAR_ADDR(a_full, i), 1); mbar_init(BAR_ADDR(a_empty, i), 1); }
    for (int i = 0; i < UMMA_SW; ++i) { mbar_init(BAR_ADDR(w_full, i), 4); mbar_init(BAR_ADDR(w_empty, i), 1); }
    mbar_init(BAR_ADDR(d_full, 0), 1);
    bars->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 9) {
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

  if (warp < 8) {
    // ================= dequantize: global -> registers -> tensor memory =================
    const int grp = warp >> 2;                      // 0: even 64-blocks, 1: odd ones
    const int nl = (warp & 3) * 32 + lane;          // lane of tensor memory = column inside the tile
    const int n = n_tile * 128 + nl;
    const bool nvalid = n < p.N;
    const int nt = n >> 4, half = (n >> 3) & 1, r = n & 7;
    // words of this column inside a block: group c, units j: ((c*2 + half)*32 + r*4 + j) * B
    const uint32_t* col_words = reinterpret_cast<const uint32_t*>(p.bq) + (size_t)nt * p.KB * (256 * B) +
                                (size_t)(half * 32 + r * 4) * B;
    const uint32_t taddr_lane = tmem + ((uint32_t)((warp & 3) * 32) << 16) + UMMA_WCOL0;

    uint32_t wcur[2 * B], wnxt[2 * B];
    __half scur = __float2half(0.f), snxt = __float2half(0.f);
    auto load_block = [&](int kk, uint32_t (&w)[2 * B], __half& s) {
      // 64-block kk: block kk / 8, group (kk % 8) / 2, units (kk % 2) * 2 + {0, 1}
      const int kb = kk >> 3, c = (kk >> 1) & 3, j0 = (kk & 1) * 2;
      if (nvalid) {
        const uint32_t* src = col_words + (size_t)kb * (256 * B) + (size_t)(c * 64 + j0) * B;
        if constexpr ((2 * B) % 4 == 0) {
#pragma unroll
          for (int q = 0; q < 2 * B / 4; ++q) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(src) + q);
            w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
          }
        } else {
#pragma unroll
          for (int q = 0; q < B; ++q) {
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(src) + q);
            w[2 * q] = v.x; w[2 * q + 1] = v.y;
          }
        }
        const int row = p.gshift >= 0 ? ((kk >> 1) >> p.gshift) : 0;
        s = __ldg(p.scales + (size_t)row * p.N + n);
      } else {
#pragma unroll
        for (int q = 0; q < 2 * B; ++q) w[q] = 0u;
        s = __float2half(0.f);
      }
    };

    int kk = kk0 + grp;
    if (kk < kk0 + nkk) load_block(kk, wcur, scur);
    for (int i = grp; i < nkk; i += 2, kk += 2) {
      if (i + 2 < nkk) load_block(kk + 2, wnxt, snxt);
      const int sw = i % UMMA_SW;
      const uint32_t par = ((uint32_t)(i / UMMA_SW) & 1u) ^ 1u;
      if (!mbar_wait_abortable(BAR_ADDR(w_empty, sw), par, abort_flag)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t out[32];
      const __half2 s2 = __half2half2(scur);
      unit_decode_scaled<VAR>(wcur, s2, out);
      unit_decode_scaled<VAR>(wcur + B, s2, out + 16);
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
#pragma unroll
      for (int q = 0; q < 2 * B; ++q) wcur[q] = wnxt[q];
      scur = snxt;
    }

    // ================= epilogue: warps 0-3 read D and write C =================
    if (warp < 4) {
      const bool got = mbar_wait_abortable(BAR_ADDR(d_full, 0), 0, abort_flag);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (got) {
        const uint32_t daddr = tmem + ((uint32_t)(warp * 32) << 16);
        for (int c0 = 0; c0 < TM; c0 += 32) {
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
          if (nvalid) {
#pragma unroll
            for (int q = 0; q < 32; ++q) {
              const int m = m0 + c0 + q;
              if (m < p.M) {
                const float x = __uint_as_float(v[q]);
                if (p.splits == 1) p.c[(size_t)m * p.ldc + n] = __float2half_rn(x);
                else atomicAdd(p.partial + (size_t)m * p.N + n, x);
              }
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  } else if (warp == 8) {
    // ================= TMA producer: activations =================
    if (lane == 0) {
      for (int i = 0; i < nkk; ++i) {
        const int sa = i % UMMA_SA;
        const uint32_t par = ((uint32_t)(i / UMMA_SA) & 1u) ^ 1u;
        if (!mbar_wait_abortable(BAR_ADDR(a_empty, sa), par, abort_flag)) break;
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
  } else {
    // ================= MMA issuer =================
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(TM);
      bool good = true;
      for (int i = 0; i < nkk && good; ++i) {
        const int sa = i % UMMA_SA, sw = i % UMMA_SW;
        good = mbar_wait_abortable(BAR_ADDR(a_full, sa), (uint32_t)(i / UMMA_SA) & 1u, abort_flag) &&
               mbar_wait_abortable(BAR_ADDR(w_full, sw), (uint32_t)(i / UMMA_SW) & 1u, abort_flag);
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
  if (warp == 9) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(UMMA_TMEM_COLS) : "memory");
  }

  // ---- split-K: the last CTA of a tile converts the fp32 sums and restores the zeros ----
  if (p.splits > 1 && !*abort_flag) {
    __shared__ int s_last;
    __syncthreads();
    if (tid == 0) {
      __threadfence();
      const int old = atomicAdd(p.counters + n_tile * p.m_tiles + m_tile, 1);
      s_last = (old + 1 == p.splits) ? 1 : 0;
      if (s_last) __threadfence();
    }
    __syncthreads();
    if (s_last) {
      for (int idx = tid; idx < 128 * TM; idx += UMMA_THREADS) {
        const int n = n_tile * 128 + (idx & 127), m = m0 + (idx >> 7);
        if (n < p.N && m < p.M) {
          float* src = p.partial + (size_t)m * p.N + n;
          p.c[(size_t)m * p.ldc + n] = __float2half_rn(__ldcg(src));
          __stcg(src, 0.f);
        }
      }
      if (tid == 0) p.counters[n_tile * p.m_tiles + m_tile] = 0;
    }
  }
#undef BAR_ADDR
}

template <int VAR>
static cudaError_t umma_launch_one(const UmmaParams& p, const CUtensorMap& tmap, int smem_bytes,
                                   cudaStream_t stream) {
  auto kern = umma_kernel<VAR>;
  static int configured_smem[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16 || configured_smem[dev] < smem_bytes) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 16) configured_smem[dev] = smem_bytes;
  }
  kern<<<p.splits * p.n_tiles * p.m_tiles, UMMA_THREADS, smem_bytes, stream>>>(p, tmap);
  return cudaGetLastError();
}

template <int VAR>
static cudaError_t umma_launch_var(int var, const UmmaParams& p, const CUtensorMap& tmap, int smem_bytes,
                                   cudaStream_t stream) {
  if constexpr (VAR % B200Q_NPARTS == B200Q_PART) {
    if (var == VAR) return umma_launch_one<VAR>(p, tmap, smem_bytes, stream);
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
int umma_smem_bytes(int tm) { return 1024 + UMMA_SA * tm * 128 + (int)sizeof(UmmaBarriers) + 64; }
#endif

}  // namespace b200q
