// Memory-bound path: C[M<=16, N] = A[M, K] x dequant(Bq[K, N]) with split-K.
//
// Data movement: the weights of a 16-column tile are consecutive blocks of 16 columns x 512
// rows (1024*b contiguous bytes, four 128-row groups each).  Every warp pulls its items -
// whole or half blocks - into its own shared-memory ring with TMA bulk copies
// (cp.async.bulk, completion on an mbarrier); nothing is staged through registers and a
// warp keeps several items in flight.  The copies are issued before the kernel waits for
// its predecessor in the stream (programmatic dependent launch), so consecutive GEMVs
// overlap their tails and heads.
//
// Compute: one 128-row group at a time.  A lane reads its two units (columns r and r+8, 32 rows) with one vector load per unit, turns them into
// tensor-core operands with the unit decoder's "linear" patterns (decode.cuh, pair_lin: one
// mask per pair of codes, no floating-point work per weight) and issues mma.sync.m16n8k16
// with the weight tile as the 16-row operand and the (up to 8-row) activation slice as the
// 8-column operand.  An integer code q lands in the mantissa of an fp16 subnormal (value
// q * 2^(T-24)), a float code in its own exponent/mantissa bits; the tensor core multiplies
// these exactly by activations that were pre-multiplied by 2^-T when the CTA staged them
// into shared memory, and accumulates one 128-row group in fp32.  Once per group and column
// the accumulator is repaired and scaled:
//     C += (s * F) * (acc_group - zero_point * sum_k(a_k) / F),   F = 2^24 (ints)
// with the activation group sums computed during staging.  Products are exact, sums are
// fp32; the weights are never rounded to fp16, so the result is at least as close to the
// real-valued product as the reference's cast-then-scale-then-dot
// (examples/quantization/matmul_a16wx.py:316-321), well inside the 1e-2 tolerance.  The
// bit-exact weight values are available from the dequantize kernel.
//
// The k index of the mma is a private permutation (a dot product does not care about the
// order of its terms): lane (r, j) owns rows j*32 .. j*32+31 of the group, so its weights
// are one contiguous unit per column and its activations contiguous 16-byte pieces.
//
// Work split: the grid is GS x P clusters of CS CTAs.  A cluster owns a range of column
// tiles; its CTAs (and the GS "global" splits) cut K into S = GS*CS chunks.  A CTA keeps
// its activation chunk [M, K/S] in shared memory (padded so that the 16-byte fragment reads
// are conflict free); its quads take contiguous runs of the (column tile, k block) items.
// Partial tiles are added into a small fp32 tile buffer in shared memory (red.shared), the
// other CTAs of the cluster add theirs into rank 0's buffer through distributed shared
// memory, and rank 0 writes C.  Only when GS > 1 do sums also meet in a global fp32 scratch
// array (red.global) with an arrival counter per column tile; the last arriver converts
// them, writes C and puts the scratch back to zero.  The only waits are on mbarriers of the
// CTA's own bulk copies (bounded) and on the cluster barrier, which every thread of every
// CTA reaches unconditionally.
//
// Reference: the computation is QuantizedMatmul.__call__ of
// examples/quantization/matmul_a16wx.py:231-405 (cast, scale multiply, fp32 dot, fp16
// store); its serial fp16 split-K (:375-398) is replaced by the fp32 reduction.
#include "common.cuh"

#ifndef B200Q_PART
#define B200Q_PART 0
#endif
#ifndef B200Q_NPARTS
#define B200Q_NPARTS 1
#endif

namespace b200q {

// Waits on an mbarrier phase for at most about two seconds; false when that ran out.
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
    else if (now - t0 > 2000000000ull) return false;
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

// An item is GI consecutive 128-row groups of one block (GI*256*B contiguous bytes): whole
// blocks for the narrow types, half blocks from 3 bits up, so that the items per warp come
// out even and a ring slot stays a few KB.
constexpr int skinny_gi(int var) { return var_bits(var) <= 2 ? 4 : 2; }
constexpr int SKINNY_WARPS = 8;

// Shared-memory layout (byte offsets from the dynamic smem base):
//   [0, 512)     mbarriers [warp][stage]
//   [512, ...)   weight rings [warp][stage][GI*256*B bytes]
//   then         output tile sums [tiles of the CTA][16 columns][8*MT rows] floats
//   then         activation chunk [M][pitch] halfs, then group sums [groups][8*MT] floats
template <int VAR, int MT>
__global__ void __launch_bounds__(SKINNY_WARPS * 32, 2) skinny_kernel(const SkinnyParams p) {
  constexpr int B = var_bits(VAR);
  constexpr int MP = 8 * MT;
  constexpr int BIAS = var_bias(VAR);
  constexpr int GI = skinny_gi(VAR);
  constexpr int NI = 4 / GI;  // items per block
  constexpr int ITEM_BYTES = GI * 256 * B;
  constexpr int NWARPS = SKINNY_WARPS;
  constexpr float F = (float)(1u << lin_factor_log2(VAR));
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const int NST = p.stages;
  const uint32_t smem_base = (uint32_t)__cvta_generic_to_shared(smem_raw);
  unsigned char* ring_all = smem_raw + 512;
  float* sAcc = reinterpret_cast<float*>(ring_all + (size_t)NWARPS * NST * ITEM_BYTES);
  __half* sA = reinterpret_cast<__half*>(sAcc + (size_t)p.tiles_max * 16 * MP);
  // -zero_point * sum of the activations of each 128-row group, divided by F: [group][MP]
  float* sNb = reinterpret_cast<float*>(reinterpret_cast<unsigned char*>(sA) + (size_t)p.M * p.pitch * 2);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, j = lane & 3;
  // blockIdx.x = (gs * P + pidx) * CS + rank; k chunk = gs * CS + rank
  const int rank = blockIdx.x % p.CS;
  const int pidx = (blockIdx.x / p.CS) % p.P;
  const int split = (blockIdx.x / (p.CS * p.P)) * p.CS + rank;
  const int nt0 = (int)((long long)p.NT * pidx / p.P);
  const int nt1 = (int)((long long)p.NT * (pidx + 1) / p.P);
  const int IPT = p.KBc * NI;  // items per column tile in this CTA's k chunk
  const int items = (nt1 - nt0) * IPT;
  const int i0 = (int)((long long)items * warp / NWARPS), i1 = (int)((long long)items * (warp + 1) / NWARPS);
  const int n_items = i1 - i0;
  const int kb_base = split * p.KBc;

  // let the next kernel of the stream start its own prologue as soon as there is room
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const uint32_t bar0 = smem_base + warp * 64;
  const uint32_t ring_s = smem_base + 512 + warp * NST * ITEM_BYTES;
  const uint32_t ring_end = ring_s + NST * ITEM_BYTES;

  // ---- producer side: lane 0 of every warp feeds the warp's own ring with bulk copies ----
  // (the weights are constants, so this runs ahead of the wait on the previous kernel)
  const unsigned char* is_src = nullptr;  // next item to request (items of a tile chunk are contiguous)
  int is_q = 0, issued = 0;               // position inside the tile chunk
  const size_t tile_skip = (size_t)(p.KB - p.KBc) * (1024 * B);  // from the end of a chunk to the next tile's
  if (n_items > 0) {
    is_q = i0 % IPT;
    is_src = reinterpret_cast<const unsigned char*>(p.bq) +
             ((size_t)(nt0 + i0 / IPT) * p.KB + kb_base) * (size_t)(1024 * B) + (size_t)is_q * ITEM_BYTES;
  }
  auto issue_next = [&](uint32_t bar, uint32_t dst) {  // lane 0 only
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(ITEM_BYTES) : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
        "l"(is_src), "r"(ITEM_BYTES), "r"(bar)
        : "memory");
    ++issued;
    is_src += ITEM_BYTES;
    if (++is_q == IPT) { is_q = 0; is_src += tile_skip; }
  };
  if (lane == 0) {
    for (int s = 0; s < NST; ++s) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0 + s * 8) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (p.debug_skip < 2)
      for (int s = 0; s < NST && issued < n_items; ++s) issue_next(bar0 + s * 8, ring_s + s * ITEM_BYTES);
  }
  __syncwarp();

  for (int idx = tid; idx < p.tiles_max * 16 * MP; idx += NWARPS * 32) sAcc[idx] = 0.f;
  __syncthreads();
  // rank 0's tile buffer is clean before any peer adds into it (waited for at the very end)
  if (p.CS > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");

  // everything below may read what the previous kernel of the stream wrote
  asm volatile("griddepcontrol.wait;" ::: "memory");

  // ---- stage the activation chunk A[0:M, kb_base*512 : +KBc*512], pre-scaled ----
  if (p.debug_skip < 3) {
    const int kc = p.KBc * 512;
    const int vec_per_row = kc / 8;  // multiple of 64
    const int total = p.M * vec_per_row;
    // a thread always lands on the same 8-column slot of a 32-column unit: pairs h0 .. h0+3
    const int h0 = (tid & 3) * 4;
    __half2 mult[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int e = lin_prescale_shift(VAR, h0 + q);
      mult[q] = h2_from_bits(dup16((uint32_t)(15 - e) << 10));  // 2^-e
    }
    int m = 0, v0 = tid;  // idx = m * vec_per_row + v0
    for (int idx = tid; idx < total; idx += NWARPS * 32) {
      while (v0 >= vec_per_row) { v0 -= vec_per_row; ++m; }
      const int kk = v0 * 8;
      v0 += NWARPS * 32;
      uint4 v = __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)m * p.lda + (size_t)kb_base * 512 + kk));
      __half2 x0 = h2_from_bits(v.x), x1 = h2_from_bits(v.y), x2 = h2_from_bits(v.z), x3 = h2_from_bits(v.w);
      if constexpr (BIAS != 0) {
        const float2 f0 = __half22float2(x0), f1 = __half22float2(x1), f2 = __half22float2(x2),
                     f3 = __half22float2(x3);
        float sum = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        sum += __shfl_xor_sync(0xffffffffu, sum, 8);
        if ((lane & 15) == 0) sNb[(kk >> 7) * MP + m] = -(float)BIAS * sum * (1.0f / F);
      }
      if constexpr (!var_is_float(VAR)) {
        x0 = __hmul2(x0, mult[0]); x1 = __hmul2(x1, mult[1]);
        x2 = __hmul2(x2, mult[2]); x3 = __hmul2(x3, mult[3]);
      }
      v.x = bits_from_h2(x0); v.y = bits_from_h2(x1); v.z = bits_from_h2(x2); v.w = bits_from_h2(x3);
      *reinterpret_cast<uint4*>(sA + (size_t)m * p.pitch + kk + (kk >> 5) * 8) = v;
    }
  }
  __syncthreads();  // activations staged

  bool ok = true;
  if (n_items > 0 && p.debug_skip < 2) {
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[mt][q] = 0.f;

    uint32_t a_addr[MT];
    bool avalid[MT];
    uint4 av[MT];  // stays zero for the lanes whose activation row does not exist
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const int m = mt * 8 + r;
      avalid[mt] = m < p.M;
      // 32 columns + 8 of padding per unit, 4 units per group
      a_addr[mt] = (uint32_t)__cvta_generic_to_shared(sA) + 2u * (uint32_t)((avalid[mt] ? m : 0) * p.pitch + j * 40);
      av[mt] = make_uint4(0u, 0u, 0u, 0u);
    }
    const uint32_t nb_base = (uint32_t)__cvta_generic_to_shared(sNb) + 4u * (uint32_t)(2 * j);
    const uint32_t w_lane = (uint32_t)(lane * B * 4);

    // scales: row (kb*4 + c) >> gshift (or row 0 when there is one group per column)
    const __half* sc_col = p.scales + r;
    const int gshift = p.gshift;

    int cur_nt = nt0 + i0 / IPT;
    int q = i0 % IPT;  // item index inside the tile chunk: k block q / NI, groups (q % NI) * GI ...
    uint32_t slot_s = ring_s, bar = bar0;
    uint32_t parity = 0;
    int it = 0;
    while (it < n_items && ok) {
      const int run = min(IPT - q, n_items - it);  // items of this column tile
      const __half* sc_tile = sc_col + cur_nt * 16;
      for (int e = 0; e < run; ++e, ++it, ++q) {
        const int g0 = q * GI;  // first 128-row group of the item, counted inside the chunk
        // this item's scales: GI groups x columns r, r+8
        uint32_t sc[GI];
#pragma unroll
        for (int gi = 0; gi < GI; ++gi) {
          const int row = gshift >= 0 ? ((kb_base * 4 + g0 + gi) >> gshift) : 0;
          const __half* sp = sc_tile + (size_t)row * p.N;
          sc[gi] = bits_from_h2(__halves2half2(__ldg(sp), __ldg(sp + 8)));
        }
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar, parity) ? 1 : 0)) { ok = false; break; }

#pragma unroll
        for (int gi = 0; gi < GI; ++gi) {
          uint32_t w0[B], w1[B];
          lds_unit_words<B>(slot_s + w_lane + gi * (256 * B), w0);
          lds_unit_words<B>(slot_s + w_lane + gi * (256 * B) + 128 * B, w1);
          if (gi == GI - 1) {
            __syncwarp();  // every lane has its copy of the last group: refill the slot
            if (lane == 0 && issued < n_items) {
              asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
              issue_next(bar, slot_s);
            }
          }
          if (p.debug_skip == 1) {  // diagnosis only: stream the weights, skip the math
            uint32_t x = 0;
#pragma unroll
            for (int v = 0; v < B; ++v) x ^= w0[v] ^ w1[v];
            acc[0][0] += __uint_as_float(x & 0x007fffffu);
            continue;
          }
          uint32_t W0[16], W1[16];
          unit_decode_linear<VAR>(w0, W0);
          unit_decode_linear<VAR>(w1, W1);
          const uint32_t koff = (uint32_t)((g0 + gi) * 320);  // bytes: 128 columns + 4 x 8 of padding per group
          float g[MT][2][4];  // two independent accumulation chains per tile
#pragma unroll
          for (int sp = 0; sp < 4; ++sp) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
              if (avalid[mt]) av[mt] = lds_u4(a_addr[mt] + koff + sp * 16);
              if (sp == 0) {
                mma_m16n8k16_init(g[mt][0], W0[0], W1[0], W0[1], W1[1], av[mt].x, av[mt].y);
                mma_m16n8k16_init(g[mt][1], W0[2], W1[2], W0[3], W1[3], av[mt].z, av[mt].w);
              } else {
                mma_m16n8k16(g[mt][0], W0[4 * sp], W1[4 * sp], W0[4 * sp + 1], W1[4 * sp + 1], av[mt].x,
                             av[mt].y);
                mma_m16n8k16(g[mt][1], W0[4 * sp + 2], W1[4 * sp + 2], W0[4 * sp + 3], W1[4 * sp + 3], av[mt].z,
                             av[mt].w);
              }
            }
          }
          const __half2 s2 = h2_from_bits(sc[gi]);
          const float sf0 = __low2float(s2) * F, sf1 = __high2float(s2) * F;
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            float2 nb = make_float2(0.f, 0.f);
            if constexpr (BIAS != 0) nb = lds_f2(nb_base + (uint32_t)((g0 + gi) * MP + mt * 8) * 4u);
            acc[mt][0] = fmaf(sf0, (g[mt][0][0] + g[mt][1][0]) + nb.x, acc[mt][0]);
            acc[mt][1] = fmaf(sf0, (g[mt][0][1] + g[mt][1][1]) + nb.y, acc[mt][1]);
            acc[mt][2] = fmaf(sf1, (g[mt][0][2] + g[mt][1][2]) + nb.x, acc[mt][2]);
            acc[mt][3] = fmaf(sf1, (g[mt][0][3] + g[mt][1][3]) + nb.y, acc[mt][3]);
          }
        }
        slot_s += ITEM_BYTES; bar += 8;
        if (slot_s == ring_end) { slot_s = ring_s; bar = bar0; parity ^= 1u; }
      }
      // end of this column tile (or of the run): add the partial tile into the CTA's tile buffer
      {
        float* dst = sAcc + (size_t)(cur_nt - nt0) * 16 * MP;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) {
            const int m = mt * 8 + 2 * j + (qq & 1);
            if (m < p.M) atomicAdd(dst + (r + (qq >> 1) * 8) * MP + m, acc[mt][qq]);
            acc[mt][qq] = 0.f;
          }
      }
      q = 0;
      ++cur_nt;
    }
  }
  if (!ok) {
    // a bulk copy never completed: report it and give the copies still in flight a bounded
    // chance to land (the CTA must not retire under them)
    if (lane == 0) {
      atomicExch(p.status, ST_DEVICE_TIMEOUT);
      p.status[1] = 1;  // where: skinny kernel weight ring
      p.status[2] = blockIdx.x;
      p.status[3] = warp;
    }
    for (int s = 0; s < NST; ++s) mbar_wait_bounded(bar0 + s * 8, 0);
  }

  // ---- reduce over the cluster and write out ----
  __syncthreads();
  const int ntile = nt1 - nt0;
  const int nelem = ntile * 16 * MP;
  if (p.CS > 1) {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");  // pairs with the early arrive
    if (rank != 0) {
      const uint32_t local = (uint32_t)__cvta_generic_to_shared(sAcc);
      uint32_t remote;
      asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(0));
      for (int idx = tid; idx < nelem; idx += NWARPS * 32) {
        if ((idx % MP) < p.M)
          asm volatile("red.relaxed.cluster.shared::cluster.add.f32 [%0], %1;" ::"r"(remote + idx * 4),
                       "f"(sAcc[idx])
                       : "memory");
      }
    }
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
  }
  if (rank != 0) return;
  if (p.GS == 1) {
    for (int idx = tid; idx < nelem; idx += NWARPS * 32) {
      const int m = idx % MP, n = nt0 * 16 + idx / MP;
      if (m < p.M) p.c[(size_t)m * p.ldc + n] = __float2half_rn(sAcc[idx]);
    }
    return;
  }
  // several clusters share these column tiles: meet in the global scratch array
  for (int idx = tid; idx < nelem; idx += NWARPS * 32) {
    const int m = idx % MP, n = nt0 * 16 + idx / MP;
    if (m < p.M) atomicAdd(p.partial + (size_t)m * p.N + n, sAcc[idx]);
  }
  __syncthreads();
  int* s_last = reinterpret_cast<int*>(sAcc);  // the tile sums are no longer needed
  if (tid == 0) __threadfence();  // cumulative over the CTA's additions (ordered by the barrier above)
  __syncthreads();
  for (int t = tid; t < ntile; t += NWARPS * 32) {
    const int old = atomicAdd(p.counters + nt0 + t, 1);
    s_last[t] = (old + 1 == p.GS) ? 1 : 0;
  }
  __syncthreads();
  for (int idx = tid; idx < nelem; idx += NWARPS * 32) {
    const int t = idx / (16 * MP);
    if (!s_last[t]) continue;
    __threadfence();
    const int m = idx % MP, n = nt0 * 16 + idx / MP;
    if (m < p.M) {
      float* src = p.partial + (size_t)m * p.N + n;
      p.c[(size_t)m * p.ldc + n] = __float2half_rn(__ldcg(src));
      __stcg(src, 0.f);
    }
    if ((idx % (16 * MP)) == 0) p.counters[nt0 + t] = 0;
  }
}

template <int VAR, int MT>
static cudaError_t launch_one(const SkinnyParams& p, int smem_bytes, cudaStream_t stream) {
  auto kern = skinny_kernel<VAR, MT>;
  static int configured_smem[16] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (smem_bytes > 48 * 1024 && (dev < 0 || dev >= 16 || configured_smem[dev] < smem_bytes)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    if (dev >= 0 && dev < 16) configured_smem[dev] = smem_bytes;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(p.GS * p.P * p.CS), 1, 1);
  cfg.blockDim = dim3(SKINNY_WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = (size_t)smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)p.CS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this kernel may start while the previous kernel of the
  // stream drains; it waits (griddepcontrol.wait) before it reads anything but the weights
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = p.pdl ? 1 : 0;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kern, p);
}

template <int VAR>
static cudaError_t launch_var(int var, const SkinnyParams& p, int mt, int smem_bytes, cudaStream_t stream) {
  if constexpr (VAR % B200Q_NPARTS == B200Q_PART) {
    if (var == VAR) {
      return mt == 1 ? launch_one<VAR, 1>(p, smem_bytes, stream) : launch_one<VAR, 2>(p, smem_bytes, stream);
    }
  }
  if constexpr (VAR + 1 < VAR_COUNT) return launch_var<VAR + 1>(var, p, mt, smem_bytes, stream);
  else return cudaErrorInvalidValue;
}

#define B200Q_CAT2(a, b) a##b
#define B200Q_CAT(a, b) B200Q_CAT2(a, b)

// One of these per compiled part; api.cu picks the part as var % B200Q_NPARTS.
cudaError_t B200Q_CAT(skinny_launch_part, B200Q_PART)(int var, const SkinnyParams& p, int mt, int smem_bytes,
                                                       cudaStream_t stream) {
  return launch_var<0>(var, p, mt, smem_bytes, stream);
}

}  // namespace b200q
