// Memory-bound path: C[M<=16, N] = A[M, K] x dequant(Bq[K, N]) with split-K.
//
// Each warp streams whole 16-column x 512-row weight blocks straight from global memory
// into registers with 128-bit loads (a block is 1024*b contiguous bytes), decodes them
// with the unit decoder (decode.cuh) into the A operand of mma.sync.m16n8k16 - the
// weight tile is the 16-row operand, the (up to 8-row) activation slice is the 8-column
// operand, so M <= 8 costs one mma per 16x16 weights - and accumulates in fp32.
// Because a dot product does not care about the order of its terms, the k index of the
// mma is a private permutation: lane (r, j) owns rows j*128 .. j*128+127 of the block
// for columns r and r+8, so every lane's weights are one 128-bit vector per bit plane
// word and its activations are contiguous 16-byte pieces of the row.
//
// Work split: grid = S k-splits x P column ranges.  A CTA keeps its activation chunk
// [M, K/S] in shared memory (padded so that the 16-byte fragment reads are conflict
// free) and its 8 warps share the (column tile, k block) items of its range in
// contiguous runs.  Partial sums of a column tile that was split over several warps or
// CTAs meet in an fp32 scratch array through red.global.add; the warp that brings the
// tile's arrival counter to K/512 converts the sums to fp16, writes C and puts the
// scratch back to zero.  Nothing spins on anything.
//
// Reference: the computation restated here is QuantizedMatmul.__call__ of
// examples/quantization/matmul_a16wx.py:231-405 (cast, scale multiply, fp32 dot,
// fp16 store); its serial fp16 split-K (:375-398) is replaced by the fp32 reduction.
#include "common.cuh"

#ifndef B200Q_PART
#define B200Q_PART 0
#endif
#ifndef B200Q_NPARTS
#define B200Q_NPARTS 1
#endif

namespace b200q {

template <int B>
struct ItemRegs {
  uint4 v[2 * B];    // [plane word][half]
  uint32_t sc[2][2]; // fp16 scales per column half, units (0,1) and (2,3) packed in pairs
};

template <int VAR, int MT>
__global__ void __launch_bounds__(256, (var_bits(VAR) <= 4 ? 2 : 1)) skinny_kernel(const SkinnyParams p) {
  constexpr int B = var_bits(VAR);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __half* sA = reinterpret_cast<__half*>(smem_raw);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int r = lane >> 2, j = lane & 3;
  const int split = blockIdx.x / p.P, pidx = blockIdx.x % p.P;
  const int nt0 = (int)((long long)p.NT * pidx / p.P);
  const int nt1 = (int)((long long)p.NT * (pidx + 1) / p.P);
  const int items = (nt1 - nt0) * p.KBc;
  const int i0 = (int)((long long)items * warp / 8), i1 = (int)((long long)items * (warp + 1) / 8);
  const int kb_base = split * p.KBc;
  const bool g128 = (p.group % 128) == 0;

  auto load_item = [&](int i, ItemRegs<B>& it) {
    const int nt = nt0 + i / p.KBc;
    const int kb = kb_base + i % p.KBc;
    const uint4* base = p.bq + ((size_t)nt * p.KB + kb) * (size_t)(B * 64) + lane;
#pragma unroll
    for (int q = 0; q < 2 * B; ++q) it.v[q] = ld_stream_u4(base + q * 32);
    const int k0 = kb * 512 + j * 128;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int n = nt * 16 + h * 8 + r;
      if (g128) {
        const __half s = __ldg(p.scales + (size_t)(k0 / p.group) * p.N + n);
        it.sc[h][0] = it.sc[h][1] = bits_from_h2(__half2half2(s));
      } else {
#pragma unroll
        for (int u = 0; u < 4; u += 2) {
          const __half sa = __ldg(p.scales + (size_t)((k0 + u * 32) / p.group) * p.N + n);
          const __half sb = __ldg(p.scales + (size_t)((k0 + u * 32 + 32) / p.group) * p.N + n);
          it.sc[h][u >> 1] = bits_from_h2(__halves2half2(sa, sb));
        }
      }
    }
  };

  ItemRegs<B> ra, rb;
  if (i0 < i1) load_item(i0, ra);  // in flight while the activation chunk is staged

  // ---- stage the activation chunk A[0:M, kb_base*512 : +KBc*512] ----
  {
    const int kc = p.KBc * 512;
    const int vec_per_row = kc / 8;
    const int total = p.M * vec_per_row;
    for (int idx = tid; idx < total; idx += 256) {
      const int m = idx / vec_per_row;
      const int kk = (idx - m * vec_per_row) * 8;
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.a + (size_t)m * p.lda + (size_t)kb_base * 512 + kk));
      *reinterpret_cast<uint4*>(sA + (size_t)m * p.pitch + kk + (kk >> 7) * 8) = v;
    }
  }
  __syncthreads();
  if (i0 >= i1) return;

  float acc[MT][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int q = 0; q < 4; ++q) acc[mt][q] = 0.f;

  const __half* arow[MT];
  bool avalid[MT];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
    const int m = mt * 8 + r;
    avalid[mt] = m < p.M;
    arow[mt] = sA + (size_t)(avalid[mt] ? m : 0) * p.pitch;
  }

  auto compute_item = [&](int i, const ItemRegs<B>& it) {
    const int kbr = i % p.KBc;  // k block relative to the chunk
    const int koff = kbr * 512 + j * 128 + (kbr * 4 + j) * 8;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint32_t w0[B], w1[B];
#pragma unroll
      for (int v = 0; v < B; ++v) {
        w0[v] = u4_comp(it.v[v * 2 + 0], u);
        w1[v] = u4_comp(it.v[v * 2 + 1], u);
      }
      uint32_t W0[16], W1[16];
      const __half2 s0 = h2_from_bits(it.sc[0][u >> 1]), s1 = h2_from_bits(it.sc[1][u >> 1]);
      unit_decode_scaled<VAR>(w0, (u & 1) ? __high2half2(s0) : __low2half2(s0), W0);
      unit_decode_scaled<VAR>(w1, (u & 1) ? __high2half2(s1) : __low2half2(s1), W1);
#pragma unroll
      for (int sp = 0; sp < 4; ++sp) {
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          uint4 av = make_uint4(0u, 0u, 0u, 0u);
          if (avalid[mt]) av = *reinterpret_cast<const uint4*>(arow[mt] + koff + u * 32 + sp * 8);
          mma_m16n8k16(acc[mt], W0[4 * sp], W1[4 * sp], W0[4 * sp + 1], W1[4 * sp + 1], av.x, av.y);
          mma_m16n8k16(acc[mt], W0[4 * sp + 2], W1[4 * sp + 2], W0[4 * sp + 3], W1[4 * sp + 3], av.z, av.w);
        }
      }
    }
  };

  auto flush = [&](int nt, int nitems) {
    const int nbase = nt * 16 + r;
    if (nitems == p.KB) {  // this warp saw all of K: write C directly
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int m = mt * 8 + 2 * j + (q & 1);
          const int n = nbase + (q >> 1) * 8;
          if (m < p.M) p.c[(size_t)m * p.ldc + n] = __float2half_rn(acc[mt][q]);
        }
    } else {
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int m = mt * 8 + 2 * j + (q & 1);
          const int n = nbase + (q >> 1) * 8;
          if (m < p.M) atomicAdd(p.partial + (size_t)m * p.N + n, acc[mt][q]);
        }
      __threadfence();
      __syncwarp();
      int last = 0;
      if (lane == 0) {
        const int old = atomicAdd(p.counters + nt, nitems);
        last = (old + nitems == p.KB) ? 1 : 0;
      }
      last = __shfl_sync(0xffffffffu, last, 0);
      if (last) {
        __threadfence();
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int m = mt * 8 + 2 * j + (q & 1);
            const int n = nbase + (q >> 1) * 8;
            if (m < p.M) {
              float* src = p.partial + (size_t)m * p.N + n;
              const float v = __ldcg(src);
              p.c[(size_t)m * p.ldc + n] = __float2half_rn(v);
              __stcg(src, 0.f);
            }
          }
        if (lane == 0) p.counters[nt] = 0;
      }
    }
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[mt][q] = 0.f;
  };

  int run = 0;  // items accumulated for the current column tile
  auto step = [&](int i, ItemRegs<B>& use, ItemRegs<B>& fill) {
    if (i + 1 < i1) load_item(i + 1, fill);
    compute_item(i, use);
    ++run;
    const int nt = nt0 + i / p.KBc;
    if (i + 1 == i1 || (nt0 + (i + 1) / p.KBc) != nt) {
      flush(nt, run);
      run = 0;
    }
  };
  for (int i = i0; i < i1; i += 2) {
    step(i, ra, rb);
    if (i + 1 < i1) step(i + 1, rb, ra);
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
  kern<<<p.S * p.P, 256, smem_bytes, stream>>>(p);
  return cudaGetLastError();
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
