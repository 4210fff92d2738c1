// Bit-exact dequantization W[K, N] = rn(value(q[k, n]) * s[k / group, n]) (one rounding, in the
// activation dtype: fp16 or bf16) of a
// b200-packed weight matrix.  Uses the same unit decoder as the GEMM kernels, so a
// bit-for-bit match of this output with the CPU oracle pins the weight values the
// GEMMs multiply by (reference semantics: examples/quantization/matmul_a16wx.py:316-320,
// b = cast(q) * scale).
//
// One warp per 16-column x 128-row group; lane (r, j) decodes columns r and r+8, rows j*32 .. +31
// of the group, as in the packed layout.  The group is transposed through shared memory so that the
// global stores are 16-byte row segments.
#include "common.cuh"

namespace b200q {

template <int VAR, int ACT>
__global__ void __launch_bounds__(128) dequant_kernel(const DequantParams p) {
  constexpr int B = var_bits(VAR);
  __shared__ unsigned short tile[4][128][16 + 2];  // per warp: one 128-row group x 16 columns
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane >> 2, j = lane & 3;
  const long long grp = (long long)blockIdx.x * 4 + warp;  // (column tile, 128-row group)
  const long long ngrp = (long long)p.NT * p.G;
  if (grp >= ngrp) return;
  const int nt = (int)(grp / p.G), g = (int)(grp % p.G);
  const uint32_t* base = reinterpret_cast<const uint32_t*>(p.bq) + (size_t)grp * (size_t)(B * 64);

#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t w[B], out[16];
    const uint32_t* src = base + (h * 32 + lane) * B;
#pragma unroll
    for (int q = 0; q < B; ++q) w[q] = __ldg(src + q);
    const int n = nt * 16 + h * 8 + r;
    const int k0 = g * 128 + j * 32;
    const uint32_t sbits = reinterpret_cast<const unsigned short*>(p.scales)[(size_t)(k0 / p.group) * p.N + n];
    unit_decode_scaled<VAR, ACT>(w, sbits * 0x00010001u, out);
#pragma unroll
    for (int pair = 0; pair < 16; ++pair) {
      tile[warp][j * 32 + 2 * pair][h * 8 + r] = (unsigned short)(out[pair] & 0xffffu);
      tile[warp][j * 32 + 2 * pair + 1][h * 8 + r] = (unsigned short)(out[pair] >> 16);
    }
  }
  __syncwarp();
  // 128 rows x 16 columns -> global; each lane writes 16-byte half rows
  for (int idx = lane; idx < 128 * 2; idx += 32) {
    const int row = idx >> 1, hh = idx & 1;
    __align__(16) unsigned short tmp[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) tmp[q] = tile[warp][row][hh * 8 + q];
    const size_t k = (size_t)g * 128 + row;
    *reinterpret_cast<uint4*>(p.w + k * p.N + nt * 16 + hh * 8) = *reinterpret_cast<uint4*>(tmp);
  }
}

template <int VAR>
static cudaError_t dq_launch_var(int var, const DequantParams& p, cudaStream_t stream) {
  if (var == VAR) {
    const long long nblk = (long long)p.NT * p.G;
    if (p.act == 0) dequant_kernel<VAR, 0><<<(unsigned)((nblk + 3) / 4), 128, 0, stream>>>(p);
    else dequant_kernel<VAR, 1><<<(unsigned)((nblk + 3) / 4), 128, 0, stream>>>(p);
    return cudaGetLastError();
  }
  if constexpr (VAR + 1 < VAR_COUNT) return dq_launch_var<VAR + 1>(var, p, stream);
  else return cudaErrorInvalidValue;
}

cudaError_t dequant_launch(int var, const DequantParams& p, cudaStream_t stream) {
  return dq_launch_var<0>(var, p, stream);
}

}  // namespace b200q
