// Per-token FP8 (e4m3) casts of 16-bit activations, with and without the SwiGLU that follows a
// gate_up projection.  One float32 scale per token and group of `group` channels:
//
//   value  = x                                         (per_token_cast)
//   value  = silu(l) * r [* routing weight],  l = x[:, :H], r = x[:, H:]   (swiglu_per_token_cast)
//   absmax = max |value| over the group
//   scale  = absmax > 0 ? absmax / 448 : 1      inv = absmax > 0 ? 448 / absmax : 1
//   out    = e4m3_rn_satfinite(value * inv)     out_sf = scale
//
// the arithmetic of the reference's PerTokenCast and SwiGLUForwardAndPerTokenCast scripts
// (examples/quantization/per_token_cast.py:75-97, swiglu_forward_and_per_token_cast.py:110-166: fp32
// throughout, silu(l) = l / (exp(-l) + 1), clamp l from above and r on both sides, rows whose expert
// index is negative are skipped).  HBM-bound: 16 lanes own one group of 128 channels (8 channels, one
// 16-byte load each - two for SwiGLU - and one 8-byte store per lane); groups of 256, 384 and 512
// channels take two to four such steps with the values kept in registers.  The kernels wait for the previous kernel of the stream with
// griddepcontrol.wait, so that they can be launched with programmatic stream serialization right
// behind the GEMM whose output they read.
#include <cuda_fp8.h>

#include "common.cuh"

namespace b200q {

template <int ACT>
__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (ACT == 0) {
      const float2 t = __half22float2(h2_from_bits(w[i]));
      f[2 * i] = t.x; f[2 * i + 1] = t.y;
    } else {
      f[2 * i] = __uint_as_float(w[i] << 16);
      f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
}

// 16 lanes per group step of 128 channels
template <int ACT, bool SWIGLU>
__global__ void __launch_bounds__(256) cast_kernel(const CastParams p) {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int lane16 = threadIdx.x & 15;
  const unsigned hmask = 0xffffu << (threadIdx.x & 16);  // the half-warp this lane belongs to
  const int groups_per_row = p.H / p.group;
  const long long total = (long long)p.T * groups_per_row;
  const long long gid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
  const bool active = gid < total;
  const int t = active ? (int)(gid / groups_per_row) : 0;
  const int g = active ? (int)(gid - (long long)t * groups_per_row) : 0;
  asm volatile("griddepcontrol.wait;" ::: "memory");  // x is the previous kernel's output
  bool skip = !active;
  float weight = 1.0f;
  bool weighted = false;
  if (SWIGLU && active) {
    if (p.pos_to_expert && p.pos_to_expert[t] < 0) skip = true;
    if (!skip && p.pos_to_token_topk && p.topk_weights) {
      const int pos = p.pos_to_token_topk[t];
      if (pos >= 0) { weight = p.topk_weights[pos]; weighted = true; }
    }
  }
  // steps of 128 channels cover the group (at most four: the values stay in registers between the
  // absmax pass and the conversion)
  const int steps = p.group / 128;
  const unsigned short* row = p.x + (size_t)t * p.ldx + (size_t)g * p.group + lane16 * 8;
  float amax = 0.f;
  float keep[4][8];
  if (!skip) {
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (s < steps) {
        float l[8];
        unpack8<ACT>(__ldg(reinterpret_cast<const uint4*>(row + s * 128)), l);
        if constexpr (SWIGLU) {
          float r[8];
          unpack8<ACT>(__ldg(reinterpret_cast<const uint4*>(row + p.H + s * 128)), r);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float a = l[i], b = r[i];
            if (p.use_clamp) {
              a = a > p.clamp ? p.clamp : a;
              b = b > p.clamp ? p.clamp : b;
              b = b < -p.clamp ? -p.clamp : b;
            }
            const float silu = __fdiv_rn(a, expf(-a) + 1.0f);
            float val = silu * b;
            if (weighted) val = val * weight;
            keep[s][i] = val;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 8; ++i) keep[s][i] = l[i];
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(keep[s][i]));
      }
    }
  }
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(hmask, amax, o));
  if (skip) return;
  const float scale = amax > 0.f ? __fdiv_rn(amax, 448.0f) : 1.0f;
  const float inv = amax > 0.f ? __fdiv_rn(448.0f, amax) : 1.0f;
  if (lane16 == 0) p.out_sf[(size_t)t * groups_per_row + g] = scale;
  unsigned char* orow = p.out + (size_t)t * p.ldo + (size_t)g * p.group + lane16 * 8;
#pragma unroll
  for (int s = 0; s < 4; ++s) {
    if (s < steps) {
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(
            make_float2(keep[s][4 * h] * inv, keep[s][4 * h + 1] * inv), __NV_SATFINITE, __NV_E4M3);
        const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(
            make_float2(keep[s][4 * h + 2] * inv, keep[s][4 * h + 3] * inv), __NV_SATFINITE, __NV_E4M3);
        w[h] = (uint32_t)lo | ((uint32_t)hi << 16);
      }
      *reinterpret_cast<uint2*>(orow + s * 128) = make_uint2(w[0], w[1]);
    }
  }
}

cudaError_t cast_launch(const CastParams& p, int act, bool swiglu, cudaStream_t stream) {
  const long long total = (long long)p.T * (p.H / p.group);
  const long long threads = total * 16;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((threads + 255) / 256), 1, 1);
  cfg.blockDim = dim3(256, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (swiglu)
    return act == 0 ? cudaLaunchKernelEx(&cfg, cast_kernel<0, true>, p) : cudaLaunchKernelEx(&cfg, cast_kernel<1, true>, p);
  return act == 0 ? cudaLaunchKernelEx(&cfg, cast_kernel<0, false>, p) : cudaLaunchKernelEx(&cfg, cast_kernel<1, false>, p);
}

}  // namespace b200q
