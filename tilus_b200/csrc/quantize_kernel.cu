// load_and_quantize on the GPU: dense weight[out, in] -> per-group scales + packed weights in
// the b200 layout, in two passes over the dense weight.
//
// The arithmetic is QuantizedLinear.load_and_quantize of the reference
// (examples/quantization/matmul_a16wx.py:470-528), operation for operation so that the codes
// and scales come out bit-identical to the host path (tilus_b200/quantize.py):
//   scales[g, n] = rn(max(absmax(w[n, group g]) / max_value, 1e-6))             (fp32 division, rounded to
//                                                                                 the activation dtype)
//   q            = clamp(w / float(scales), min_value, max_value)               (fp32 division)
//   integer types: code = rint(q) & mask   (round half to even, as torch.round)
//   float types:   code = the reference's fp32 -> sub-byte encode: round to nearest even at the
//                  target's precision, saturate, flush fp32 subnormals to signed zero
//                  (python/tilus/hidet/ir/primitives/cuda/cast.py:44-100)
// Pass 1: one warp per (column, group) reduces the absmax.  Pass 2: one thread per unit (32 codes
// of one column) quantizes its 32 weights, builds the unit's b plane words (layout described in
// decode.cuh / tilus_b200/packing.py; signed integers in offset binary) and stores them at the
// unit's place in the [column tile][128-row group][half][lane] order.
#include "common.cuh"

namespace b200q {

struct QuantParams {
  const void* w;   // [N, K] row-major (row = output feature), leading dimension ldw
  int w_dtype;     // 0 fp16, 1 fp32, 2 bf16
  int ldw;
  uint32_t* bq;    // packed output, K*N*nbits/8 bytes
  unsigned short* scales;  // [K/group, N], 16-bit patterns of the activation dtype
  int act;         // 0 fp16, 1 bf16
  int N, K, G, group;  // G = K / 128
  int kind, nbits, ebits, mbits;  // kind: 0 unsigned, 1 two's complement, 2 float
  float minv, maxv;
};

__device__ __forceinline__ float load_w(const QuantParams& p, size_t idx) {
  if (p.w_dtype == 1) return reinterpret_cast<const float*>(p.w)[idx];
  if (p.w_dtype == 2) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.w)[idx]);
  return __half2float(reinterpret_cast<const __half*>(p.w)[idx]);
}
__device__ __forceinline__ float load_scale(const QuantParams& p, size_t idx) {
  const unsigned short b = p.scales[idx];
  return p.act == 0 ? __half2float(__ushort_as_half(b)) : __uint_as_float((uint32_t)b << 16);
}

__global__ void __launch_bounds__(256) quant_scales_kernel(const QuantParams p) {
  const int lane = threadIdx.x & 31;
  const long long wid = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int groups = p.K / p.group;
  if (wid >= (long long)p.N * groups) return;
  const int n = (int)(wid / groups), g = (int)(wid % groups);
  const size_t base = (size_t)n * p.ldw + (size_t)g * p.group;
  float m = 0.f;
  for (int i = lane; i < p.group; i += 32) m = fmaxf(m, fabsf(load_w(p, base + i)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if (lane == 0) {
    const float sc = fmaxf(__fdiv_rn(m, p.maxv), 1e-6f);
    p.scales[(size_t)g * p.N + n] = p.act == 0 ? __half_as_ushort(__float2half_rn(sc))
                                               : __bfloat16_as_ushort(__float2bfloat16_rn(sc));
  }
}

// fp32 -> sub-byte float code (sign / e exponent bits / m mantissa bits)
__device__ __forceinline__ uint32_t encode_float_code(float x, int nbits, int e, int m) {
  const uint32_t u = __float_as_uint(x);
  const uint32_t sign = ((u >> 31) & 1u) << (nbits - 1);
  const int exps = (int)((u >> 23) & 0xFFu);
  if (exps == 0) return sign;                                   // zero and fp32 subnormals
  if (exps == 0xFF) return (sign | ((1u << nbits) - 1u)) & ((1u << nbits) - 1u);  // Inf / NaN: all ones
  uint32_t mant = (u & 0x7FFFFFu) | 0x800000u;
  const int shift = 23 - m;
  const uint32_t round_bit = (mant >> (shift - 1)) & 1u;
  const bool sticky = (mant & ((1u << (shift - 1)) - 1u)) != 0u;
  const uint32_t lsb = (mant >> shift) & 1u;
  if (round_bit && (sticky || lsb)) mant += 1u << shift;
  int carry = 0;
  if (mant & 0x01000000u) { mant >>= 1; carry = 1; }
  int exp_value = exps - 127 + carry + (1 << (e - 1)) - 1;
  mant >>= shift;
  if (exp_value >= (1 << e)) return sign | ((1u << (nbits - 1)) - 1u);  // saturate
  if (exp_value <= 0) {
    if (exp_value >= 1 - m) return sign | (mant >> (1 - exp_value));   // subnormal of the target
    return sign;
  }
  return sign | ((uint32_t)exp_value << m) | (mant ^ (1u << m));
}

__global__ void __launch_bounds__(128) quant_pack_kernel(const QuantParams p) {
  // unit index = ((nt * G + g) * 2 + half) * 32 + lane,  lane = r * 4 + j,  g = 128-row group of K
  const long long unit = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long units = (long long)p.N * p.K / 32;
  if (unit >= units) return;
  const int lane = (int)(unit & 31), half = (int)((unit >> 5) & 1);
  const long long grp = unit >> 6;
  const int g = (int)(grp % p.G), nt = (int)(grp / p.G);
  const int r = lane >> 2, j = lane & 3;
  const int n = nt * 16 + half * 8 + r;
  const int k0 = g * 128 + j * 32;
  const float s = load_scale(p, (size_t)(k0 / p.group) * p.N + n);
  const uint32_t mask = (1u << p.nbits) - 1u;
  const uint32_t flip = p.kind == 1 ? (1u << (p.nbits - 1)) : 0u;  // offset binary for signed integers
  uint32_t words[8];
#pragma unroll
  for (int v = 0; v < 8; ++v) words[v] = 0u;
  const size_t base = (size_t)n * p.ldw + k0;
  for (int i = 0; i < 32; ++i) {
    float q = __fdiv_rn(load_w(p, base + i), s);
    q = fminf(fmaxf(q, p.minv), p.maxv);
    uint32_t code;
    if (p.kind == 2) code = encode_float_code(q, p.nbits, p.ebits, p.mbits);
    else code = ((uint32_t)(int)rintf(q)) & mask;
    code ^= flip;
    // spread the code over the unit's planes (widths = the set bits of nbits, widest first)
    const int h = i >> 1, odd = i & 1;
    int lo = p.nbits, wbase = 0;
    for (int pw = 8; pw >= 1; pw >>= 1) {
      if (!(p.nbits & pw)) continue;
      lo -= pw;
      const int per = 16 / pw;
      const uint32_t field = (code >> lo) & ((1u << pw) - 1u);
      words[wbase + h / per] |= field << ((h % per) * pw + 16 * odd);
      wbase += pw;
    }
  }
  uint32_t* dst = p.bq + (size_t)unit * p.nbits;
  for (int v = 0; v < p.nbits; ++v) dst[v] = words[v];
}

cudaError_t quantize_launch(const void* w, int w_dtype, int ldw, void* bq, void* scales, int N, int K, int group,
                            int kind, int nbits, int ebits, int mbits, float minv, float maxv, int act,
                            cudaStream_t stream) {
  QuantParams p;
  p.w = w; p.w_dtype = w_dtype; p.ldw = ldw;
  p.bq = reinterpret_cast<uint32_t*>(bq);
  p.scales = reinterpret_cast<unsigned short*>(scales);
  p.act = act;
  p.N = N; p.K = K; p.G = K / 128; p.group = group;
  p.kind = kind; p.nbits = nbits; p.ebits = ebits; p.mbits = mbits;
  p.minv = minv; p.maxv = maxv;
  const long long warps = (long long)N * (K / group);
  const long long blocks1 = (warps * 32 + 255) / 256;
  quant_scales_kernel<<<(unsigned)blocks1, 256, 0, stream>>>(p);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return e;
  const long long units = (long long)N * K / 32;
  quant_pack_kernel<<<(unsigned)((units + 127) / 128), 128, 0, stream>>>(p);
  return cudaGetLastError();
}

}  // namespace b200q
