// Unit decode: 32 packed b-bit codes of one weight column -> 16 half2 values.
//
// A "unit" is the 32 codes q[k0 .. k0+31, n] of one column, stored in b 32-bit words
// split into bit planes of width 8/4/2/1 (most significant plane first; 3 = 2+1,
// 5 = 4+1, 6 = 4+2, 7 = 4+2+1).  A plane of width p takes p words; pair h = 0..15
// (codes k0+2h, k0+2h+1) is field f = h % (16/p) of plane word h / (16/p): the even-k
// code in bits [f*p, f*p+p), the odd-k code in bits [16+f*p, 16+f*p+p).  One mask thus
// isolates a k-adjacent pair as the two halves of a 32-bit register.
//
// Integer types: the pair is OR-ed into the mantissa of the fp16 constant 1024 at bit
// position T (0x6400 | q << T = 1024 + q * 2^T) and one fma(x, 2^-T, -(2^(10-T) + bias))
// yields q - bias exactly.  Signed types are stored with the sign bit flipped (offset
// binary), so bias = 2^(b-1) decodes two's complement, and the same bias on an unsigned
// type is the symmetric zero point.  The arithmetic restates the reference's cast
// (python/tilus/backends/emitters/cast.py:174-348: OR with 0x64006400, subtract the
// magic, fma by 1/16 for the high nibble) for every width, and its result is the same
// exact fp16 value.
//
// Float types (sign / e exponent bits / m mantissa bits, bias 2^(e-1)-1, every exponent
// code finite for e < 5): the code is placed with its mantissa ending at fp16 mantissa
// bit 9 and its exponent starting at bit 10, the sign is moved to bit 15, and one exact
// multiply by 2^(15 - bias) rebases the exponent; fp16 subnormal arithmetic makes this
// exact for the source subnormals too.  Same values as
// python/tilus/hidet/ir/primitives/cuda/cast.py:103-118.
//
// The bit gathering (gather_pair) is plain integer C++ so that it also compiles for the
// host, where a test checks it against the packer for every width and variant.
#pragma once
#include <stdint.h>

#if defined(__CUDACC__)
#define B200Q_HD __host__ __device__ __forceinline__
#else
#define B200Q_HD inline
#endif

namespace b200q {

// ---- weight type variants ------------------------------------------------------------
// 0..15  : integer, id = (b-1)*2 + biasmode; biasmode 0: value = code,
//          biasmode 1: value = code - 2^(b-1)
// 16..23 : float types below
enum : int {
  VAR_F8E5M2 = 16, VAR_F7E4M2, VAR_F6E3M2, VAR_F6E2M3, VAR_F5E3M1, VAR_F5E2M2, VAR_F4E2M1, VAR_F3E1M1,
  VAR_COUNT
};

B200Q_HD constexpr bool var_is_float(int v) { return v >= 16; }
B200Q_HD constexpr int var_float_bits(int v) {
  return v == VAR_F8E5M2 ? 8 : v == VAR_F7E4M2 ? 7 : (v == VAR_F6E3M2 || v == VAR_F6E2M3) ? 6
       : (v == VAR_F5E3M1 || v == VAR_F5E2M2) ? 5 : v == VAR_F4E2M1 ? 4 : 3;
}
B200Q_HD constexpr int var_float_ebits(int v) {
  return v == VAR_F8E5M2 ? 5 : v == VAR_F7E4M2 ? 4 : (v == VAR_F6E3M2 || v == VAR_F5E3M1) ? 3
       : (v == VAR_F6E2M3 || v == VAR_F5E2M2 || v == VAR_F4E2M1) ? 2 : 1;
}
B200Q_HD constexpr int var_bits(int v) { return var_is_float(v) ? var_float_bits(v) : (v >> 1) + 1; }
B200Q_HD constexpr int var_bias(int v) { return (!var_is_float(v) && (v & 1)) ? (1 << (var_bits(v) - 1)) : 0; }

// ---- plane structure -------------------------------------------------------------------
B200Q_HD constexpr int plane_count(int b) {
  int c = 0;
  for (int p = 8; p >= 1; p >>= 1) if (b & p) ++c;
  return c;
}
// width of plane i (most significant first)
B200Q_HD constexpr int plane_width(int b, int i) {
  int idx = 0;
  for (int p = 8; p >= 1; p >>= 1) {
    if (b & p) { if (idx == i) return p; ++idx; }
  }
  return 0;
}
// lowest code bit covered by plane i
B200Q_HD constexpr int plane_lo(int b, int i) {
  int lo = b;
  for (int j = 0; j <= i; ++j) lo -= plane_width(b, j);
  return lo;
}
// first word of plane i inside the unit
B200Q_HD constexpr int plane_word_base(int b, int i) {
  int w = 0;
  for (int j = 0; j < i; ++j) w += plane_width(b, j);
  return w;
}

// Mantissa bit position T at which pair H of a b-bit integer type is assembled.
B200Q_HD constexpr int int_target(int b, int h) {
  const int p0 = plane_width(b, 0);
  const int q0 = (h % (16 / p0)) * p0;
  const int lo0 = plane_lo(b, 0);
  const int t0 = q0 - lo0;             // top plane would need no shift
  if (t0 >= 0 && t0 + b <= 10) return t0;
  if (t0 - 8 >= 0 && t0 - 8 + b <= 10) return t0 - 8;   // one shared shift by 8
  if (t0 < 0) return 0;
  return 10 - b;
}

template <int B, int H, int T, int I>
struct GatherPlanes {
  static B200Q_HD uint32_t run(const uint32_t* w, uint32_t acc) {
    constexpr int p = plane_width(B, I);
    constexpr int per = 16 / p;
    constexpr int word = plane_word_base(B, I) + H / per;
    constexpr int q = (H % per) * p;
    constexpr int dst = T + plane_lo(B, I);
    constexpr int s = q - dst;
    constexpr uint32_t mask = (((1u << p) - 1u) << dst) * 0x00010001u;
    uint32_t x = w[word];
    uint32_t xs = s > 0 ? (x >> (s > 0 ? s : 0)) : (s < 0 ? (x << (s < 0 ? -s : 0)) : x);
    acc |= xs & mask;
    if constexpr (I + 1 < plane_count(B)) return GatherPlanes<B, H, T, I + 1>::run(w, acc);
    else return acc;
  }
};

// Both codes of pair H, each shifted to bit T of its 16-bit half, OR-ed onto `base`.
template <int B, int H, int T>
B200Q_HD uint32_t gather_pair(const uint32_t* w, uint32_t base) {
  return GatherPlanes<B, H, T, 0>::run(w, base);
}

// fp16 bit pattern of a non-negative integer < 2048 (exactly representable)
B200Q_HD constexpr uint32_t half_bits_of_uint(uint32_t v) {
  if (v == 0) return 0;
  int e = 0;
  while ((2u << e) <= v) ++e;
  return ((uint32_t)(15 + e) << 10) | ((v - (1u << e)) << (10 - e));
}
B200Q_HD constexpr uint32_t dup16(uint32_t h) { return h | (h << 16); }

// raw pattern of pair H for variant VAR, before the fp16 arithmetic (see unit_decode)
template <int VAR, int H>
B200Q_HD uint32_t pair_raw(const uint32_t* w) {
  constexpr int B = var_bits(VAR);
  if constexpr (!var_is_float(VAR)) {
    constexpr int T = int_target(B, H);
    return gather_pair<B, H, T>(w, 0x64006400u);
  } else {
    constexpr int E = var_float_ebits(VAR);
    constexpr int M = B - 1 - E;
    constexpr int T = 10 - M;
    uint32_t r = gather_pair<B, H, T>(w, 0u);
    if constexpr (E < 5) {
      constexpr uint32_t mag = (((1u << (B - 1)) - 1u) << T) * 0x00010001u;
      r = (r & mag) | ((r << (5 - E)) & 0x80008000u);
    }
    return r;
  }
}

// "Linear" pattern of pair H: a half2 bit pattern whose fp16 value is proportional to the
// decoded value, with no arithmetic at all.  Integers: the code sits in the mantissa of an
// fp16 subnormal at bit T, value = code * 2^(T-24).  Floats: pair_raw, value = true value *
// 2^-(15 - bias).  The GEMV path feeds these straight to the tensor core and repairs the
// factors afterwards (activations pre-multiplied by 2^-T, accumulators by lin_factor).
template <int VAR, int H>
B200Q_HD uint32_t pair_lin(const uint32_t* w) {
  constexpr int B = var_bits(VAR);
  if constexpr (!var_is_float(VAR)) {
    constexpr int T = int_target(B, H);
    return gather_pair<B, H, T>(w, 0u);
  } else {
    return pair_raw<VAR, H>(w);
  }
}

// exponent e such that activations of pair h are pre-multiplied by 2^-e
B200Q_HD constexpr int lin_prescale_shift(int var, int h) {
  return var_is_float(var) ? 0 : int_target(var_bits(var), h);
}
// log2 of the factor the accumulated linear products are multiplied by
B200Q_HD constexpr int lin_factor_log2(int var) {
  return var_is_float(var) ? 15 - ((1 << (var_float_ebits(var) - 1)) - 1) : 24;
}

template <int VAR, int H>
B200Q_HD constexpr int pair_target() {
  constexpr int B = var_bits(VAR);
  if constexpr (!var_is_float(VAR)) return int_target(B, H);
  else return 10 - (B - 1 - var_float_ebits(VAR));
}

}  // namespace b200q

#if defined(__CUDACC__)
#include <cuda_bf16.h>
#include <cuda_fp16.h>
namespace b200q {

__device__ __forceinline__ __half2 h2_from_bits(uint32_t x) {
  return *reinterpret_cast<__half2*>(&x);
}
__device__ __forceinline__ uint32_t bits_from_h2(__half2 x) {
  return *reinterpret_cast<uint32_t*>(&x);
}

// exact value (code - bias, or the float value) of pair H as half2
template <int VAR, int H>
__device__ __forceinline__ __half2 pair_value(const uint32_t* w) {
  constexpr int B = var_bits(VAR);
  const uint32_t raw = pair_raw<VAR, H>(w);
  if constexpr (!var_is_float(VAR)) {
    constexpr int T = int_target(B, H);
    constexpr uint32_t mul = dup16((uint32_t)(15 - T) << 10);                                  // 2^-T
    constexpr uint32_t add = dup16(0x8000u | half_bits_of_uint((1u << (10 - T)) + var_bias(VAR)));  // -(2^(10-T)+bias)
    return __hfma2(h2_from_bits(raw), h2_from_bits(mul), h2_from_bits(add));
  } else {
    constexpr int E = var_float_ebits(VAR);
    if constexpr (E == 5) return h2_from_bits(raw);
    constexpr int ebias = (1 << (E - 1)) - 1;
    constexpr uint32_t mul = dup16((uint32_t)(30 - ebias) << 10);  // 2^(15 - ebias)
    return __hmul2(h2_from_bits(raw), h2_from_bits(mul));
  }
}

// pair H times the scale, in the arithmetic of the activation dtype.  ACT 0: one fp16 multiply,
// fp16_rn(value * s).  ACT 1: the value (at most 8 significant bits, so exact in bf16) is
// converted fp16 -> fp32 -> bf16 without rounding and multiplied once in bf16, bf16_rn(value * s):
// the reference's cast to the activation dtype followed by its elementwise multiply
// (examples/quantization/matmul_a16wx.py:316-320).  `scale2` holds the 16-bit scale in both halves.
template <int VAR, int H, int ACT>
__device__ __forceinline__ uint32_t pair_scaled(const uint32_t* w, uint32_t scale2) {
  const __half2 v = pair_value<VAR, H>(w);
  if constexpr (ACT == 0) {
    return bits_from_h2(__hmul2(v, h2_from_bits(scale2)));
  } else {
    const float2 f = __half22float2(v);
    const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
    const __nv_bfloat162 r = __hmul2(b, *reinterpret_cast<const __nv_bfloat162*>(&scale2));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
}

template <int VAR, int H, int ACT>
struct UnitLoop {
  static __device__ __forceinline__ void run(const uint32_t* w, uint32_t scale2, uint32_t* out) {
    out[H] = pair_scaled<VAR, H, ACT>(w, scale2);
    if constexpr (H + 1 < 16) UnitLoop<VAR, H + 1, ACT>::run(w, scale2, out);
  }
};

template <int VAR, int H>
struct UnitLinLoop {
  static __device__ __forceinline__ void run(const uint32_t* w, uint32_t* out) {
    out[H] = pair_lin<VAR, H>(w);
    if constexpr (H + 1 < 16) UnitLinLoop<VAR, H + 1>::run(w, out);
  }
};
// out[h] = linear patterns of pair h (see pair_lin)
template <int VAR>
__device__ __forceinline__ void unit_decode_linear(const uint32_t* w, uint32_t* out) {
  UnitLinLoop<VAR, 0>::run(w, out);
}

// out[h] = rn(value(k0+2h) * s) | rn(value(k0+2h+1) * s) << 16, h = 0..15, in fp16 (ACT 0) or bf16 (ACT 1);
// scale2 = the 16-bit scale pattern in both halves
template <int VAR, int ACT = 0>
__device__ __forceinline__ void unit_decode_scaled(const uint32_t* w, uint32_t scale2, uint32_t* out) {
  UnitLoop<VAR, 0, ACT>::run(w, scale2, out);
}

}  // namespace b200q
#endif
