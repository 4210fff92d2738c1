"""CPU oracle for the weight-only quantized matmul  C[M,N] = A[M,K] x dequant(Bq[K,N]).

TEST INFRASTRUCTURE ONLY.  This module is a plain numpy / torch-CPU restatement of
the reference's algorithm.  It is imported by tests/, by the smoke check and by the
CPU-baseline / reference legs of bench.py, always as the checker or the timed CPU
baseline, never by the product package: the product path is the CUDA library and
fails loudly without it.

Parity status: the sub-byte decode / encode arithmetic and the 16x16 weight-tile
permutation are PINNED against the reference's own known-answer functions and
layout algebra (fixtures under tests/golden/, produced by
tests/golden/make_golden.py by importing the reference on CPU).  The GEMM result
itself has no test or golden vector in the reference (its example only compares
with the unquantized product at atol=rtol=1e-2), so for the GEMM output this
oracle is the definition: dequantize, then fp32-accumulate matmul, then one
rounding to fp16.

Each function cites the reference lines it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

import numpy as np

KIND_UINT, KIND_INT, KIND_FLOAT = 0, 1, 2


# ---------------------------------------------------------------------------
# dtype description (duck-typed: anything with nbits/kind/exponent_nbits/mantissa_nbits)
# ---------------------------------------------------------------------------
def _desc(dt):
    return int(dt.nbits), int(dt.kind), int(dt.exponent_nbits), int(dt.mantissa_nbits)


# ---------------------------------------------------------------------------
# decode: code -> real value
# ---------------------------------------------------------------------------
def decode_table(dt) -> np.ndarray:
    """float64 value of every code 0 .. 2^nbits-1.

    ints  : python/tilus/hidet/transforms/lower_subbyte_type.py:670-677
            ((int32)(x << (32-b)) >> (32-b) for signed, x for unsigned).
    floats: python/tilus/hidet/ir/primitives/cuda/cast.py:103-118 (place sign and
            exponent|mantissa bits into an fp32 pattern, multiply by
            2^(128 - 2^(e-1)) without flushing subnormals): every exponent code is
            a finite binade, exponent code 0 is subnormal.
    """
    nbits, kind, e, m = _desc(dt)
    codes = np.arange(1 << nbits, dtype=np.int64)
    if kind == KIND_UINT:
        return codes.astype(np.float64)
    if kind == KIND_INT:
        return np.where(codes >= (1 << (nbits - 1)), codes - (1 << nbits), codes).astype(np.float64)
    sign = (codes >> (nbits - 1)) & 1
    em = codes & ((1 << (nbits - 1)) - 1)
    # fp32 pattern sign<<31 | em << (23-m), then * 2^(128 - 2^(e-1))
    bits = (sign.astype(np.uint64) << 31) | (em.astype(np.uint64) << (23 - m))
    f = bits.astype(np.uint32).view(np.float32).astype(np.float64)
    return f * 2.0 ** (128 - (1 << (e - 1)))


def decode_codes(codes: np.ndarray, dt) -> np.ndarray:
    """Elementwise decode of integer codes to float32 (exact for all <= 8-bit types)."""
    return decode_table(dt).astype(np.float32)[np.asarray(codes, dtype=np.int64)]


# ---------------------------------------------------------------------------
# encode: real value -> code
# ---------------------------------------------------------------------------
def encode_float_codes(x: np.ndarray, dt) -> np.ndarray:
    """fp32 -> sub-byte float code, python/tilus/hidet/ir/primitives/cuda/cast.py:44-100.

    Round to nearest even at the target's normal precision; overflow saturates to
    the largest-magnitude code with the sign kept; NaN/Inf map to all-ones; fp32
    subnormals flush to signed zero; results below the normal range are shifted
    (truncated) into the subnormal encoding exactly as the reference does.
    """
    nbits, kind, e, m = _desc(dt)
    assert kind == KIND_FLOAT
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.int64)
    sign = ((u >> 31) & 1) << (nbits - 1)
    exps = (u >> 23) & 0xFF
    mant = (u & 0x7FFFFF) | 0x800000
    shift = 23 - m
    round_bit = (mant >> (shift - 1)) & 1
    sticky = (mant & ((1 << (shift - 1)) - 1)) != 0
    lsb = (mant >> shift) & 1
    up = (round_bit != 0) & (sticky | (lsb != 0))
    mant = np.where(up, mant + (1 << shift), mant)
    carry = (mant & 0x01000000) != 0
    mant = np.where(carry, mant >> 1, mant)
    exp_value = exps - 127 + carry.astype(np.int64)
    mant = mant >> shift
    exp_value = exp_value + (1 << (e - 1)) - 1

    out = np.zeros_like(u)
    overflow = exp_value >= (1 << e)
    under = exp_value <= 0
    sub_ok = under & (exp_value >= 1 - m)
    normal = ~overflow & ~under
    sh = np.clip(1 - exp_value, 0, 31)
    out = np.where(normal, sign | (exp_value << m) | (mant ^ (1 << m)), out)
    out = np.where(sub_ok, sign | (mant >> sh), out)
    out = np.where(under & ~sub_ok, sign, out)
    out = np.where(overflow, sign | ((1 << (nbits - 1)) - 1), out)
    out = np.where(exps == 0, sign, out)
    out = np.where(exps == 0xFF, sign | ((1 << nbits) - 1), out)
    return (out & ((1 << nbits) - 1)).astype(np.uint8)


def encode_int_codes(x: np.ndarray, dt) -> np.ndarray:
    """Integer values (already rounded and clamped) -> b-bit codes: `& mask`
    (python/tilus/hidet/transforms/lower_subbyte_type.py:679-683)."""
    nbits = int(dt.nbits)
    return (np.asarray(x).astype(np.int64) & ((1 << nbits) - 1)).astype(np.uint8)


# ---------------------------------------------------------------------------
# canonical packed storage
# ---------------------------------------------------------------------------
def pack_canonical(codes: np.ndarray, nbits: int) -> np.ndarray:
    """Row-major bit-dense little-endian stream: element i occupies bits
    [i*b, (i+1)*b) of the byte stream, bit 0 = LSB of byte 0; elements may straddle
    bytes (python/tilus/tensor.py:112-115;
    python/tilus/hidet/ir/primitives/cuda/subbyte.py:36-52)."""
    flat = np.asarray(codes, dtype=np.uint8).reshape(-1)
    assert (flat.size * nbits) % 8 == 0
    bits = ((flat[:, None] >> np.arange(nbits, dtype=np.uint8)) & 1).astype(np.uint8).reshape(-1)
    return np.packbits(bits, bitorder="little")


def unpack_canonical(storage: np.ndarray, nbits: int, numel: int) -> np.ndarray:
    bits = np.unpackbits(np.asarray(storage, dtype=np.uint8).reshape(-1), bitorder="little")[: numel * nbits]
    bits = bits.reshape(numel, nbits).astype(np.uint16)
    return (bits << np.arange(nbits, dtype=np.uint16)).sum(axis=1).astype(np.uint8)


def pack_along_k(codes: np.ndarray, nbits: int) -> np.ndarray:
    """Alternative packing order named by some benchmark descriptions: consecutive
    K elements of one column share a byte.  Same byte count as pack_canonical."""
    return pack_canonical(np.ascontiguousarray(np.asarray(codes).T), nbits)


# ---------------------------------------------------------------------------
# the reference's tiled weight layout  uint8[K/16, N/16, 32*b]
# ---------------------------------------------------------------------------
def ref_tile_bit_map(nbits: int) -> np.ndarray:
    """[16,16,b] -> absolute bit index, within the tile's 32*b bytes, of every bit of
    every code of the 16x16 (k, n) weight tile
    (examples/quantization/matmul_a16wx.py:29-61, :64-98).

    tile_layout = local(1, 2) * mma.lb with lb = local(2,1).column_spatial(4,8).local(2,1)
    (python/tilus/ir/instructions/cuda/mma_dot.py:88-103): element (k, n) is held by
    lane t = (n%8)*4 + (k%8)//2 in slot e = (n//8)*4 + (k//8)*2 + (k%2); the lane's 8
    codes are bit-packed little-endian into b bytes; the byte view
    local(outer).spatial(32).local(inner) with inner = gcd(b, 16), outer = b/inner
    puts lane-local byte j = o*inner + i at tile byte o*32*inner + t*inner + i.
    """
    from math import gcd

    k = np.arange(16)[:, None, None]
    n = np.arange(16)[None, :, None]
    bit = np.arange(nbits)[None, None, :]
    lane = (n % 8) * 4 + (k % 8) // 2
    slot = (n // 8) * 4 + (k // 8) * 2 + (k % 2)
    inner = gcd(nbits, 16)
    lane_bit = slot * nbits + bit
    j = lane_bit // 8
    o, i = j // inner, j % inner
    return (o * 32 * inner + lane * inner + i) * 8 + lane_bit % 8


def pack_ref_tiled(codes: np.ndarray, nbits: int) -> np.ndarray:
    """codes[K,N] -> uint8[K/16 * N/16 * 32*b], the layout produced by the reference's
    QuantizedMatmulChangeLayout kernel (examples/quantization/matmul_a16wx.py:64-98)."""
    codes = np.asarray(codes, dtype=np.uint8)
    K, N = codes.shape
    assert K % 16 == 0 and N % 16 == 0
    tiles = codes.reshape(K // 16, 16, N // 16, 16).transpose(0, 2, 1, 3)  # [kt, nt, k, n]
    bmap = ref_tile_bit_map(nbits)  # [16,16,b]
    tile_bits = 32 * nbits * 8
    out_bits = np.zeros((K // 16, N // 16, tile_bits), dtype=np.uint8)
    src_bits = (tiles[..., None] >> np.arange(nbits, dtype=np.uint8)) & 1  # [kt,nt,16,16,b]
    out_bits[:, :, bmap.reshape(-1)] = src_bits.reshape(K // 16, N // 16, -1)
    return np.packbits(out_bits.reshape(-1), bitorder="little")


def unpack_ref_tiled(storage: np.ndarray, nbits: int, K: int, N: int) -> np.ndarray:
    """Inverse of pack_ref_tiled (the reference's QuantizedMatmulRestoreLayout,
    examples/quantization/matmul_a16wx.py:101-132)."""
    tile_bits = 32 * nbits * 8
    bits = np.unpackbits(np.asarray(storage, dtype=np.uint8).reshape(-1), bitorder="little")
    bits = bits.reshape(K // 16, N // 16, tile_bits)
    bmap = ref_tile_bit_map(nbits)
    src = bits[:, :, bmap.reshape(-1)].reshape(K // 16, N // 16, 16, 16, nbits).astype(np.uint16)
    tiles = (src << np.arange(nbits, dtype=np.uint16)).sum(axis=-1).astype(np.uint8)
    return np.ascontiguousarray(tiles.transpose(0, 2, 1, 3)).reshape(K, N)


# ---------------------------------------------------------------------------
# dequantize and GEMM
# ---------------------------------------------------------------------------
def dequantize(codes: np.ndarray, scales: np.ndarray, dt, group_size: int, zero_point: int = 0) -> np.ndarray:
    """W[k,n] = fp16_rn( fp16(decode(q[k,n]) - zp) * s[k // g, n] ).

    examples/quantization/matmul_a16wx.py:319-320 (b = cast(q) * scale) with the
    cast of python/tilus/backends/emitters/cast.py:101-121 (exact in fp16) and the
    product of python/tilus/backends/emitters/elementwise.py:35-53 (one fp16
    multiply, round to nearest).  The reference has no zero point; zp != 0 covers
    benchmark descriptions that use unsigned codes with w = (q - 2^(b-1)) * s, and
    decode(q) - zp is still exact in fp16, so there is still exactly one rounding.
    """
    codes = np.asarray(codes)
    K, N = codes.shape
    v = decode_codes(codes, dt) - np.float32(zero_point)
    v16 = v.astype(np.float16)
    assert np.array_equal(v16.astype(np.float32), v), "decoded value not exact in fp16"
    s = np.asarray(scales, dtype=np.float16)
    assert s.shape == (K // group_size, N)
    s_full = np.repeat(s, group_size, axis=0)
    # fp16 x fp16 is exact in fp32 (22-bit product), so this is a single rounding.
    return (v16.astype(np.float32) * s_full.astype(np.float32)).astype(np.float16)


def gemm_fp16(a: np.ndarray, w: np.ndarray) -> np.ndarray:
    """C = fp16_rn( sum_k fp32(A[m,k]) * fp32(W[k,n]) ), fp32 accumulation
    (examples/quantization/matmul_a16wx.py:321 self.dot into an fp32 accumulator,
    :366 cast to fp16)."""
    import torch

    at = torch.from_numpy(np.asarray(a, dtype=np.float16)).float()
    wt = torch.from_numpy(np.asarray(w, dtype=np.float16)).float()
    return (at @ wt).half().numpy()


def quantized_matmul(a, codes, scales, dt, group_size, zero_point=0) -> np.ndarray:
    return gemm_fp16(a, dequantize(codes, scales, dt, group_size, zero_point))


# ---------------------------------------------------------------------------
# bfloat16 activations (a_dtype = bfloat16, examples/quantization/matmul_a16wx.py:35-41, :418-419)
# numpy has no bfloat16: these take and return torch CPU tensors
# ---------------------------------------------------------------------------
def dequantize_bf16(codes: np.ndarray, scales, dt, group_size: int, zero_point: int = 0):
    """W[k,n] = bf16_rn( bf16(decode(q[k,n]) - zp) * s[k // g, n] ) as a torch.bfloat16 tensor.

    Same two steps as `dequantize` in the other activation dtype: the cast of the code to
    bfloat16 (exact: every value of an at-most-8-bit type has at most 8 significant bits) and
    one bfloat16 multiply, rounded to nearest even (the 16-bit product of two bfloat16 numbers
    is exact in fp32, so rounding that product once is the same thing)."""
    import torch

    codes = np.asarray(codes)
    K, N = codes.shape
    v = torch.from_numpy(decode_codes(codes, dt) - np.float32(zero_point))
    v16 = v.to(torch.bfloat16)
    assert torch.equal(v16.float(), v), "decoded value not exact in bfloat16"
    s = scales if isinstance(scales, torch.Tensor) else torch.from_numpy(np.asarray(scales))
    s = s.to(torch.bfloat16)
    assert tuple(s.shape) == (K // group_size, N)
    s_full = s.float().repeat_interleave(group_size, dim=0)
    return (v16.float() * s_full).to(torch.bfloat16)


def gemm_bf16(a, w):
    """C = bf16_rn( sum_k fp32(A[m,k]) * fp32(W[k,n]) ), fp32 accumulation; torch.bfloat16 in and out."""
    return (a.float() @ w.float()).to(a.dtype)


def quantized_matmul_bf16(a, codes, scales, dt, group_size, zero_point=0):
    return gemm_bf16(a, dequantize_bf16(codes, scales, dt, group_size, zero_point))


# ---------------------------------------------------------------------------
# weight quantization (QuantizedLinear.load_and_quantize)
# ---------------------------------------------------------------------------
def quantize_weight(weight: np.ndarray, dt, group_size: int, bf16_scales: bool = False):
    """weight[out, in] (any float) -> (codes[K=in, N=out] uint8, scales[K/g, N] fp16; with
    bf16_scales the scales are rounded to bfloat16 instead and returned as float32 values).

    examples/quantization/matmul_a16wx.py:470-528: transpose to [K, N] in fp32, view
    as [K/g, g, N], scales = max(absmax / max_value, 1e-6) cast to fp16, q = w / scales
    clamped to [min, max], rounded half-to-even for integer types (torch.round) or by
    the float encode for float types.
    """
    nbits, kind, e, m = _desc(dt)
    w = np.ascontiguousarray(np.asarray(weight, dtype=np.float32).T)  # [K, N]
    K, N = w.shape
    wg = w.reshape(K // group_size, group_size, N)
    absmax = np.abs(wg).max(axis=1, keepdims=True)
    scales = np.maximum(absmax / np.float32(dt.max_value), np.float32(1e-6))
    if bf16_scales:
        import torch

        scales = torch.from_numpy(scales).to(torch.bfloat16).float().numpy()
    else:
        scales = scales.astype(np.float16)
    q = wg / scales.astype(np.float32)
    q = np.clip(q, np.float32(dt.min_value), np.float32(dt.max_value))
    if kind == KIND_FLOAT:
        codes = encode_float_codes(q.astype(np.float32), dt)
    else:
        codes = encode_int_codes(np.rint(q), dt)
    return codes.reshape(K, N), scales.reshape(K // group_size, N)
