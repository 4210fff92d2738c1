"""Weight quantization: on the GPU through the library (quantize_and_pack), and on the host (PyTorch): the arithmetic of
QuantizedLinear.load_and_quantize (examples/quantization/matmul_a16wx.py:470-528 of the
reference) - per-group absmax scales, clamp, round - producing integer codes.

Float targets are encoded with the reference's fp32 -> sub-byte rule
(python/tilus/hidet/ir/primitives/cuda/cast.py:44-100): round to nearest even, saturate,
flush fp32 subnormals to signed zero.
"""
from __future__ import annotations

import torch

from .dtypes import KIND_FLOAT, WeightDType, weight_dtype


def encode_float(x: torch.Tensor, dt: WeightDType) -> torch.Tensor:
    """fp32 tensor -> uint8 codes of a sub-byte float type."""
    nbits, e, m = dt.nbits, dt.exponent_nbits, dt.mantissa_nbits
    u = x.contiguous().to(torch.float32).view(torch.int32).to(torch.int64) & 0xFFFFFFFF
    sign = ((u >> 31) & 1) << (nbits - 1)
    exps = (u >> 23) & 0xFF
    mant = (u & 0x7FFFFF) | 0x800000
    shift = 23 - m
    round_bit = (mant >> (shift - 1)) & 1
    sticky = (mant & ((1 << (shift - 1)) - 1)) != 0
    lsb = (mant >> shift) & 1
    up = (round_bit != 0) & (sticky | (lsb != 0))
    mant = torch.where(up, mant + (1 << shift), mant)
    carry = (mant & 0x01000000) != 0
    mant = torch.where(carry, mant >> 1, mant)
    exp_value = exps - 127 + carry.to(torch.int64)
    mant = mant >> shift
    exp_value = exp_value + (1 << (e - 1)) - 1
    overflow = exp_value >= (1 << e)
    under = exp_value <= 0
    sub_ok = under & (exp_value >= 1 - m)
    normal = ~overflow & ~under
    sh = torch.clamp(1 - exp_value, 0, 31)
    out = torch.zeros_like(u)
    out = torch.where(normal, sign | (exp_value << m) | (mant ^ (1 << m)), out)
    out = torch.where(sub_ok, sign | (mant >> sh), out)
    out = torch.where(under & ~sub_ok, sign, out)
    out = torch.where(overflow, sign | ((1 << (nbits - 1)) - 1), out)
    out = torch.where(exps == 0, sign, out)
    out = torch.where(exps == 0xFF, sign | ((1 << nbits) - 1), out)
    return (out & ((1 << nbits) - 1)).to(torch.uint8)


def quantize_weight(weight: torch.Tensor, w_dtype, group_size: int, x_dtype: torch.dtype = torch.float16):
    """weight[out, in] -> (codes uint8[K=in, N=out], scales x_dtype[K/group, N]).

    Symmetric: scales = max(absmax / max_value, 1e-6) per (group, column), cast to the activation dtype;
    q = clamp(w / scales, min, max); integers round half to even (torch.round), floats
    are rounded by the encode.
    """
    dt = weight_dtype(w_dtype)
    out_f, in_f = weight.shape
    w = weight.float().transpose(1, 0).contiguous().view(in_f // group_size, group_size, out_f)
    absmax = w.abs().max(dim=1, keepdim=True)[0]
    scales = torch.max(absmax / float(dt.max_value), torch.tensor(1e-6, dtype=w.dtype, device=w.device))
    scales = scales.to(x_dtype)
    q = torch.clamp(w / scales, float(dt.min_value), float(dt.max_value))
    if dt.kind == KIND_FLOAT:
        codes = encode_float(q, dt)
    else:
        codes = (torch.round(q).to(torch.int64) & ((1 << dt.nbits) - 1)).to(torch.uint8)
    return codes.view(in_f, out_f), scales.view(in_f // group_size, out_f)


def quantize_and_pack(weight: torch.Tensor, w_dtype, group_size: int, x_dtype: torch.dtype = torch.float16):
    """weight[out, in] on a CUDA device (fp16, bf16 or fp32) -> (packed b200 bytes uint8[K*N*b/8],
    scales x_dtype[K/group, N]) in one library call (two kernels): the same arithmetic as
    quantize_weight followed by packing.interleave, bit for bit."""
    from . import _lib
    from .ops import act_code

    dt = weight_dtype(w_dtype)
    if not weight.is_cuda:
        raise ValueError("quantize_and_pack needs a CUDA tensor (use quantize_weight + packing.interleave on the host)")
    if weight.dtype not in (torch.float16, torch.float32, torch.bfloat16):
        weight = weight.float()
    wcode = {torch.float16: 0, torch.float32: 1, torch.bfloat16: 2}[weight.dtype]
    weight = weight.contiguous()
    out_f, in_f = weight.shape
    bq = torch.empty(in_f * out_f * dt.nbits // 8, dtype=torch.uint8, device=weight.device)
    scales = torch.empty(in_f // group_size, out_f, dtype=x_dtype, device=weight.device)
    with torch.cuda.device(weight.device):
        st = _lib.load().b200q_quantize(weight.data_ptr(), wcode, in_f,
                                        bq.data_ptr(), scales.data_ptr(), out_f, in_f, dt.code, group_size,
                                        act_code(x_dtype), torch.cuda.current_stream(weight.device).cuda_stream)
    _lib.check(st)
    return bq, scales
