"""Seeded synthetic problems in the shapes and value distributions of the benchmark
configurations: activations fp16 ~ N(0,1), codes uniform over the type's codes (all
non-NaN patterns), fp16 scales uniform in a range, one per (group, column)."""
from __future__ import annotations

import torch

from .dtypes import KIND_UINT, weight_dtype


def make_problem(M: int, N: int, K: int, w_dtype, group_size: int, seed: int = 0, scale_range=(0.005, 0.02),
                 symmetric_unsigned: bool = True):
    """Returns dict(a fp16[M,K], codes uint8[K,N], scales fp16[K/g,N], zero_point) on CPU."""
    dt = weight_dtype(w_dtype)
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g, dtype=torch.float32).to(torch.float16)
    codes = torch.randint(0, 1 << dt.nbits, (K, N), generator=g, dtype=torch.int32).to(torch.uint8)
    if dt.is_float() and dt.exponent_nbits == 5:
        # keep to finite, in-range patterns: clear the all-ones exponent
        top = ((1 << dt.exponent_nbits) - 1) << dt.mantissa_nbits
        codes = torch.where((codes & top) == top, codes & ~(1 << dt.mantissa_nbits) & 0xFF, codes)
    lo, hi = scale_range
    scales = (torch.rand(K // group_size, N, generator=g, dtype=torch.float32) * (hi - lo) + lo).to(torch.float16)
    zp = (1 << (dt.nbits - 1)) if (dt.kind == KIND_UINT and symmetric_unsigned) else 0
    return dict(a=a, codes=codes, scales=scales, zero_point=zp, dtype=dt, group_size=group_size)


def gemm_bytes(M: int, N: int, K: int, nbits: int, group_size: int) -> int:
    """Algorithmic bytes of one GEMM: packed weights + scales + activations + output."""
    return K * N * nbits // 8 + (K // group_size) * N * 2 + M * K * 2 + M * N * 2


def gemm_flops(M: int, N: int, K: int) -> int:
    return 2 * M * N * K
