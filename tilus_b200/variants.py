"""Kernel variants: which (weight dtype, zero point) pairs the CUDA kernels decode.

Mirrors the variant ids of csrc/decode.cuh.  Integer variant id = (b-1)*2 + biasmode
with biasmode 1 meaning "subtract 2^(b-1)"; signed types are stored in offset binary
and always use biasmode 1; unsigned types use biasmode 0 (zero point 0, the
reference's own behaviour) or biasmode 1 (symmetric zero point 2^(b-1)).
"""
from __future__ import annotations

from .dtypes import KIND_FLOAT, KIND_INT, KIND_UINT, WeightDType, weight_dtype

FLOAT_VARIANTS = {
    "float8_e5m2": 16, "float7_e4m2": 17, "float6_e3m2": 18, "float6_e2m3": 19,
    "float5_e3m1": 20, "float5_e2m2": 21, "float4_e2m1": 22, "float3_e1m1": 23,
}
VARIANT_COUNT = 24


def variant_id(dt, zero_point: int = 0) -> int:
    dt = weight_dtype(dt)
    if dt.kind == KIND_FLOAT:
        if zero_point != 0:
            raise ValueError("float weight types take no zero point")
        if dt.name not in FLOAT_VARIANTS:
            raise ValueError(f"no kernel variant for {dt.name}")
        return FLOAT_VARIANTS[dt.name]
    half = 1 << (dt.nbits - 1)
    if dt.kind == KIND_INT:
        if zero_point != 0:
            raise ValueError("signed integer weight types take no zero point")
        return (dt.nbits - 1) * 2 + 1
    assert dt.kind == KIND_UINT
    if zero_point == 0:
        return (dt.nbits - 1) * 2
    if zero_point == half:
        return (dt.nbits - 1) * 2 + 1
    raise ValueError(f"zero point of {dt.name} must be 0 or {half}, got {zero_point}")


def supported_weight_dtypes():
    from .dtypes import ALL_WEIGHT_DTYPES

    return [d for d in ALL_WEIGHT_DTYPES if d.kind != KIND_FLOAT or d.name in FLOAT_VARIANTS]
